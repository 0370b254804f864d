// Sharded optimizer step fused with its collectives over NVLink peer memory.
//
// Every rank holds, in peer-mapped device memory, the full bf16 gradient buffer it
// produced (flat_g) and the full bf16 weight buffer it computes with (flat_w).  Rank r
// owns elements [r*S, (r+1)*S) of both ("its shard") plus fp32 master weights and AdamW
// moments for that shard.  One optimizer step is two kernels, with no NCCL call:
//
//   kernel A  reduce-scatter + norm: after a cross-rank "gradients ready" barrier, read
//             the shard range of flat_g from every peer with plain loads through the
//             peer mapping, sum in fp32 in rank order (bitwise identical on reruns),
//             keep the fp32 sum in a local scratch shard, reduce the sum of squares and
//             push it into slot r of every peer's norm table;
//   kernel B  AdamW + all-gather: wait for all norm slots, form the global clip
//             coefficient (every rank adds the slots in the same order), update master /
//             moments for the shard and store the refreshed bf16 weights straight into
//             the shard range of every peer's flat_w; a closing cross-rank barrier makes
//             sure nobody runs ahead while a peer still writes its weights or reads its
//             gradients.
//
// When the gradient and weight buffers are also mapped through an NVLink multicast object
// (NVSwitch), the two bulk transfers go through the switch instead of through per-peer
// loads and stores: kernel A reads its shard with multimem.ld_reduce (the switch adds the
// ranks' copies, fp32 accumulation, one bf16 rounding) and kernel B writes it with
// multimem.st (the switch replicates the store to every rank), so a rank moves 1/world of
// the buffer per direction instead of (world-1)/world.
//
// Barriers are generation counters in peer memory (release store / acquire load at
// system scope).  The generation is a device-side step counter, so a captured CUDA
// graph can be replayed.  Every wait is bounded; on expiry a status word is set, the
// kernel finishes without touching peers further, and the host raises.
#include "common.cuh"

namespace sb200 {
namespace fo {

constexpr int kMaxRanks = 8;
constexpr int kThreads = 256;
constexpr int kBlocks = 2 * kNumSM;
constexpr uint32_t kSpinsPerSecond = 1u << 24;  // one poll + 64 ns back-off: about 60 ns
// The wait budget (poll iterations) is a kernel argument: the host passes tens of seconds by
// default, since the collectives this replaces tolerate long rank skew; it stays bounded.

enum Status : int { kOk = 0, kTimeoutGradBarrier = 11, kTimeoutNormBarrier = 12, kTimeoutEndBarrier = 13, kTimeoutLocal = 14 };

// Layout of the per-rank control block (uint32 words) in peer memory:
//   [0, 8)   flag A: "rank p's gradients are ready"    (written by p)
//   [8, 16)  flag B: "rank p's norm slot is written"   (written by p)
//   [16, 24) flag C: "rank p finished the step"        (written by p)
//   [24, 32) norm slots (fp32 bit patterns)            (slot p written by p)
//   [32]     local release word A   [33] local release word B   [34] step counter
//   [35]     block ticket A         [36] block ticket B         [37] local norm_sq (fp32)
constexpr int kCtlWords = 64;

struct Params {
  int world, rank;
  int64_t shard;  // elements per rank (multiple of 8)
  const __nv_bfloat16* g[kMaxRanks];
  __nv_bfloat16* w[kMaxRanks];
  const __nv_bfloat16* g_mc;  // multicast mapping of the gradient buffers (nullptr: per-peer loads)
  __nv_bfloat16* w_mc;        // multicast mapping of the weight buffers (nullptr: per-peer stores)
  uint32_t* ctl[kMaxRanks];
  float* master;
  float* m;
  float* v;
  float* gred;     // fp32 reduced gradient shard (local scratch)
  float* partial;  // [kBlocks] local scratch
  const float* hyper;
  int* status;
  uint32_t spin_limit;  // poll iterations every wait may use
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Sum of the eight bf16 at the same offset of every rank's buffer, added in the switch.
__device__ __forceinline__ bf16x8 multimem_ld_reduce8(const __nv_bfloat16* mc_ptr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc_ptr)
               : "memory");
  return *reinterpret_cast<bf16x8*>(&v);
}
// Store sixteen bytes to the same offset of every rank's buffer.
__device__ __forceinline__ void multimem_st8(__nv_bfloat16* mc_ptr, const bf16x8& val) {
  const uint4 v = *reinterpret_cast<const uint4*>(&val);
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc_ptr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Bounded wait until *p == want (acquire at the given scope).
template <bool SYS>
__device__ __forceinline__ bool wait_eq(const uint32_t* p, uint32_t want, int* status, int code, uint32_t spin_limit) {
  for (uint32_t i = 0; i < spin_limit; ++i) {
    const uint32_t v = SYS ? ld_acquire_sys(p) : ld_acquire_gpu(p);
    if (v == want) return true;
    if ((i & 0x3ff) == 0x3ff && *reinterpret_cast<volatile int*>(status) != kOk) return false;
    __nanosleep(64);
  }
  atomicCAS(status, kOk, code);
  return false;
}

// Block 0 runs `leader` (cross-rank part) and publishes `gen` in the local release word;
// every other block waits for that word.  Returns false if anything timed out.
template <typename F>
__device__ __forceinline__ bool leader_then_release(uint32_t* release_word, uint32_t gen, int* status, uint32_t spin_limit, F leader) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    bool ok = true;
    if (blockIdx.x == 0) {
      ok = leader();
      // publish even on failure (with a poisoned value) so the other blocks do not wait out their budget
      st_release_gpu(release_word, ok ? gen : 0xffffffffu);
    } else {
      // the leader's own waits use the same budget one after another (up to `world` of them)
      const uint64_t local_limit = (uint64_t)spin_limit * (kMaxRanks + 1);
      for (uint64_t i = 0; i < local_limit; ++i) {
        const uint32_t v = ld_acquire_gpu(release_word);
        if (v == gen) break;
        if (v == 0xffffffffu || (((i & 0x3ff) == 0x3ff) && *reinterpret_cast<volatile int*>(status) != kOk)) { ok = false; break; }
        if (i + 1 == local_limit) { atomicCAS(status, kOk, kTimeoutLocal); ok = false; }
        __nanosleep(64);
      }
    }
    ok_s = ok;
  }
  __syncthreads();
  return ok_s != 0;
}

__global__ void __launch_bounds__(kThreads)
reduce_scatter_norm_kernel(const Params p) {
  __shared__ float scratch[33];
  uint32_t* ctl = p.ctl[p.rank];
  const uint32_t gen = ctl[34] + 1;  // step counter is advanced at the end of kernel B

  const bool ok = leader_then_release(ctl + 32, gen, p.status, p.spin_limit, [&]() {
    __threadfence_system();
    for (int q = 0; q < p.world; ++q) st_release_sys(p.ctl[q] + 0 + p.rank, gen);
    for (int q = 0; q < p.world; ++q)
      if (!wait_eq<true>(ctl + 0 + q, gen, p.status, kTimeoutGradBarrier, p.spin_limit)) return false;
    return true;
  });

  float acc = 0.f;
  if (ok) {
    const int64_t base = (int64_t)p.rank * p.shard;
    const int64_t nvec = p.shard >> 3;
    for (int64_t vi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; vi < nvec; vi += (int64_t)gridDim.x * blockDim.x) {
      float sum[8];
      if (p.g_mc != nullptr) {
        unpack8(multimem_ld_reduce8(p.g_mc + base + (vi << 3)), sum);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] = 0.f;
        for (int q = 0; q < p.world; ++q) {  // fixed order: deterministic sum
          float f[8];
          unpack8(ld8(p.g[q] + base + (vi << 3)), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) sum[j] += f[j];
        }
      }
      float4* dst = reinterpret_cast<float4*>(p.gred + (vi << 3));
      dst[0] = make_float4(sum[0], sum[1], sum[2], sum[3]);
      dst[1] = make_float4(sum[4], sum[5], sum[6], sum[7]);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += sum[j] * sum[j];
    }
  }
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) {
    p.partial[blockIdx.x] = acc;
    __threadfence();
    const uint32_t ticket = atomicAdd(ctl + 35, 1u);
    if (ticket == gridDim.x - 1) {  // last block: fixed-order final sum, then publish to every peer
      __threadfence();
      float total = 0.f;
      for (int b = 0; b < (int)gridDim.x; ++b) total += reinterpret_cast<volatile float*>(p.partial)[b];
      ctl[35] = 0;
      if (ok) {
        for (int q = 0; q < p.world; ++q) reinterpret_cast<volatile uint32_t*>(p.ctl[q] + 24)[p.rank] = __float_as_uint(total);
        __threadfence_system();
        for (int q = 0; q < p.world; ++q) st_release_sys(p.ctl[q] + 8 + p.rank, gen);
      }
    }
  }
}

__global__ void __launch_bounds__(kThreads)
adamw_all_gather_kernel(const Params p) {
  uint32_t* ctl = p.ctl[p.rank];
  const uint32_t gen = ctl[34] + 1;

  const bool ok = leader_then_release(ctl + 33, gen, p.status, p.spin_limit, [&]() {
    for (int q = 0; q < p.world; ++q)
      if (!wait_eq<true>(ctl + 8 + q, gen, p.status, kTimeoutNormBarrier, p.spin_limit)) return false;
    float total = 0.f;
    for (int q = 0; q < p.world; ++q) total += __uint_as_float(reinterpret_cast<volatile uint32_t*>(ctl + 24)[q]);
    reinterpret_cast<volatile uint32_t*>(ctl)[37] = __float_as_uint(total);
    __threadfence();
    return true;
  });

  if (ok) {
    const float norm_sq = __uint_as_float(reinterpret_cast<volatile uint32_t*>(ctl)[37]);
    const float lr = p.hyper[0], b1 = p.hyper[1], b2 = p.hyper[2], eps = p.hyper[3], wd = p.hyper[4];
    const float bc1 = p.hyper[5], bc2 = p.hyper[6], max_norm = p.hyper[7];
    float gscale = p.hyper[8];
    if (max_norm > 0.f) {
      const float coef = max_norm / (gscale * sqrtf(norm_sq) + 1e-6f);
      if (coef < 1.f) gscale *= coef;
    }
    const float step_size = lr / bc1, inv_sqrt_bc2 = rsqrtf(bc2);
    const int64_t base = (int64_t)p.rank * p.shard;
    const int64_t nvec = p.shard >> 3;
    for (int64_t vi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; vi < nvec; vi += (int64_t)gridDim.x * blockDim.x) {
      const int64_t i0 = vi << 3;
      float out[8];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float4 g4 = reinterpret_cast<const float4*>(p.gred + i0)[h];
        float4 w4 = reinterpret_cast<float4*>(p.master + i0)[h];
        float4 m4 = reinterpret_cast<float4*>(p.m + i0)[h];
        float4 v4 = reinterpret_cast<float4*>(p.v + i0)[h];
        const float g[4] = {g4.x * gscale, g4.y * gscale, g4.z * gscale, g4.w * gscale};
        float w[4] = {w4.x, w4.y, w4.z, w4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          w[j] *= (1.f - lr * wd);
          mm[j] = b1 * mm[j] + (1.f - b1) * g[j];
          vv[j] = b2 * vv[j] + (1.f - b2) * g[j] * g[j];
          w[j] -= step_size * (mm[j] / (sqrtf(vv[j]) * inv_sqrt_bc2 + eps));
          out[h * 4 + j] = w[j];
        }
        reinterpret_cast<float4*>(p.master + i0)[h] = make_float4(w[0], w[1], w[2], w[3]);
        reinterpret_cast<float4*>(p.m + i0)[h] = make_float4(mm[0], mm[1], mm[2], mm[3]);
        reinterpret_cast<float4*>(p.v + i0)[h] = make_float4(vv[0], vv[1], vv[2], vv[3]);
      }
      const bf16x8 packed = pack8(out);
      if (p.w_mc != nullptr) {
        multimem_st8(p.w_mc + base + i0, packed);  // all-gather by one store, replicated in the switch
      } else {
        for (int q = 0; q < p.world; ++q) st8(p.w[q] + base + i0, packed);  // all-gather by push
      }
    }
  }
  // closing barrier: the last block of this rank signals every peer and waits for all of them
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t ticket = atomicAdd(ctl + 36, 1u);
    if (ticket == gridDim.x - 1) {
      ctl[36] = 0;
      if (ok) {
        for (int q = 0; q < p.world; ++q) st_release_sys(p.ctl[q] + 16 + p.rank, gen);
        for (int q = 0; q < p.world; ++q)
          if (!wait_eq<true>(ctl + 16 + q, gen, p.status, kTimeoutEndBarrier, p.spin_limit)) break;
      }
      ctl[34] = gen;  // advance the step counter (also after a failure, so a retry starts a fresh generation)
      __threadfence();
    }
  }
}

}  // namespace fo

int fused_optim_ctl_words() { return fo::kCtlWords; }
int fused_optim_num_partials() { return fo::kBlocks; }

// Pointers are device addresses valid on the calling rank (peer-mapped for q != rank).
// g_mc / w_mc: multicast addresses of the gradient / weight buffers, or nullptr for per-peer access.
int launch_fused_sharded_adamw(int world, int rank, int64_t shard, const void* const* g_peers, void* const* w_peers,
                               void* const* ctl_peers, const void* g_mc, void* w_mc, float* master, float* m, float* v, float* gred,
                               float* partial, const float* hyper, int* status, uint32_t spin_limit, cudaStream_t stream) {
  if (world < 1 || world > fo::kMaxRanks || rank < 0 || rank >= world || shard <= 0 || (shard & 7)) return -1;
  fo::Params p{};
  p.world = world;
  p.rank = rank;
  p.shard = shard;
  for (int q = 0; q < world; ++q) {
    p.g[q] = static_cast<const __nv_bfloat16*>(g_peers[q]);
    p.w[q] = static_cast<__nv_bfloat16*>(w_peers[q]);
    p.ctl[q] = static_cast<uint32_t*>(ctl_peers[q]);
  }
  p.g_mc = static_cast<const __nv_bfloat16*>(g_mc);
  p.w_mc = static_cast<__nv_bfloat16*>(w_mc);
  p.master = master;
  p.m = m;
  p.v = v;
  p.gred = gred;
  p.partial = partial;
  p.hyper = hyper;
  p.status = status;
  p.spin_limit = spin_limit ? spin_limit : fo::kSpinsPerSecond;
  count_launch(2);
  fo::reduce_scatter_norm_kernel<<<fo::kBlocks, fo::kThreads, 0, stream>>>(p);
  fo::adamw_all_gather_kernel<<<fo::kBlocks, fo::kThreads, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace sb200
