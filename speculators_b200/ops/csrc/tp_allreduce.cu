// Second half of the row-parallel product of a tensor-parallel layer (first half: the GEMM whose
// epilogue stores every tile into its owner's staging area, gemm_tcgen05.cu `Scatter`).
//
//   opening barrier   every rank's GEMM has finished, so its stores into this rank's staging area
//                     have landed (flag per rank, release / acquire at system scope)
//   reduce            this rank adds the `world` staged partial slices of the columns it owns in
//                     fp32 (fixed order: the result does not depend on timing), adds the residual
//                     stream's slice when one is given, rounds once to bf16
//   all-gather        and stores the slice into every rank's output: one multimem.st per 16 bytes
//                     when the outputs are bound to an NVLink multicast object (the switch
//                     replicates the store), else one store per peer
//   closing barrier   every rank has written its slice everywhere; when the kernel ends the
//                     whole [rows, N] output is complete on this device and the staging area may
//                     be written again
//
// so the layer's "GEMM -> all-reduce -> residual add" is two launches with the reduce-scatter's
// transfer hidden under the GEMM's tiles.  Barriers are generation counters kept on the device
// (graph replay safe); every wait is bounded and reports through a status word.
#include "common.cuh"

namespace sb200 {
namespace tpar {

constexpr int kMaxRanks = 8;
constexpr int kThreads = 256;
constexpr int kBlocks = 2 * kNumSM;
constexpr uint32_t kSpinsPerSecond = 1u << 24;  // one poll + 64 ns back-off: about 60 ns

enum Status : int { kOk = 0, kTimeoutOpen = 61, kTimeoutClose = 62, kTimeoutLocal = 63 };

// Control block of a rank (uint32 words, peer memory):
//   [0, 8)  "rank q's product is stored" (word q written by q)    [8, 16) "rank q's slice is written everywhere"
//   [16] local release word   [17] generation   [18] block ticket
constexpr int kCtlWords = 32;

struct Params {
  int world, rank;
  int rows, cols;               // cols = N / world: the slice this rank reduces
  int64_t ld_out;               // N
  const __nv_bfloat16* stage;   // local [world][rows][cols]
  __nv_bfloat16* out[kMaxRanks];  // every rank's [rows][N] output as mapped here
  __nv_bfloat16* out_mc;        // multicast address of the outputs, or nullptr
  const __nv_bfloat16* residual;  // local [rows][N] or nullptr
  uint32_t* ctl[kMaxRanks];
  int barrier;                  // 0: several virtual ranks of one process, run one after another (stream order is the order)
  int* status;
  uint32_t spin_limit;
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
__device__ __forceinline__ void multimem_st8(__nv_bfloat16* mc_ptr, const bf16x8& val) {
  const uint4 v = *reinterpret_cast<const uint4*>(&val);
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc_ptr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Bounded wait until *p == want; false = gave up (status word set) or another wait already failed.
__device__ __forceinline__ bool wait_flag(const uint32_t* p, uint32_t want, int* status, int code, uint32_t spin_limit) {
  for (uint32_t i = 0; i < spin_limit; ++i) {
    if (ld_acquire_sys(p) == want) return true;
    if ((i & 0x3ff) == 0x3ff && *reinterpret_cast<volatile int*>(status) != kOk) return false;
    __nanosleep(64);
  }
  atomicCAS(status, kOk, code);
  return false;
}

__global__ void __launch_bounds__(kThreads)
reduce_broadcast_kernel(const Params p) {
  __shared__ int ok_s;
  uint32_t* ctl = p.ctl[p.rank];
  const uint32_t gen = ctl[17] + 1;  // advanced by the last block on its way out

  // ---- opening barrier: block 0 talks to the other ranks, the others wait for its word
  if (threadIdx.x == 0) {
    bool ok = true;
    if (p.barrier) {
      if (blockIdx.x == 0) {
        __threadfence_system();
        for (int q = 0; q < p.world; ++q) st_release_sys(p.ctl[q] + p.rank, gen);
        for (int q = 0; q < p.world && ok; ++q) ok = wait_flag(ctl + q, gen, p.status, kTimeoutOpen, p.spin_limit);
        st_release_gpu(ctl + 16, ok ? gen : 0xffffffffu);  // a poisoned word releases the other blocks at once
      } else {
        const uint64_t limit = (uint64_t)p.spin_limit * (kMaxRanks + 1);  // the leader's waits run one after another
        for (uint64_t i = 0; i < limit; ++i) {
          const uint32_t v = ld_acquire_gpu(ctl + 16);
          if (v == gen) break;
          if (v == 0xffffffffu || (((i & 0x3ff) == 0x3ff) && *reinterpret_cast<volatile int*>(p.status) != kOk)) { ok = false; break; }
          if (i + 1 == limit) { atomicCAS(p.status, kOk, kTimeoutLocal); ok = false; }
          __nanosleep(64);
        }
      }
    }
    ok_s = ok;
  }
  __syncthreads();
  const bool ok = ok_s != 0;

  // ---- reduce the owned slice and write it to every rank
  if (ok) {
    const int vec_per_row = p.cols >> 3;
    const int64_t nvec = (int64_t)p.rows * vec_per_row, slot = (int64_t)p.rows * p.cols;
    for (int64_t vi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; vi < nvec; vi += (int64_t)gridDim.x * blockDim.x) {
      const int r = (int)(vi / vec_per_row), c = (int)(vi - (int64_t)r * vec_per_row) << 3;
      const int64_t at = (int64_t)r * p.cols + c, out_at = (int64_t)r * p.ld_out + (int64_t)p.rank * p.cols + c;
      float sum[8];
      if (p.residual != nullptr) unpack8(ld8(p.residual + out_at), sum);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] = 0.f;
      }
      for (int q = 0; q < p.world; ++q) {
        float f[8];
        unpack8(ld8(p.stage + q * slot + at), f);
#pragma unroll
        for (int j = 0; j < 8; ++j) sum[j] += f[j];
      }
      const bf16x8 packed = pack8(sum);
      if (p.out_mc != nullptr) multimem_st8(p.out_mc + out_at, packed);
      else
        for (int q = 0; q < p.world; ++q) st8(p.out[q] + out_at, packed);
    }
  }

  // ---- closing barrier: the last block of this rank signals every peer and waits for all of them
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t ticket = atomicAdd(ctl + 18, 1u);
    if (ticket == gridDim.x - 1) {
      ctl[18] = 0;
      if (ok && p.barrier) {
        for (int q = 0; q < p.world; ++q) st_release_sys(p.ctl[q] + 8 + p.rank, gen);
        for (int q = 0; q < p.world; ++q)
          if (!wait_flag(ctl + 8 + q, gen, p.status, kTimeoutClose, p.spin_limit)) break;
      }
      ctl[17] = gen;  // also after a failure, so a retry starts a fresh generation
      __threadfence();
    }
  }
}

}  // namespace tpar

int tp_allreduce_ctl_words() { return tpar::kCtlWords; }

// stage: this rank's staging area [world][rows][cols]; out_peers[q]: rank q's [rows][world * cols] output as mapped on this
// device; out_mc: multicast address of the outputs or nullptr; residual: local [rows][world * cols] or nullptr;
// ctl_peers[q]: rank q's control block.  barrier = 0 skips the cross-rank barriers (virtual ranks of one process).
int launch_tp_reduce_broadcast(int world, int rank, int rows, int cols, const void* stage, void* const* out_peers, void* out_mc,
                               const void* residual, void* const* ctl_peers, int barrier, int* status, uint32_t spin_limit, cudaStream_t stream) {
  if (world < 1 || world > tpar::kMaxRanks || rank < 0 || rank >= world || rows <= 0 || cols <= 0 || (cols & 7)) return -1;
  tpar::Params p{};
  p.world = world;
  p.rank = rank;
  p.rows = rows;
  p.cols = cols;
  p.ld_out = (int64_t)world * cols;
  p.stage = static_cast<const __nv_bfloat16*>(stage);
  for (int q = 0; q < world; ++q) {
    p.out[q] = static_cast<__nv_bfloat16*>(out_peers[q]);
    p.ctl[q] = static_cast<uint32_t*>(ctl_peers[q]);
  }
  p.out_mc = static_cast<__nv_bfloat16*>(out_mc);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.barrier = barrier;
  p.status = status;
  p.spin_limit = spin_limit ? spin_limit : tpar::kSpinsPerSecond;
  count_launch(1);
  const int64_t nvec = (int64_t)rows * (cols >> 3);
  const int blocks = (int)((nvec + tpar::kThreads - 1) / tpar::kThreads < tpar::kBlocks ? (nvec + tpar::kThreads - 1) / tpar::kThreads : tpar::kBlocks);
  tpar::reduce_broadcast_kernel<<<blocks, tpar::kThreads, 0, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace sb200
