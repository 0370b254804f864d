// Masked attention forward on the 5th-generation tensor cores (head_dim 128).
//
// One CTA per (128-query tile, head), 192 threads:
//
//   warp 0   TMA producer: the Q tile once, then K / V tiles of 128 keys into a two-stage
//            ring (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//   warp 1   MMA issuer (one thread): S = Q K^T into one of two TMEM score buffers, and
//            O_tile = P V into a third TMEM buffer; owns the TMEM allocation.  The score
//            GEMM of tile j+1 is issued before the P V GEMM of tile j, so it runs while the
//            softmax threads work on tile j.
//   warps 2-5  softmax: thread i owns query row i (= TMEM lane i).  Per tile it reads its
//            score row from TMEM (tcgen05.ld), applies the row's key interval [lo, hi),
//            keeps the running max / sum in the log2 domain, writes P as bf16 into a
//            swizzled shared-memory tile (the A operand of the second GEMM), then folds the
//            finished O_tile into its fp32 output row held in registers
//            (O = O * alpha + O_tile).  The individually addressed extra keys of a row
//            (training-time-test diagonals, rollout members) are handled by the same thread
//            with plain dot products after the tiled part.
//
// V is consumed as the B operand of the second GEMM straight from its [key, head_dim]
// tile: an MN-major shared-memory descriptor (rows = the contraction index), so no
// transpose is materialised.
//
// All waits are bounded (tcgen05_utils.cuh): a role that runs out of budget records a code
// in the status word, every role then leaves its loop, the CTA meets at the final barrier,
// frees its TMEM and returns.
#include "attention_params.h"
#include "tcgen05_utils.cuh"

namespace sb200 {
namespace atc {

using namespace tc;

constexpr int BM = 128, BN = 128, HD = 128, THREADS = 192;
constexpr int SUB_BYTES = 128 * 64 * 2;   // one [128 rows x 64 columns] bf16 sub-tile
constexpr int TILE_BYTES = 2 * SUB_BYTES;  // a [128 x 128] operand tile
constexpr int TMEM_COLS = 512;             // scores 0: [0,128)  scores 1: [128,256)  O tile: [256,384)
constexpr float kLog2e = 1.4426950408889634f;

enum Status : int { kTimeoutProducer = 31, kTimeoutMma = 32, kTimeoutSoftmax = 33 };

// kind::f16 instruction descriptor: D fp32, A / B bf16, A K-major, B K-major or MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, bool b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// MN-major operand, 128-byte swizzle: shared-memory rows are the contraction index (128 B =
// 64 MN-elements each, 8-row groups 1024 B apart), the next 64 MN-elements start `lbo` bytes on.
__device__ __forceinline__ uint64_t smem_desc_mnmajor_sw128(uint32_t addr, uint32_t lbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3ffff) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const AttnParams p, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* q_s = smem;                       // 32 KB
  unsigned char* k_s = q_s + TILE_BYTES;           // 2 x 32 KB
  unsigned char* v_s = k_s + 2 * TILE_BYTES;       // 2 x 32 KB
  unsigned char* p_s = v_s + 2 * TILE_BYTES;       // 32 KB
  __shared__ __align__(8) uint64_t bar_q, bar_kv_full[2], bar_kv_empty[2], bar_s_full[2], bar_p_ready, bar_o_full;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_range[2];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // late query tiles see the most keys under a causal mask: hand them out first
  const int tile_m = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
  const int kvh = h / (p.nh / p.nkv);
  const int q0 = tile_m * BM;

  if (threadIdx.x == 0) {
    mbar_init(smem_addr(&bar_q), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_addr(&bar_kv_full[s]), 1);
      mbar_init(smem_addr(&bar_kv_empty[s]), 1);
      mbar_init(smem_addr(&bar_s_full[s]), 1);
    }
    mbar_init(smem_addr(&bar_p_ready), 128);
    mbar_init(smem_addr(&bar_o_full), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_range[0] = 0x7fffffff;
    s_range[1] = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  // key range of the CTA: union of the rows' intervals
  int my_lo = 0x7fffffff, my_hi = 0;
  if (threadIdx.x < BM) {
    const int r = q0 + threadIdx.x;
    if (r < p.Tq) {
      const int l = p.lo[r], hgh = min(p.hi[r], p.Tc);
      if (l >= 0 && hgh > l) {
        my_lo = l;
        my_hi = hgh;
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    my_lo = min(my_lo, __shfl_xor_sync(0xffffffffu, my_lo, o));
    my_hi = max(my_hi, __shfl_xor_sync(0xffffffffu, my_hi, o));
  }
  if (lane == 0) {
    atomicMin(&s_range[0], my_lo);
    atomicMax(&s_range[1], my_hi);
  }
  __syncthreads();
  const int c_lo = s_range[0], c_hi = s_range[1];
  const int j0 = c_hi > c_lo ? c_lo / BN : 0;
  const int n_tiles = c_hi > c_lo ? (c_hi + BN - 1) / BN - j0 : 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && n_tiles > 0) {
      const uint32_t qb = smem_addr(&bar_q);
      mbar_expect_tx(qb, TILE_BYTES);
      tma_load_2d(smem_addr(q_s), &map_q, qb, h * HD, q0);
      tma_load_2d(smem_addr(q_s) + SUB_BYTES, &map_q, qb, h * HD + 64, q0);
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t & 1;
        if (!mbar_wait(smem_addr(&bar_kv_empty[st]), ((t >> 1) & 1) ^ 1, status, kTimeoutProducer)) break;
        const uint32_t full = smem_addr(&bar_kv_full[st]);
        mbar_expect_tx(full, 2 * TILE_BYTES);
        const int key0 = (j0 + t) * BN;
        const uint32_t ka = smem_addr(k_s + st * TILE_BYTES), va = smem_addr(v_s + st * TILE_BYTES);
        tma_load_2d(ka, &map_k, full, kvh * HD, key0);
        tma_load_2d(ka + SUB_BYTES, &map_k, full, kvh * HD + 64, key0);
        tma_load_2d(va, &map_v, full, kvh * HD, key0);
        tma_load_2d(va + SUB_BYTES, &map_v, full, kvh * HD + 64, key0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = instr_desc(BM, BN, false);  // S = Q K^T: both operands K-major
      constexpr uint32_t idesc_o = instr_desc(BM, HD, true);   // O = P V: V tile is MN-major
      const uint32_t qa = smem_addr(q_s), pa = smem_addr(p_s);
      auto issue_scores = [&](int t) {  // S[t & 1] = Q K_t^T
        const uint32_t ka = smem_addr(k_s + (t & 1) * TILE_BYTES);
        const uint32_t tmem_s = tmem_base + (t & 1) * BN;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * SUB_BYTES;
          umma_bf16(tmem_s, smem_desc_kmajor_sw128(qa + off) + 2 * (kk & 3), smem_desc_kmajor_sw128(ka + off) + 2 * (kk & 3), idesc_s, kk != 0);
        }
        umma_commit(smem_addr(&bar_s_full[t & 1]));
      };
      bool ok = mbar_wait(smem_addr(&bar_q), 0, status, kTimeoutMma) && mbar_wait(smem_addr(&bar_kv_full[0]), 0, status, kTimeoutMma);
      if (ok) {
        fence_after_sync();
        issue_scores(0);
      }
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) {
          if (!(ok = mbar_wait(smem_addr(&bar_kv_full[(t + 1) & 1]), ((t + 1) >> 1) & 1, status, kTimeoutMma))) break;
          fence_after_sync();
          issue_scores(t + 1);  // runs while the softmax threads are busy with tile t
        }
        if (!(ok = mbar_wait(smem_addr(&bar_p_ready), t & 1, status, kTimeoutMma))) break;
        fence_after_sync();
        const uint32_t va = smem_addr(v_s + (t & 1) * TILE_BYTES);
        const uint32_t tmem_o = tmem_base + 2 * BN;
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // A: P, K-major, 16 keys = 32 bytes inside a swizzled row of the 64-key sub-tile;
          // B: V, MN-major, 16 keys = 16 rows of 128 bytes, head_dim 64.. in the second sub-tile
          const uint64_t adesc = smem_desc_kmajor_sw128(pa + (kk >> 2) * SUB_BYTES) + 2 * (kk & 3);
          const uint64_t bdesc = smem_desc_mnmajor_sw128(va + kk * 2048, SUB_BYTES);
          umma_bf16(tmem_o, adesc, bdesc, idesc_o, kk != 0);
        }
        umma_commit(smem_addr(&bar_o_full));
        umma_commit(smem_addr(&bar_kv_empty[t & 1]));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax (warps 2..5)
    const int quarter = warp & 3;
    const int row = q0 + quarter * 32 + lane;
    const bool row_ok = row < p.Tq;
    const int lo = row_ok ? p.lo[row] : 0x7fffffff;
    const int hi = row_ok ? min(p.hi[row], p.Tc) : 0;
    const float sc = p.scale * kLog2e;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int prow = quarter * 32 + lane;  // row inside the tile
    unsigned char* p_row = p_s + prow * 128;
    const int sw = prow & 7;

    float o[HD];
#pragma unroll
    for (int i = 0; i < HD; ++i) o[i] = 0.f;
    float m = -INFINITY, l = 0.f;
    bool ok = true;

    for (int t = 0; t < n_tiles; ++t) {
      ok = mbar_wait(smem_addr(&bar_s_full[t & 1]), (t >> 1) & 1, status, kTimeoutSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      fence_after_sync();
      const uint32_t tmem_s = lane_base + (t & 1) * BN;
      const int key0 = (j0 + t) * BN;
      // pass 1: row maximum over the allowed keys of this tile
      float tmax = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_s + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int key = key0 + c * 32 + i;
          if (key >= lo && key < hi) tmax = fmaxf(tmax, __uint_as_float(r[i]) * sc);
        }
      }
      const float m_new = fmaxf(m, tmax);
      const float alpha = (m_new == -INFINITY) ? 1.f : exp2f(m - m_new);
      // pass 2: probabilities -> bf16 P tile in shared memory (swizzled like a TMA tile)
      float tsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_s + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int key = key0 + c * 32 + v * 8 + i;
            const bool allowed = key >= lo && key < hi;
            f[i] = allowed ? exp2f(__uint_as_float(r[v * 8 + i]) * sc - m_new) : 0.f;
            tsum += f[i];
          }
          const int chunk = c * 4 + v;  // 16-byte chunk of the 128-key row: sub-tile chunk >> 3, slot chunk & 7
          const bf16x8 packed = pack8(f);
          *reinterpret_cast<uint4*>(p_row + (chunk >> 3) * SUB_BYTES + (((chunk & 7) ^ sw) << 4)) = *reinterpret_cast<const uint4*>(&packed);
        }
      }
      l = l * alpha + tsum;
      m = m_new;
      fence_proxy_async();  // the P tile is read by the tensor core (async proxy)
      fence_before_sync();
      mbar_arrive(smem_addr(&bar_p_ready));
      // fold the finished O tile into the output row
      ok = mbar_wait(smem_addr(&bar_o_full), t & 1, status, kTimeoutSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      fence_after_sync();
      const uint32_t tmem_o = lane_base + 2 * BN;
#pragma unroll
      for (int c = 0; c < HD / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem_o + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = o[c * 32 + i] * alpha + __uint_as_float(r[i]);
      }
      fence_before_sync();
    }

    // individually addressed extra keys of this row
    if (ok && row_ok && p.E > 0) {
      const __nv_bfloat16* qrow = p.q + (int64_t)row * p.q_rs + h * HD;
      for (int e = 0; e < p.E; ++e) {
        const int idx = p.ext_idx[(int64_t)row * p.E + e];
        if (idx < 0 || idx >= p.Te) continue;
        const __nv_bfloat16* kr = p.ke + (int64_t)idx * p.ke_rs + kvh * HD;
        const __nv_bfloat16* vr = p.ve + (int64_t)idx * p.ve_rs + kvh * HD;
        float dot = 0.f;
#pragma unroll 4
        for (int c = 0; c < HD / 8; ++c) {
          float a[8], b[8];
          unpack8(ld8(qrow + c * 8), a);
          unpack8(ld8(kr + c * 8), b);
#pragma unroll
          for (int i = 0; i < 8; ++i) dot += a[i] * b[i];
        }
        const float sv = dot * sc;
        const float m_new = fmaxf(m, sv);
        const float alpha = exp2f(m - m_new), pe = exp2f(sv - m_new);
        l = l * alpha + pe;
        m = m_new;
#pragma unroll
        for (int c = 0; c < HD / 8; ++c) {
          float b[8];
          unpack8(ld8(vr + c * 8), b);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[c * 8 + i] = o[c * 8 + i] * alpha + pe * b[i];
        }
      }
    }

    if (ok && row_ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = p.out + (int64_t)row * p.o_rs + h * HD;
#pragma unroll
      for (int c = 0; c < HD / 8; ++c) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = o[c * 8 + i] * inv;
        st8(orow + c * 8, pack8(f));
      }
      p.lse2[(int64_t)h * p.Tq + row] = l > 0.f ? m + log2f(l) : INFINITY;
    }
  }

  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

}  // namespace atc

// head_dim 128 only; q / k / v rows 16-byte aligned.  `status`: device int for expired waits.
int launch_attn_fwd_tc(const AttnParams& p, int* status, cudaStream_t stream) {
  using namespace atc;
  if (p.Tq <= 0) return 0;
  CUtensorMap map_q, map_k, map_v;
  int rc = tc::make_map_bf16(&map_q, p.q, p.Tq, (int64_t)p.nh * HD, p.q_rs, BM);
  if (rc) return rc;
  rc = tc::make_map_bf16(&map_k, p.k, p.Tc, (int64_t)p.nkv * HD, p.k_rs, BN);
  if (rc) return rc;
  rc = tc::make_map_bf16(&map_v, p.v, p.Tc, (int64_t)p.nkv * HD, p.v_rs, BN);
  if (rc) return rc;
  constexpr int smem_bytes = 6 * TILE_BYTES + 1024;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return -2;
    configured = true;
  }
  dim3 grid((p.Tq + BM - 1) / BM, p.nh);
  count_launch(1);
  attn_fwd_tc_kernel<<<grid, THREADS, smem_bytes, stream>>>(map_q, map_k, map_v, p, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace sb200
