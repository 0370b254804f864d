// Masked attention backward on the 5th-generation tensor cores (head_dim 128): two kernels
// with the same role split as the forward (warp 0 TMA producer, warp 1 single-thread MMA
// issuer and TMEM owner, warps 2-9 element-wise work, two threads per TMEM lane with 64
// columns each).  Every product runs on tcgen05.mma with fp32 accumulators in TMEM; the
// probability / score-gradient tiles go back into TMEM as bf16 pairs and are consumed from
// there as the A operand of the next product, so they never touch shared memory.
//
//   dQ kernel, one CTA per (query tile, head), loop over the key tiles the tile can see:
//       S = Q K^T, dP = dO V^T                 (queries on the TMEM lanes)
//       P = 2^(S * scale * log2e - lse),  dS = P * (dP - delta)      -> TMEM (bf16)
//       dQ += dS K                             (A from TMEM, K tile as MN-major B operand)
//     It also handles the individually addressed extra keys (their dK / dV through fp32
//     atomics).  delta = rowsum(dO * O) comes from a small streaming kernel in front.
//
//   dK/dV kernel, one CTA per (query head, key tile), loop over the query tiles that see it:
//       S^T = K Q^T, dP^T = V dO^T             (keys on the TMEM lanes)
//       P^T, dS^T as above with the per-query statistics read from shared memory
//       dV += P^T dO,  dK += dS^T Q            (A from TMEM, dO / Q tiles as MN-major B)
//     P^T / dS^T overwrite the first half of each thread's own S^T / dP^T columns.  With
//     grouped queries the CTAs of a group write fp32 partials that a reduction kernel sums
//     in head order.
//
// All waits are bounded: a role that runs out of budget records a code in the status word;
// the element-wise threads then keep walking their loops without waiting (so that no
// partner is left alone at a named barrier) and store nothing.
#include "attention_params.h"
#include "tcgen05_utils.cuh"

namespace sb200 {
namespace abtc {

using namespace tc;

constexpr int BM = 128, BN = 128, HD = 128, THREADS = 320;
constexpr int SUB_BYTES = 128 * 64 * 2;    // one [128 rows x 64 columns] bf16 sub-tile
constexpr int TILE_BYTES = 2 * SUB_BYTES;  // a [128 x 128] operand tile
constexpr int TMEM_COLS = 512;
constexpr int SMEM_BYTES = 6 * TILE_BYTES + 1024;
constexpr float kLog2e = 1.4426950408889634f;

enum Status : int {
  kTimeoutDqProducer = 41, kTimeoutDqMma = 42, kTimeoutDqCompute = 43,
  kTimeoutDkvProducer = 44, kTimeoutDkvMma = 45, kTimeoutDkvCompute = 46,
};

// D (+)= A B^T, both operands [128 rows x 128] K-major tiles in shared memory
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint32_t a_tile, uint32_t b_tile, uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint32_t off = (kk >> 2) * SUB_BYTES;
    umma_bf16(tmem_d, smem_desc_kmajor_sw128(a_tile + off) + 2 * (kk & 3), smem_desc_kmajor_sw128(b_tile + off) + 2 * (kk & 3), idesc, kk != 0);
  }
}
// D (+)= A B with A [128 x 128] as bf16 pairs in TMEM (contraction index 0..63 from column
// a0, 64..127 from column a1) and B a [128 contraction rows x 128] tile read MN-major
__device__ __forceinline__ void mma_ts(uint32_t tmem_d, uint32_t a0, uint32_t a1, uint32_t b_tile, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
    const uint32_t a = kk < 4 ? a0 + kk * 8 : a1 + (kk - 4) * 8;
    umma_bf16_ts(tmem_d, a, smem_desc_mnmajor_sw128(b_tile + kk * 2048, SUB_BYTES), idesc, accumulate || kk != 0);
  }
}

// like tc::store_rows64_f32, adding into global memory (several query heads of a group meet on one KV head)
__device__ __forceinline__ void atomic_rows64_f32(unsigned char* stage, const float (&vals)[64], float* gbase, int64_t row_stride, int rows_valid,
                                                  int lane) {
  __syncwarp();
  float4* mine = reinterpret_cast<float4*>(stage + lane * 256);
#pragma unroll
  for (int c = 0; c < 16; ++c) mine[c ^ (lane & 7)] = make_float4(vals[c * 4], vals[c * 4 + 1], vals[c * 4 + 2], vals[c * 4 + 3]);
  __syncwarp();
#pragma unroll
  for (int it = 0; it < 16; ++it) {
    const int r = it * 2 + (lane >> 4), pc = lane & 15;
    const float4 v = reinterpret_cast<const float4*>(stage + r * 256)[pc ^ (r & 7)];
    if (r < rows_valid) atomicAdd(reinterpret_cast<float4*>(gbase + (int64_t)r * row_stride + pc * 4), v);
  }
  __syncwarp();
}

__device__ __forceinline__ void pair_barrier(int quarter) { asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory"); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  const __nv_bfloat162 h2 = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h2);
}

// ---------------------------------------------------------------------------------- delta
// delta[h, row] = sum_c dO[row, h, c] * O[row, h, c]: 16 lanes per (row, head), 16 bytes per lane.
__global__ void __launch_bounds__(256)
attn_delta_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ out, float* __restrict__ delta, int Tq, int nh,
                  int64_t do_rs, int64_t o_rs) {
  const int lane = threadIdx.x & 31, sub = lane >> 4, l16 = lane & 15;
  const int64_t n = (int64_t)Tq * nh;
  for (int64_t base = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * 2; base < n; base += (int64_t)gridDim.x * 16) {
    const int64_t idx = base + sub;
    float acc = 0.f;
    if (idx < n) {
      const int row = (int)(idx / nh), h = (int)(idx % nh);
      float a[8], b[8];
      unpack8(ld8(dout + (int64_t)row * do_rs + h * HD + l16 * 8), a);
      unpack8(ld8(out + (int64_t)row * o_rs + h * HD + l16 * 8), b);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc = fmaf(a[i], b[i], acc);
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (l16 == 0 && idx < n) delta[(int64_t)(idx % nh) * Tq + idx / nh] = acc;
  }
}

// ------------------------------------------------------------------------------------- dQ
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                      const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                      const __grid_constant__ CUtensorMap map_ke, const __grid_constant__ CUtensorMap map_ve,
                      const AttnParams p, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* q_s = smem;
  unsigned char* do_s = q_s + TILE_BYTES;
  // A K tile is read twice, at the start of its tile (S = Q K^T) and at the very end (dQ += dS K),
  // so a stage is only released a whole tile after the next one is needed: three stages keep
  // the refill out of the critical path.  A V tile is done with as soon as dP = dO V^T has
  // been multiplied, before the tile's element-wise work even starts: one buffer, refilled
  // during that work, is enough.
  unsigned char* k_s = do_s + TILE_BYTES;     // 3 stages
  unsigned char* v_s = k_s + 3 * TILE_BYTES;  // 1 buffer
  __shared__ __align__(8) uint64_t bar_qdo, bar_k_full[3], bar_k_empty[3], bar_v_full, bar_v_empty, bar_sdp_full, bar_sdp_free, bar_ds_ready,
      bar_dq_done;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_range[2];
  __shared__ float2 s_xchg[2][2][BM];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, tile_m = gridDim.y - 1 - blockIdx.y;  // heaviest (latest) query tiles first
  const int kvh = h / (p.nh / p.nkv);
  const int q0 = tile_m * BM;

  if (threadIdx.x == 0) {
    mbar_init(smem_addr(&bar_qdo), 1);
    for (int s = 0; s < 3; ++s) {
      mbar_init(smem_addr(&bar_k_full[s]), 1);
      mbar_init(smem_addr(&bar_k_empty[s]), 1);
    }
    mbar_init(smem_addr(&bar_v_full), 1);
    mbar_init(smem_addr(&bar_v_empty), 1);
    mbar_init(smem_addr(&bar_sdp_full), 1);
    mbar_init(smem_addr(&bar_sdp_free), 8);  // one arrival per element-wise warp
    mbar_init(smem_addr(&bar_ds_ready), 8);  // one arrival per element-wise warp
    mbar_init(smem_addr(&bar_dq_done), 1);
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
  // TMEM columns: S [0,128)  dP [128,256)  dQ [256,384)  dS of even / odd tiles [384,448) [448,512)
  constexpr uint32_t COL_S = 0, COL_DP = 128, COL_DQ = 256, COL_DS = 384;

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
  const int n_ctx = c_hi > c_lo ? (c_hi + BN - 1) / BN - j0 : 0;
  // block-structured extras: the query tile's own 128 extra rows are one more key tile (the last); their dK / dV
  // come from the dK/dV kernel's pass over the extra tensors, not from here
  const int n_tiles = n_ctx + (p.ext_block > 0 ? 1 : 0);

  if (warp == 0) {
    if (lane == 0) {
      const uint32_t qb = smem_addr(&bar_qdo);
      mbar_expect_tx(qb, 2 * TILE_BYTES);
      tma_load_2d(smem_addr(q_s), &map_q, qb, h * HD, q0);
      tma_load_2d(smem_addr(q_s) + SUB_BYTES, &map_q, qb, h * HD + 64, q0);
      tma_load_2d(smem_addr(do_s), &map_do, qb, h * HD, q0);
      tma_load_2d(smem_addr(do_s) + SUB_BYTES, &map_do, qb, h * HD + 64, q0);
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t % 3;
        const bool ext = t >= n_ctx;
        const int key0 = ext ? q0 : (j0 + t) * BN;
        const CUtensorMap* mk = ext ? &map_ke : &map_k;
        const CUtensorMap* mv = ext ? &map_ve : &map_v;
        if (!mbar_wait(smem_addr(&bar_k_empty[st]), ((t / 3) & 1) ^ 1, status, kTimeoutDqProducer)) break;
        const uint32_t kfull = smem_addr(&bar_k_full[st]);
        mbar_expect_tx(kfull, TILE_BYTES);
        const uint32_t ka = smem_addr(k_s + st * TILE_BYTES), va = smem_addr(v_s);
        tma_load_2d(ka, mk, kfull, kvh * HD, key0);
        tma_load_2d(ka + SUB_BYTES, mk, kfull, kvh * HD + 64, key0);
        if (!mbar_wait(smem_addr(&bar_v_empty), (t & 1) ^ 1, status, kTimeoutDqProducer)) break;
        const uint32_t vfull = smem_addr(&bar_v_full);
        mbar_expect_tx(vfull, TILE_BYTES);
        tma_load_2d(va, mv, vfull, kvh * HD, key0);
        tma_load_2d(va + SUB_BYTES, mv, vfull, kvh * HD + 64, key0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_kk = instr_desc(BM, BN, false);
      constexpr uint32_t idesc_mn = instr_desc(BM, HD, true);
      const uint32_t qa = smem_addr(q_s), da = smem_addr(do_s);
      auto issue_scores = [&](int t) {  // S = Q K_t^T and dP = dO V_t^T
        mma_ss(tmem_base + COL_S, qa, smem_addr(k_s + (t % 3) * TILE_BYTES), idesc_kk);
        mma_ss(tmem_base + COL_DP, da, smem_addr(v_s), idesc_kk);
        umma_commit(smem_addr(&bar_sdp_full));
        umma_commit(smem_addr(&bar_v_empty));  // the V buffer may be refilled
      };
      bool ok = mbar_wait(smem_addr(&bar_qdo), 0, status, kTimeoutDqMma) && mbar_wait(smem_addr(&bar_k_full[0]), 0, status, kTimeoutDqMma) &&
                mbar_wait(smem_addr(&bar_v_full), 0, status, kTimeoutDqMma);
      if (ok) {
        fence_after_sync();
        issue_scores(0);
      }
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) {
          if (!(ok = mbar_wait(smem_addr(&bar_k_full[(t + 1) % 3]), ((t + 1) / 3) & 1, status, kTimeoutDqMma))) break;
          if (!(ok = mbar_wait(smem_addr(&bar_v_full), (t + 1) & 1, status, kTimeoutDqMma))) break;
          // the element-wise threads hold tile t's S / dP in registers from here on
          if (!(ok = mbar_wait(smem_addr(&bar_sdp_free), t & 1, status, kTimeoutDqMma))) break;
          fence_after_sync();
          issue_scores(t + 1);
        }
        if (!(ok = mbar_wait(smem_addr(&bar_ds_ready), t & 1, status, kTimeoutDqMma))) break;
        fence_after_sync();
        const uint32_t ds = tmem_base + COL_DS + (t & 1) * 64;
        mma_ts(tmem_base + COL_DQ, ds, ds + 32, smem_addr(k_s + (t % 3) * TILE_BYTES), idesc_mn, t > 0);
        umma_commit(smem_addr(&bar_dq_done));
        umma_commit(smem_addr(&bar_k_empty[t % 3]));
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int prow = quarter * 32 + lane;
    const int row = q0 + prow;
    const bool row_ok = row < p.Tq;
    const int lo = row_ok ? p.lo[row] : 0x7fffffff;
    const int hi = row_ok ? min(p.hi[row], p.Tc) : 0;
    const float lse = row_ok ? p.lse2[(int64_t)h * p.Tq + row] : INFINITY;
    const int elo = (row_ok && p.ext_block > 0) ? (row / p.ext_block) * p.ext_block : 0x7fffffff;  // interval in rows of the extra tensors
    const int ehi = (row_ok && p.ext_block > 0) ? min(p.ext_causal ? row + 1 : elo + p.ext_block, p.Te) : 0;
    const float sc = p.scale * kLog2e;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int colh = half * 64;
    const int sw = prow & 7;
    int xc = 0;
    auto exchange = [&](float2 mine) -> float2 {
      float2* slot = s_xchg[xc & 1][0];
      ++xc;
      slot[half * BM + prow] = mine;
      pair_barrier(quarter);
      return slot[(half ^ 1) * BM + prow];
    };

    bool ok = mbar_wait(smem_addr(&bar_qdo), 0, status, kTimeoutDqCompute);
    ok = __all_sync(0xffffffffu, ok);
    const unsigned char* q_row = q_s + half * SUB_BYTES + prow * 128;    // this thread's 64 head-dim columns of q
    const unsigned char* do_row = do_s + half * SUB_BYTES + prow * 128;  // ... and of dO
    const float delta = row_ok ? p.delta[(int64_t)h * p.Tq + row] : 0.f;  // rowsum(dO * O), from attn_delta_kernel

    for (int t = 0; t < n_tiles; ++t) {
      if (ok) ok = mbar_wait(smem_addr(&bar_sdp_full), t & 1, status, kTimeoutDqCompute);
      ok = __all_sync(0xffffffffu, ok);
      fence_after_sync();
      const bool ext = t >= n_ctx;
      const int key0 = (ext ? q0 : (j0 + t) * BN) + colh;
      const int tlo = ext ? elo : lo, thi = ext ? ehi : hi;
      const bool full = __all_sync(0xffffffffu, tlo <= key0 && thi >= key0 + 64);
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t s[32], d[32];
        tmem_ld32(lane_base + COL_S + colh + c * 32, s);
        tmem_ld32(lane_base + COL_DP + colh + c * 32, d);
        tmem_ld_wait();
        if (c == 1) {  // S and dP of the tile are in registers: the next tile's products may overwrite them
          fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_addr(&bar_sdp_free));
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pr0 = ex2(fmaf(__uint_as_float(s[i]), sc, -lse));
          float pr1 = ex2(fmaf(__uint_as_float(s[i + 1]), sc, -lse));
          if (!full) {
            const int key = key0 + c * 32 + i;
            if (key < tlo || key >= thi) pr0 = 0.f;
            if (key + 1 < tlo || key + 1 >= thi) pr1 = 0.f;
          }
          const float ds0 = pr0 * (__uint_as_float(d[i]) - delta);
          const float ds1 = pr1 * (__uint_as_float(d[i + 1]) - delta);
          pk[c * 16 + (i >> 1)] = pack_bf16(ds0, ds1);
        }
      }
      if (t > 0) {
        // the previous dS K product has retired: its dS block (and, one tile on, this one) is free
        if (ok) ok = mbar_wait(smem_addr(&bar_dq_done), (t - 1) & 1, status, kTimeoutDqCompute);
        ok = __all_sync(0xffffffffu, ok);
        fence_after_sync();
      }
      tmem_st32(lane_base + COL_DS + (t & 1) * 64 + half * 32, pk);
      tmem_st_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar_ds_ready));
    }

    float dq[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) dq[i] = 0.f;
    if (n_tiles > 0) {
      if (ok) ok = mbar_wait(smem_addr(&bar_dq_done), (n_tiles - 1) & 1, status, kTimeoutDqCompute);
      ok = __all_sync(0xffffffffu, ok);
      fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t a[32];
        tmem_ld32(lane_base + COL_DQ + colh + c * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) dq[c * 32 + i] = __uint_as_float(a[i]);
      }
      fence_before_sync();
    }

    // Individually addressed extra keys: each thread of the pair takes 64 of the 128
    // dimensions of q.k and dO.v, the halves meet through the exchange slots.  Rows of the
    // extra K / V tensors and the dK / dV contributions travel through a per-warp staging
    // area (the K / V stages, idle once the tile loop has drained) so that global loads and
    // atomics are issued warp-wide over whole rows instead of one row per lane.
    if (p.E > 0) {
      unsigned char* stage = k_s + (warp - 2) * 16384;  // 16 KB per warp
      for (int e = 0; e < p.E; ++e) {
        const int idx = row_ok ? p.ext_idx[(int64_t)row * p.E + e] : -1;
        const bool valid = idx >= 0 && idx < p.Te;
        const int idc = valid ? idx : 0;
        // stage in: 8 lanes fetch the 128 bytes of one row's half, 4 rows per instruction
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int r = it * 4 + (lane >> 3), pc = lane & 7;
          const int64_t ir = __shfl_sync(0xffffffffu, idc, r);
          const bf16x8 kx = ld8(p.ke + ir * p.ke_rs + kvh * HD + colh + pc * 8);
          const bf16x8 vx = ld8(p.ve + ir * p.ve_rs + kvh * HD + colh + pc * 8);
          *reinterpret_cast<bf16x8*>(stage + r * 128 + ((pc ^ (r & 7)) << 4)) = kx;
          *reinterpret_cast<bf16x8*>(stage + 4096 + r * 128 + ((pc ^ (r & 7)) << 4)) = vx;
        }
        __syncwarp();
        const unsigned char* k_row = stage + lane * 128;
        const unsigned char* v_row = stage + 4096 + lane * 128;
        const int lsw = lane & 7;
        float dot = 0.f, dpe = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float a[8], b[8], g[8], w[8];
          unpack8(*reinterpret_cast<const bf16x8*>(q_row + ((c ^ sw) << 4)), a);
          unpack8(*reinterpret_cast<const bf16x8*>(k_row + ((c ^ lsw) << 4)), b);
          unpack8(*reinterpret_cast<const bf16x8*>(do_row + ((c ^ sw) << 4)), g);
          unpack8(*reinterpret_cast<const bf16x8*>(v_row + ((c ^ lsw) << 4)), w);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dot = fmaf(a[i], b[i], dot);
            dpe = fmaf(g[i], w[i], dpe);
          }
        }
        const float2 other = exchange(make_float2(dot, dpe));
        const float pe = valid ? ex2(fmaf(dot + other.x, sc, -lse)) : 0.f;
        const float dse = pe * (dpe + other.y - delta);
        const float dss = dse * p.scale;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float b[8];
          unpack8(*reinterpret_cast<const bf16x8*>(k_row + ((c ^ lsw) << 4)), b);
#pragma unroll
          for (int i = 0; i < 8; ++i) dq[c * 8 + i] = fmaf(dse, b[i], dq[c * 8 + i]);
        }
        // contributions to the extra keys' dK (dss * q) then dV (pe * dO): each lane lays its
        // row's 64 floats into the staging area, then 16 lanes add one row's 256 bytes
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          const unsigned char* src_row = which ? do_row : q_row;
          const float mul = which ? pe : dss;
          float* dst_base = (which ? p.dve : p.dke) + kvh * HD + colh;
          __syncwarp();
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float a[8];
            unpack8(*reinterpret_cast<const bf16x8*>(src_row + ((c ^ sw) << 4)), a);
            float4* out4 = reinterpret_cast<float4*>(stage + 8192 + lane * 256);
            out4[(2 * c) ^ lsw] = make_float4(mul * a[0], mul * a[1], mul * a[2], mul * a[3]);
            out4[(2 * c + 1) ^ lsw] = make_float4(mul * a[4], mul * a[5], mul * a[6], mul * a[7]);
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 16; ++it) {
            const int r = it * 2 + (lane >> 4), pc = lane & 15;
            const int ir = __shfl_sync(0xffffffffu, valid && ok ? idx : -1, r);
            const float4 val = reinterpret_cast<const float4*>(stage + 8192 + r * 256)[pc ^ (r & 7)];
            if (ir >= 0) atomicAdd(reinterpret_cast<float4*>(dst_base + (int64_t)ir * p.nkv * HD + pc * 4), val);
          }
        }
      }
    }

    if (__all_sync(0xffffffffu, ok)) {
      // whole rows through the warp's staging area (the K / V stages are idle by now)
      const int warp_row0 = q0 + quarter * 32;
      store_rows64_bf16(k_s + (warp - 2) * 16384, dq, p.scale, p.dq + (int64_t)warp_row0 * p.dq_rs + h * HD + colh, p.dq_rs, p.Tq - warp_row0, lane);
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

// ---------------------------------------------------------------------------------- dK / dV
__global__ void __launch_bounds__(THREADS, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                       const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const AttnParams p, int n_range_tiles, int ext_mode, int* status) {
  // ext_mode (block-structured extras): the key tiles are tiles of the extra K / V tensors (the caller passes their
  // tensor maps as map_k / map_v); key tile j is seen by query tile j alone, under the block mask, and the result is
  // added (fp32 atomics over the query heads of a group) into dke / dve.
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* k_s = smem;
  unsigned char* v_s = k_s + TILE_BYTES;
  unsigned char* q_s = v_s + TILE_BYTES;       // 2 stages
  unsigned char* do_s = q_s + 2 * TILE_BYTES;  // 2 stages
  __shared__ __align__(8) uint64_t bar_kv, bar_qdo_full[2], bar_qdo_empty[2], bar_s_full, bar_dp_full, bar_p_ready, bar_ds_ready,
      bar_dv_done, bar_dk_done;
  __shared__ uint32_t tmem_base_slot;
  // per-query statistics of the query tile in flight, two buffers
  __shared__ __align__(16) float st_lse[2][BM];
  __shared__ __align__(16) float st_delta[2][BM];
  __shared__ __align__(16) int st_lo[2][BM];
  __shared__ __align__(16) int st_hi[2][BM];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.x, j = blockIdx.y;  // key tile 0 is seen by the most queries under a causal mask: first
  const int group = p.nh / p.nkv;
  const int kvh = h / group;
  const int key_base = j * BN;

  if (threadIdx.x == 0) {
    mbar_init(smem_addr(&bar_kv), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_addr(&bar_qdo_full[s]), 1);
      mbar_init(smem_addr(&bar_qdo_empty[s]), 1);
    }
    mbar_init(smem_addr(&bar_s_full), 1);
    mbar_init(smem_addr(&bar_dp_full), 1);
    mbar_init(smem_addr(&bar_p_ready), 8);  // one arrival per element-wise warp
    mbar_init(smem_addr(&bar_ds_ready), 8);  // one arrival per element-wise warp
    mbar_init(smem_addr(&bar_dv_done), 1);
    mbar_init(smem_addr(&bar_dk_done), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;
  // TMEM columns: S^T [0,128)  dP^T [128,256)  dV [256,384)  dK [384,512); P^T / dS^T reuse
  // columns [0,32) + [64,96) of the S^T / dP^T block
  constexpr uint32_t COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 384;

  // query rows that can see this key tile (ranges are kept per 64 keys)
  int qmin = 0x7fffffff, qmax = 0;
#pragma unroll
  for (int s = 0; s < BN / kAttnKeyTile; ++s) {
    const int rt = j * (BN / kAttnKeyTile) + s;
    if (rt < n_range_tiles) {
      qmin = min(qmin, p.tile_qmin[rt]);
      qmax = max(qmax, p.tile_qmax[rt]);
    }
  }
  const int i0 = ext_mode ? j : (qmax > qmin ? qmin / BM : 0);
  const int n_tiles = ext_mode ? (j * BM < p.Tq ? 1 : 0) : (qmax > qmin ? (qmax + BM - 1) / BM - i0 : 0);
  const int n_keys = ext_mode ? p.Te : p.Tc;

  if (warp == 0) {
    if (lane == 0 && n_tiles > 0) {
      const uint32_t kvb = smem_addr(&bar_kv);
      mbar_expect_tx(kvb, 2 * TILE_BYTES);
      tma_load_2d(smem_addr(k_s), &map_k, kvb, kvh * HD, key_base);
      tma_load_2d(smem_addr(k_s) + SUB_BYTES, &map_k, kvb, kvh * HD + 64, key_base);
      tma_load_2d(smem_addr(v_s), &map_v, kvb, kvh * HD, key_base);
      tma_load_2d(smem_addr(v_s) + SUB_BYTES, &map_v, kvb, kvh * HD + 64, key_base);
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t & 1;
        if (!mbar_wait(smem_addr(&bar_qdo_empty[st]), ((t >> 1) & 1) ^ 1, status, kTimeoutDkvProducer)) break;
        const uint32_t full = smem_addr(&bar_qdo_full[st]);
        mbar_expect_tx(full, 2 * TILE_BYTES);
        const int r0 = (i0 + t) * BM;
        const uint32_t qa = smem_addr(q_s + st * TILE_BYTES), da = smem_addr(do_s + st * TILE_BYTES);
        tma_load_2d(qa, &map_q, full, h * HD, r0);
        tma_load_2d(qa + SUB_BYTES, &map_q, full, h * HD + 64, r0);
        tma_load_2d(da, &map_do, full, h * HD, r0);
        tma_load_2d(da + SUB_BYTES, &map_do, full, h * HD + 64, r0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_kk = instr_desc(BN, BM, false);
      constexpr uint32_t idesc_mn = instr_desc(BN, HD, true);
      const uint32_t ka = smem_addr(k_s), va = smem_addr(v_s);
      const uint32_t t_st = tmem_base + COL_ST, t_dpt = tmem_base + COL_DPT;
      bool ok = mbar_wait(smem_addr(&bar_kv), 0, status, kTimeoutDkvMma) && mbar_wait(smem_addr(&bar_qdo_full[0]), 0, status, kTimeoutDkvMma);
      if (ok) {
        fence_after_sync();
        mma_ss(t_st, ka, smem_addr(q_s), idesc_kk);  // S^T = K Q^T
        umma_commit(smem_addr(&bar_s_full));
        mma_ss(t_dpt, va, smem_addr(do_s), idesc_kk);  // dP^T = V dO^T
        umma_commit(smem_addr(&bar_dp_full));
      }
      for (int t = 0; t < n_tiles && ok; ++t) {
        const uint32_t q_t = smem_addr(q_s + (t & 1) * TILE_BYTES), do_t = smem_addr(do_s + (t & 1) * TILE_BYTES);
        const uint32_t q_n = smem_addr(q_s + ((t + 1) & 1) * TILE_BYTES), do_n = smem_addr(do_s + ((t + 1) & 1) * TILE_BYTES);
        if (!(ok = mbar_wait(smem_addr(&bar_p_ready), t & 1, status, kTimeoutDkvMma))) break;
        fence_after_sync();
        mma_ts(tmem_base + COL_DV, t_st, t_st + 64, do_t, idesc_mn, t > 0);  // dV += P^T dO
        umma_commit(smem_addr(&bar_dv_done));
        if (t + 1 < n_tiles) {
          if (!(ok = mbar_wait(smem_addr(&bar_qdo_full[(t + 1) & 1]), ((t + 1) >> 1) & 1, status, kTimeoutDkvMma))) break;
          // P^T of tile t shares its columns with S^T: wait until the product above has read it
          if (!(ok = mbar_wait(smem_addr(&bar_dv_done), t & 1, status, kTimeoutDkvMma))) break;
          fence_after_sync();
          mma_ss(t_st, ka, q_n, idesc_kk);
          umma_commit(smem_addr(&bar_s_full));
        }
        if (!(ok = mbar_wait(smem_addr(&bar_ds_ready), t & 1, status, kTimeoutDkvMma))) break;
        fence_after_sync();
        mma_ts(tmem_base + COL_DK, t_dpt, t_dpt + 64, q_t, idesc_mn, t > 0);  // dK += dS^T Q
        umma_commit(smem_addr(&bar_dk_done));
        umma_commit(smem_addr(&bar_qdo_empty[t & 1]));
        if (t + 1 < n_tiles) {
          if (!(ok = mbar_wait(smem_addr(&bar_dk_done), t & 1, status, kTimeoutDkvMma))) break;
          fence_after_sync();
          mma_ss(t_dpt, va, do_n, idesc_kk);
          umma_commit(smem_addr(&bar_dp_full));
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int krow = quarter * 32 + lane;  // key row inside the tile = TMEM lane
    const int key = key_base + krow;
    const int ct = (warp - 2) * 32 + lane;  // 0..255: loader index for the per-query statistics
    const float sc = p.scale * kLog2e;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int colh = half * 64;  // this thread's 64 queries of the tile / 64 head-dim columns of the outputs
    bool ok = true;

    // statistics of query `i0 * BM + ..` go through registers one tile ahead
    float ld_a = 0.f, ld_b = 0.f;  // lse, delta (ct < 128) or lo, hi as bit patterns (ct >= 128)
    uint32_t ld_full = 1;
    auto fetch_stats = [&](int t) {
      const int r = (i0 + t) * BM + (ct & (BM - 1));
      const bool in = r < p.Tq;
      if (ct < BM) {
        ld_a = in ? p.lse2[(int64_t)h * p.Tq + r] : INFINITY;
        ld_b = in ? p.delta[(int64_t)h * p.Tq + r] : 0.f;
        ld_full = 1;
      } else {
        int l = in ? p.lo[r] : 0x7fffffff;
        int hgh = in ? min(p.hi[r], p.Tc) : 0;
        if (ext_mode) {  // the query's interval in rows of the extra tensors
          l = in ? (r / p.ext_block) * p.ext_block : 0x7fffffff;
          hgh = in ? min(p.ext_causal ? r + 1 : l + p.ext_block, p.Te) : 0;
        }
        ld_a = __int_as_float(l);
        ld_b = __int_as_float(hgh);
        ld_full = (l <= key_base && hgh >= key_base + BN) ? 1u : 0u;
      }
    };
    auto stash_stats = [&](int t) {
      const int b = t & 1, c = ct & (BM - 1);
      if (ct < BM) {
        st_lse[b][c] = ld_a;
        st_delta[b][c] = ld_b;
      } else {
        st_lo[b][c] = __float_as_int(ld_a);
        st_hi[b][c] = __float_as_int(ld_b);
      }
    };
    if (n_tiles > 0) {
      fetch_stats(0);
      stash_stats(0);
    }

    for (int t = 0; t < n_tiles; ++t) {
      // all 256 threads meet: statistics of tile t are visible, and `full` says whether every
      // query of the tile sees every key of this key tile
      uint32_t full;
      asm volatile(
          "{\n\t.reg .pred pi, po;\n\t"
          "setp.ne.u32 pi, %1, 0;\n\t"
          "bar.red.and.pred po, 9, 256, pi;\n\t"
          "selp.u32 %0, 1, 0, po;\n\t}"
          : "=r"(full)
          : "r"(ld_full)
          : "memory");
      if (t + 1 < n_tiles) fetch_stats(t + 1);  // in flight during the tile's work
      const int b = t & 1;

      if (ok) ok = mbar_wait(smem_addr(&bar_s_full), t & 1, status, kTimeoutDkvCompute);
      ok = __all_sync(0xffffffffu, ok);
      fence_after_sync();
      uint32_t s[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) tmem_ld32(lane_base + COL_ST + colh + c * 32, s[c]);
      tmem_ld_wait();
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const int qi = colh + c * 32 + i;
          const float4 l4 = *reinterpret_cast<const float4*>(&st_lse[b][qi]);
          float pr[4];
          pr[0] = ex2(fmaf(__uint_as_float(s[c][i]), sc, -l4.x));
          pr[1] = ex2(fmaf(__uint_as_float(s[c][i + 1]), sc, -l4.y));
          pr[2] = ex2(fmaf(__uint_as_float(s[c][i + 2]), sc, -l4.z));
          pr[3] = ex2(fmaf(__uint_as_float(s[c][i + 3]), sc, -l4.w));
          if (!full) {
            const int4 lo4 = *reinterpret_cast<const int4*>(&st_lo[b][qi]);
            const int4 hi4 = *reinterpret_cast<const int4*>(&st_hi[b][qi]);
            if (key < lo4.x || key >= hi4.x) pr[0] = 0.f;
            if (key < lo4.y || key >= hi4.y) pr[1] = 0.f;
            if (key < lo4.z || key >= hi4.z) pr[2] = 0.f;
            if (key < lo4.w || key >= hi4.w) pr[3] = 0.f;
          }
#pragma unroll
          for (int u = 0; u < 4; ++u) s[c][i + u] = __float_as_uint(pr[u]);
          pk[c * 16 + (i >> 1)] = pack_bf16(pr[0], pr[1]);
          pk[c * 16 + (i >> 1) + 1] = pack_bf16(pr[2], pr[3]);
        }
      tmem_st32(lane_base + COL_ST + colh, pk);  // P^T over the first half of this thread's own S^T columns
      tmem_st_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar_p_ready));

      if (ok) ok = mbar_wait(smem_addr(&bar_dp_full), t & 1, status, kTimeoutDkvCompute);
      ok = __all_sync(0xffffffffu, ok);
      fence_after_sync();
      uint32_t d[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) tmem_ld32(lane_base + COL_DPT + colh + c * 32, d[c]);
      tmem_ld_wait();
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          const float4 d4 = *reinterpret_cast<const float4*>(&st_delta[b][colh + c * 32 + i]);
          const float ds0 = __uint_as_float(s[c][i]) * (__uint_as_float(d[c][i]) - d4.x);
          const float ds1 = __uint_as_float(s[c][i + 1]) * (__uint_as_float(d[c][i + 1]) - d4.y);
          const float ds2 = __uint_as_float(s[c][i + 2]) * (__uint_as_float(d[c][i + 2]) - d4.z);
          const float ds3 = __uint_as_float(s[c][i + 3]) * (__uint_as_float(d[c][i + 3]) - d4.w);
          pk[c * 16 + (i >> 1)] = pack_bf16(ds0, ds1);
          pk[c * 16 + (i >> 1) + 1] = pack_bf16(ds2, ds3);
        }
      tmem_st32(lane_base + COL_DPT + colh, pk);  // dS^T over the first half of this thread's own dP^T columns
      tmem_st_wait();
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar_ds_ready));
      if (t + 1 < n_tiles) stash_stats(t + 1);
    }

    // results: this thread's key row, 64 head-dim columns of dV and of dK
    float acc[64];
    const int64_t plane = (int64_t)p.Tc * p.nkv * HD;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {  // 0: dK, 1: dV
#pragma unroll
      for (int i = 0; i < 64; ++i) acc[i] = 0.f;
      if (n_tiles > 0) {
        if (ok) ok = mbar_wait(smem_addr(which ? &bar_dv_done : &bar_dk_done), (n_tiles - 1) & 1, status, kTimeoutDkvCompute);
        ok = __all_sync(0xffffffffu, ok);
        fence_after_sync();
        const float mul = which ? 1.f : p.scale;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t a[32];
          tmem_ld32(lane_base + (which ? COL_DV : COL_DK) + colh + c * 32, a);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[c * 32 + i] = __uint_as_float(a[i]) * mul;
        }
        fence_before_sync();
      }
      if (__all_sync(0xffffffffu, ok)) {
        // whole rows through the warp's staging area (the Q / dO stages are idle by now)
        unsigned char* stage = q_s + (warp - 2) * 16384;
        const int warp_key0 = key_base + quarter * 32;
        const int64_t off0 = ((int64_t)warp_key0 * p.nkv + kvh) * HD + colh;
        if (ext_mode)
          atomic_rows64_f32(stage, acc, (which ? p.dve : p.dke) + off0, (int64_t)p.nkv * HD, n_keys - warp_key0, lane);
        else if (p.dkv_part != nullptr)
          store_rows64_f32(stage, acc, p.dkv_part + (int64_t)(h - kvh * group) * 2 * plane + which * plane + off0, (int64_t)p.nkv * HD,
                           p.Tc - warp_key0, lane);
        else
          store_rows64_bf16(stage, acc, 1.f, (which ? p.dv : p.dk) + off0, (int64_t)p.nkv * HD, p.Tc - warp_key0, lane);
      }
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

}  // namespace abtc

// head_dim 128; tile_qmin / tile_qmax: scratch of one int per 64-key tile, fully written here.
int launch_attn_bwd_tc(const AttnParams& p, int* tile_qmin, int* tile_qmax, int* status, cudaStream_t stream) {
  using namespace abtc;
  if (p.Tq <= 0) return 0;
  CUtensorMap map_q, map_do, map_k, map_v;
  int rc = tc::make_map_bf16(&map_q, p.q, p.Tq, (int64_t)p.nh * HD, p.q_rs, BM);
  if (rc) return rc;
  rc = tc::make_map_bf16(&map_do, p.dout, p.Tq, (int64_t)p.nh * HD, p.do_rs, BM);
  if (rc) return rc;
  rc = tc::make_map_bf16(&map_k, p.k, p.Tc, (int64_t)p.nkv * HD, p.k_rs, BN);
  if (rc) return rc;
  rc = tc::make_map_bf16(&map_v, p.v, p.Tc, (int64_t)p.nkv * HD, p.v_rs, BN);
  if (rc) return rc;
  CUtensorMap map_ke = map_k, map_ve = map_v;
  if (p.ext_block > 0) {
    if (p.E != 0 || BM % p.ext_block != 0 || p.ke == nullptr || p.ve == nullptr || p.dke == nullptr || p.dve == nullptr) return -4;
    rc = tc::make_map_bf16(&map_ke, p.ke, p.Te, (int64_t)p.nkv * HD, p.ke_rs, BN);
    if (rc) return rc;
    rc = tc::make_map_bf16(&map_ve, p.ve, p.Te, (int64_t)p.nkv * HD, p.ve_rs, BN);
    if (rc) return rc;
  }
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(attn_bwd_dq_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -2;
    if (cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) return -2;
    configured.mark();
  }
  count_launch(3);
  {
    const int64_t pairs = (int64_t)p.Tq * p.nh;
    const int64_t blocks = (pairs + 15) / 16;
    attn_delta_kernel<<<(int)(blocks < 16 * kNumSM ? blocks : 16 * kNumSM), 256, 0, stream>>>(p.dout, p.out, p.delta, p.Tq, p.nh, p.do_rs, p.o_rs);
  }
  dim3 grid_q(p.nh, (p.Tq + BM - 1) / BM);
  attn_bwd_dq_tc_kernel<<<grid_q, THREADS, SMEM_BYTES, stream>>>(map_q, map_do, map_k, map_v, map_ke, map_ve, p, status);
  rc = launch_kv_tile_range(p, tile_qmin, tile_qmax, stream);
  if (rc) return rc;
  dim3 grid_kv(p.nh, (p.Tc + BN - 1) / BN);
  attn_bwd_dkv_tc_kernel<<<grid_kv, THREADS, SMEM_BYTES, stream>>>(map_q, map_do, map_k, map_v, p, (p.Tc + kAttnKeyTile - 1) / kAttnKeyTile, 0, status);
  if (p.ext_block > 0) {  // gradients of the extra keys: one key tile per query tile, read from the extra tensors
    count_launch(1);
    dim3 grid_ext(p.nh, (p.Te + BN - 1) / BN);
    attn_bwd_dkv_tc_kernel<<<grid_ext, THREADS, SMEM_BYTES, stream>>>(map_q, map_do, map_ke, map_ve, p, 0, 1, status);
  }
  if (p.dkv_part != nullptr) {
    rc = launch_dkv_reduce(p, stream);
    if (rc) return rc;
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace sb200
