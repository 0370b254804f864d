// Masked attention forward on the 5th-generation tensor cores (head_dim 128).
//
// One CTA per (128-query tile, head), 320 threads:
//
//   warp 0   TMA producer: the Q tile once, then K / V tiles of 128 keys into a two-stage
//            ring (cp.async.bulk.tensor, 128-byte swizzle, no multicast)
//   warp 1   MMA issuer (one thread): S = Q K^T into one of two TMEM score buffers, and
//            O += P V into a third TMEM buffer; owns the TMEM allocation.  The score
//            GEMM of tile j+1 is issued before the P V GEMM of tile j, so it runs while the
//            softmax threads work on tile j.
//   warps 2-9  softmax: two threads per query row (= TMEM lane), 64 columns each.  Per tile a
//            thread reads its half of the score row from TMEM (tcgen05.ld), applies the
//            row's key interval [lo, hi), keeps the running max / sum in the log2 domain and
//            writes P as bf16 pairs back into TMEM (tcgen05.st), from where the second GEMM
//            takes it as its A operand - P never touches shared memory.  O accumulates in TMEM across the tiles; a thread rescales its part of
//            the TMEM row (tcgen05.ld / st) only when the row maximum has moved by more than
//            2^8 since the last rescale.  The individually addressed extra keys of a row
//            (training-time-test diagonals, rollout members) are handled by the same two
//            threads with plain dot products after the tiled part.
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

constexpr int BM = 128, BN = 128, HD = 128, THREADS = 320;
constexpr int SUB_BYTES = 128 * 64 * 2;   // one [128 rows x 64 columns] bf16 sub-tile
constexpr int TILE_BYTES = 2 * SUB_BYTES;  // a [128 x 128] operand tile
constexpr int TMEM_COLS = 512;             // scores 0: [0,128)  scores 1: [128,256)  O: [256,384)  P 0 / P 1 (bf16 pairs): [384,448) [448,512)
constexpr float kLog2e = 1.4426950408889634f;

enum Status : int { kTimeoutProducer = 31, kTimeoutMma = 32, kTimeoutSoftmax = 33 };

__global__ void __launch_bounds__(THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                   const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_ke,
                   const __grid_constant__ CUtensorMap map_ve, const AttnParams p, int* status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char* q_s = smem;                       // 32 KB
  unsigned char* k_s = q_s + TILE_BYTES;           // 2 x 32 KB
  unsigned char* v_s = k_s + 2 * TILE_BYTES;       // 2 x 32 KB
  __shared__ __align__(8) uint64_t bar_q, bar_k_full[2], bar_k_empty[2], bar_v_full[2], bar_v_empty[2], bar_s_full[2], bar_p_ready, bar_o_full;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int s_range[2];
  __shared__ float s_xchg[2][2][BM];  // [slot][column half][row]: values the two threads of a row hand each other

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // late query tiles see the most keys under a causal mask: hand them out first (heads vary
  // fastest, so the hardware's block order is heaviest-first over the whole grid)
  const int tile_m = gridDim.y - 1 - blockIdx.y, h = blockIdx.x;
  const int kvh = h / (p.nh / p.nkv);
  const int q0 = tile_m * BM;

  if (threadIdx.x == 0) {
    mbar_init(smem_addr(&bar_q), 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(smem_addr(&bar_k_full[s]), 1);
      mbar_init(smem_addr(&bar_k_empty[s]), 1);
      mbar_init(smem_addr(&bar_v_full[s]), 1);
      mbar_init(smem_addr(&bar_v_empty[s]), 1);
      mbar_init(smem_addr(&bar_s_full[s]), 1);
    }
    mbar_init(smem_addr(&bar_p_ready), 8);  // one arrival per softmax warp
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
  const int n_ctx = c_hi > c_lo ? (c_hi + BN - 1) / BN - j0 : 0;
  // block-structured extras: the tile's own 128 extra rows are one more key tile (the last one)
  const int n_tiles = n_ctx + (p.ext_block > 0 ? 1 : 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0 && (n_tiles > 0 || p.E > 0)) {
      const uint32_t qb = smem_addr(&bar_q);
      mbar_expect_tx(qb, TILE_BYTES);
      tma_load_2d(smem_addr(q_s), &map_q, qb, h * HD, q0);
      tma_load_2d(smem_addr(q_s) + SUB_BYTES, &map_q, qb, h * HD + 64, q0);
      // K stages are released by the score GEMM, V stages by the P.V GEMM one tile later, so a
      // K tile can be fetched a whole tile ahead of its V tile
      for (int t = 0; t < n_tiles; ++t) {
        const int st = t & 1;
        const uint32_t par = ((t >> 1) & 1) ^ 1;
        const bool ext = t >= n_ctx;
        const int key0 = ext ? q0 : (j0 + t) * BN;
        const CUtensorMap* mk = ext ? &map_ke : &map_k;
        const CUtensorMap* mv = ext ? &map_ve : &map_v;
        if (!mbar_wait(smem_addr(&bar_k_empty[st]), par, status, kTimeoutProducer)) break;
        const uint32_t kfull = smem_addr(&bar_k_full[st]);
        mbar_expect_tx(kfull, TILE_BYTES);
        const uint32_t ka = smem_addr(k_s + st * TILE_BYTES), va = smem_addr(v_s + st * TILE_BYTES);
        tma_load_2d(ka, mk, kfull, kvh * HD, key0);
        tma_load_2d(ka + SUB_BYTES, mk, kfull, kvh * HD + 64, key0);
        if (!mbar_wait(smem_addr(&bar_v_empty[st]), par, status, kTimeoutProducer)) break;
        const uint32_t vfull = smem_addr(&bar_v_full[st]);
        mbar_expect_tx(vfull, TILE_BYTES);
        tma_load_2d(va, mv, vfull, kvh * HD, key0);
        tma_load_2d(va + SUB_BYTES, mv, vfull, kvh * HD + 64, key0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0 && n_tiles > 0) {
      constexpr uint32_t idesc_s = instr_desc(BM, BN, false);  // S = Q K^T: both operands K-major
      constexpr uint32_t idesc_o = instr_desc(BM, HD, true);   // O = P V: V tile is MN-major
      const uint32_t qa = smem_addr(q_s);
      auto issue_scores = [&](int t) {  // S[t & 1] = Q K_t^T
        const uint32_t ka = smem_addr(k_s + (t & 1) * TILE_BYTES);
        const uint32_t tmem_s = tmem_base + (t & 1) * BN;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * SUB_BYTES;
          umma_bf16(tmem_s, smem_desc_kmajor_sw128(qa + off) + 2 * (kk & 3), smem_desc_kmajor_sw128(ka + off) + 2 * (kk & 3), idesc_s, kk != 0);
        }
        umma_commit(smem_addr(&bar_s_full[t & 1]));
        umma_commit(smem_addr(&bar_k_empty[t & 1]));
      };
      bool ok = mbar_wait(smem_addr(&bar_q), 0, status, kTimeoutMma) && mbar_wait(smem_addr(&bar_k_full[0]), 0, status, kTimeoutMma);
      if (ok) {
        fence_after_sync();
        issue_scores(0);
      }
      for (int t = 0; t < n_tiles && ok; ++t) {
        if (t + 1 < n_tiles) {
          if (!(ok = mbar_wait(smem_addr(&bar_k_full[(t + 1) & 1]), ((t + 1) >> 1) & 1, status, kTimeoutMma))) break;
          fence_after_sync();
          issue_scores(t + 1);  // runs while the softmax threads are busy with tile t
        }
        if (!(ok = mbar_wait(smem_addr(&bar_v_full[t & 1]), (t >> 1) & 1, status, kTimeoutMma))) break;
        if (!(ok = mbar_wait(smem_addr(&bar_p_ready), t & 1, status, kTimeoutMma))) break;
        fence_after_sync();
        const uint32_t va = smem_addr(v_s + (t & 1) * TILE_BYTES);
        const uint32_t tmem_o = tmem_base + 2 * BN;
        const uint32_t tmem_p = tmem_base + 3 * BN + (t & 1) * (BN / 2);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          // A: P from TMEM, 16 keys = 8 columns of bf16 pairs;
          // B: V, MN-major, 16 keys = 16 rows of 128 bytes, head_dim 64.. in the second sub-tile
          const uint64_t bdesc = smem_desc_mnmajor_sw128(va + kk * 2048, SUB_BYTES);
          umma_bf16_ts(tmem_o, tmem_p + kk * 8, bdesc, idesc_o, (t | kk) != 0);
        }
        umma_commit(smem_addr(&bar_o_full));
        umma_commit(smem_addr(&bar_v_empty[t & 1]));
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax (warps 2..9)
    // Two threads per query row: warps w and w + 4 reach the same TMEM lanes (lane quarter =
    // warp % 4) and split the columns - 64 keys of a score tile, 64 head-dim columns of O.
    // They exchange their partial row maxima (and partial dot products of the extra keys)
    // through shared memory across a 64-thread named barrier.  No early exit on an expired
    // wait: a thread that gave up keeps walking the loop without waiting, so its partner is
    // never left alone at the named barrier; nothing is stored in that case.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int prow = quarter * 32 + lane;  // row inside the tile
    const int row = q0 + prow;
    const bool row_ok = row < p.Tq;
    const int lo = row_ok ? p.lo[row] : 0x7fffffff;
    const int hi = row_ok ? min(p.hi[row], p.Tc) : 0;
    // block-structured extras: the row's interval in rows of the extra tensors
    const int elo = (row_ok && p.ext_block > 0) ? (row / p.ext_block) * p.ext_block : 0x7fffffff;
    const int ehi = (row_ok && p.ext_block > 0) ? min(p.ext_causal ? row + 1 : elo + p.ext_block, p.Te) : 0;
    const float sc = p.scale * kLog2e;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const int colh = half * 64;
    const int sw = prow & 7;
    int xc = 0;  // exchange counter (double-buffered slots)
    auto exchange = [&](float mine) -> float {
      float* slot = s_xchg[xc & 1][0];
      ++xc;
      slot[half * BM + prow] = mine;
      asm volatile("bar.sync %0, 64;" ::"r"(1 + quarter) : "memory");
      return slot[(half ^ 1) * BM + prow];
    };

    // O accumulates in TMEM over the tiles.  `m` is the reference maximum the exponentials are
    // taken against; it follows the running row maximum lazily: only when a tile's maximum
    // exceeds it by more than kRescaleLog2 (or it is still -inf) is it moved and the TMEM row
    // rescaled, so probabilities stay below 2^kRescaleLog2 and most tiles skip the rescale.
    constexpr float kRescaleLog2 = 8.f;
    float m = -INFINITY, l = 0.f;  // l: partial sum over this thread's keys
    bool ok = true;
    const uint32_t tmem_o = lane_base + 2 * BN + colh;

    for (int t = 0; t < n_tiles; ++t) {
      if (ok) ok = mbar_wait(smem_addr(&bar_s_full[t & 1]), (t >> 1) & 1, status, kTimeoutSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      fence_after_sync();
      const uint32_t tmem_s = lane_base + (t & 1) * BN + colh;
      const bool ext = t >= n_ctx;  // the tile of the query tile's own extra rows
      const int key0 = (ext ? q0 : (j0 + t) * BN) + colh;
      const int tlo = ext ? elo : lo, thi = ext ? ehi : hi;
      uint32_t r[2][32];
#pragma unroll
      for (int c = 0; c < 2; ++c) tmem_ld32(tmem_s + c * 32, r[c]);
      tmem_ld_wait();
      // keys that every row of the warp sees need no per-element test
      const bool full = __all_sync(0xffffffffu, tlo <= key0 && thi >= key0 + 64);
      if (!full) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + c * 32 + i;
            if (key < tlo || key >= thi) r[c][i] = 0xff800000u;  // -inf
          }
      }
      float cmax[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // independent chains
#pragma unroll
      for (int i = 0; i < 32; i += 2)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          cmax[2 * c] = fmaxf(cmax[2 * c], __uint_as_float(r[c][i]));
          cmax[2 * c + 1] = fmaxf(cmax[2 * c + 1], __uint_as_float(r[c][i + 1]));
        }
      const float hmax = fmaxf(fmaxf(cmax[0], cmax[1]), fmaxf(cmax[2], cmax[3]));
      const float tmax = fmaxf(hmax, exchange(hmax)) * sc;  // sc > 0
      const bool move = tmax > m + kRescaleLog2 || (m == -INFINITY && tmax > -INFINITY);
      const float m_new = move ? tmax : m;
      const float alpha = move ? ex2(m - m_new) : 1.f;  // m = -inf: 0
      const float m_sub = m_new == -INFINITY ? 0.f : m_new;
      float csum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < 32; i += 2)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float p0 = ex2(fmaf(__uint_as_float(r[c][i]), sc, -m_sub));
          const float p1 = ex2(fmaf(__uint_as_float(r[c][i + 1]), sc, -m_sub));
          csum[2 * c] += p0;
          csum[2 * c + 1] += p1;
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(p0, p1);
          r[c][i >> 1] = *reinterpret_cast<const uint32_t*>(&h2);  // packed pairs reuse the front of the row
        }
      l = l * alpha + ((csum[0] + csum[1]) + (csum[2] + csum[3]));
      m = m_new;
      if (t > 0) {
        // the previous P.V product must have retired before O is rescaled (and, one tile on,
        // before its P block is overwritten)
        if (ok) ok = mbar_wait(smem_addr(&bar_o_full), (t - 1) & 1, status, kTimeoutSoftmax);
        ok = __all_sync(0xffffffffu, ok);
        fence_after_sync();
        if (__any_sync(0xffffffffu, move)) {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t a[32];
            tmem_ld32(tmem_o + c * 32, a);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) * alpha);
            tmem_st32(tmem_o + c * 32, a);
          }
          tmem_st_wait();
        }
      }
      // P goes to TMEM as the A operand of the P.V product: key k of the row sits in the
      // 16-bit half (k & 1) of column k / 2 of the tile's P block; this thread's 64 keys are
      // 32 columns
      {
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          pk[i] = r[0][i];
          pk[16 + i] = r[1][i];
        }
        tmem_st32(lane_base + 3 * BN + (t & 1) * (BN / 2) + half * 32, pk);
        tmem_st_wait();
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_addr(&bar_p_ready));
    }

    // this thread's 64 columns of the finished output row come back into registers
    float o[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) o[i] = 0.f;
    if (n_tiles > 0) {
      if (ok) ok = mbar_wait(smem_addr(&bar_o_full), (n_tiles - 1) & 1, status, kTimeoutSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      fence_after_sync();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t a[32];
        tmem_ld32(tmem_o + c * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = __uint_as_float(a[i]);
      }
      fence_before_sync();
    }

    // individually addressed extra keys of the row: each thread of the pair takes 64 of the
    // 128 dimensions of q.k (q from the shared-memory tile), the halves meet through the
    // exchange slots; the extra's probability is counted in the first thread's partial sum
    if (p.E > 0) {
      if (ok) ok = mbar_wait(smem_addr(&bar_q), 0, status, kTimeoutSoftmax);
      ok = __all_sync(0xffffffffu, ok);
      const unsigned char* q_row = q_s + half * SUB_BYTES + prow * 128;
      // rows of the extra K / V tensors come in through a per-warp staging area (the K / V
      // stages, idle once the tile loop has drained): 8 lanes fetch the 128 bytes of one row's
      // half, 4 rows per instruction, instead of every lane walking its own row
      unsigned char* stage = k_s + (warp - 2) * 8192;
      const int lsw = lane & 7;
      for (int e = 0; e < p.E; ++e) {
        const int idx = row_ok ? p.ext_idx[(int64_t)row * p.E + e] : -1;
        const bool valid = idx >= 0 && idx < p.Te;
        const int idc = valid ? idx : 0;
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
        bf16x8 kreg[8], vreg[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) kreg[c] = *reinterpret_cast<const bf16x8*>(stage + lane * 128 + ((c ^ lsw) << 4));
#pragma unroll
        for (int c = 0; c < 8; ++c) vreg[c] = *reinterpret_cast<const bf16x8*>(stage + 4096 + lane * 128 + ((c ^ lsw) << 4));
        float d4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float a[8], b[8];
          unpack8(*reinterpret_cast<const bf16x8*>(q_row + ((c ^ sw) << 4)), a);
          unpack8(kreg[c], b);
#pragma unroll
          for (int i = 0; i < 8; ++i) d4[i & 3] = fmaf(a[i], b[i], d4[i & 3]);
        }
        const float part = (d4[0] + d4[1]) + (d4[2] + d4[3]);
        const float other = exchange(part);
        const float sv = valid ? (part + other) * sc : -INFINITY;
        const float m_new = fmaxf(m, sv);
        const float m_sub = m_new == -INFINITY ? 0.f : m_new;
        const float alpha = m_new == -INFINITY ? 1.f : ex2(m - m_sub), pe = ex2(sv - m_sub);
        l = l * alpha + (half == 0 ? pe : 0.f);
        m = m_new;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float b[8];
          unpack8(vreg[c], b);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[c * 8 + i] = fmaf(pe, b[i], o[c * 8 + i] * alpha);
        }
      }
    }

    const float l_all = l + exchange(l);
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    if (ok && row_ok && half == 0) p.lse2[(int64_t)h * p.Tq + row] = l_all > 0.f ? m + log2f(l_all) : INFINITY;
    if (__all_sync(0xffffffffu, ok)) {
      // whole rows through the warp's staging area (the K / V stages are idle by now)
      const int warp_row0 = q0 + quarter * 32;
      store_rows64_bf16(k_s + (warp - 2) * 8192, o, inv, p.out + (int64_t)warp_row0 * p.o_rs + h * HD + colh, p.o_rs, p.Tq - warp_row0, lane);
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
  CUtensorMap map_ke = map_k, map_ve = map_v;
  if (p.ext_block > 0) {
    if (p.E != 0 || BM % p.ext_block != 0 || p.ke == nullptr || p.ve == nullptr) return -4;
    rc = tc::make_map_bf16(&map_ke, p.ke, p.Te, (int64_t)p.nkv * HD, p.ke_rs, BN);
    if (rc) return rc;
    rc = tc::make_map_bf16(&map_ve, p.ve, p.Te, (int64_t)p.nkv * HD, p.ve_rs, BN);
    if (rc) return rc;
  }
  constexpr int smem_bytes = 5 * TILE_BYTES + 1024;
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(attn_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return -2;
    configured.mark();
  }
  dim3 grid(p.nh, (p.Tq + BM - 1) / BM);
  count_launch(1);
  attn_fwd_tc_kernel<<<grid, THREADS, smem_bytes, stream>>>(map_q, map_k, map_v, map_ke, map_ve, p, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace sb200
