// Masked attention for draft-model training (forward and backward).
//
// Mask model.  Query row i may attend to
//   * the contiguous interval [lo[i], hi[i]) of a context K/V tensor, and
//   * up to E individually addressed rows extra_idx[i, 0..E) of a second
//     ("extra") K/V tensor (-1 = unused slot).
// Causal / same-document / sliding-window masks are intervals; the diagonal keys
// of EAGLE-3's training-time-test passes, the same-rollout keys of P-EAGLE and
// the in-block keys of DFlash are the extras.  The KV tile range of a query tile
// comes straight from min(lo) / max(hi) of its rows, so there is no separate
// block-mask object to build.
//
// Kernel structure (FlashAttention-2 style on mma.sync m16n8k16 bf16, fp32
// accumulation, online softmax in the log2 domain):
//   forward : grid (q tiles of 64, heads); 4 warps x 16 rows; K/V tiles of 64 keys
//             double-buffered with cp.async; extras handled after the tile loop as
//             per-row dot products that reuse the accumulator register layout.
//   backward: dQ kernel (grid like forward; also produces D = rowsum(dO*O) and the
//             extra keys' dK/dV via fp32 atomics), and a dK/dV kernel (grid
//             (kv tiles, kv heads), loops over the group's query heads and the
//             query tiles that can see the kv tile).
// GQA: query head h reads kv head h / (nh / nkv).  Head dims 64 and 128.
#include "attention_params.h"
#include "mma_utils.cuh"

namespace sb200 {

constexpr int kBM = 64;   // query rows per CTA
constexpr int kBN = 64;   // keys per tile
constexpr int kAttnThreads = 128;
constexpr float kLog2e = 1.4426950408889634f;


template <int HD>
struct SmemLayout {
  static constexpr int LD = HD + 8;  // +16 B per row: conflict-free ldmatrix
  static constexpr int kTile = kBN * LD;
};

// Load a [64, HD] tile (rows row0.. of a strided [rows_total, *] tensor at column offset col0)
// into smem with cp.async; rows >= rows_total are zero-filled.
template <int HD>
__device__ __forceinline__ void load_tile_async(__nv_bfloat16* smem, const __nv_bfloat16* g,
                                                int64_t row_stride, int row0, int rows_total,
                                                int col0) {
  constexpr int LD = SmemLayout<HD>::LD;
  constexpr int kChunksPerRow = HD / 8;
  constexpr int kChunks = 64 * kChunksPerRow;
#pragma unroll
  for (int c = threadIdx.x; c < kChunks; c += kAttnThreads) {
    const int r = c / kChunksPerRow;
    const int cc = (c % kChunksPerRow) << 3;
    const int row = row0 + r;
    const bool ok = row < rows_total;
    const __nv_bfloat16* src = g + (int64_t)(ok ? row : 0) * row_stride + col0 + cc;
    cp_async16(smem + r * LD + cc, src, ok);
  }
}

template <int HD>
__global__ void __launch_bounds__(kAttnThreads)
attn_fwd_kernel(const AttnParams p) {
  constexpr int LD = SmemLayout<HD>::LD;
  constexpr int kTile = SmemLayout<HD>::kTile;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ks = Qs + kTile;      // 2 buffers
  __nv_bfloat16* Vs = Ks + 2 * kTile;  // 2 buffers
  __shared__ int s_range[2];

  // late query tiles see the most keys under a causal mask: hand them out first
  const int tile_m = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
  const int kvh = h / (p.nh / p.nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = tile_m * kBM;

  load_tile_async<HD>(Qs, p.q, p.q_rs, row0, p.Tq, h * HD);
  cp_async_commit();

  // rows owned by this thread inside the CTA tile: r_a = 16*warp + g, r_b = r_a + 8
  const int ra = row0 + warp * 16 + g, rb = ra + 8;
  const int lo_a = ra < p.Tq ? p.lo[ra] : 0x7fffffff, hi_a = ra < p.Tq ? min(p.hi[ra], p.Tc) : 0;
  const int lo_b = rb < p.Tq ? p.lo[rb] : 0x7fffffff, hi_b = rb < p.Tq ? min(p.hi[rb], p.Tc) : 0;
  // warp range and CTA range of keys
  int wlo = min(hi_a > lo_a ? lo_a : 0x7fffffff, hi_b > lo_b ? lo_b : 0x7fffffff);
  int whi = max(hi_a > lo_a ? hi_a : 0, hi_b > lo_b ? hi_b : 0);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    wlo = min(wlo, __shfl_xor_sync(0xffffffffu, wlo, o));
    whi = max(whi, __shfl_xor_sync(0xffffffffu, whi, o));
  }
  if (threadIdx.x == 0) {
    s_range[0] = 0x7fffffff;
    s_range[1] = 0;
  }
  __syncthreads();
  if (lane == 0) {
    atomicMin(&s_range[0], wlo);
    atomicMax(&s_range[1], whi);
  }
  __syncthreads();
  const int c_lo = s_range[0], c_hi = s_range[1];
  const int j0 = c_hi > c_lo ? c_lo / kBN : 0;
  const int j1 = c_hi > c_lo ? (c_hi + kBN - 1) / kBN : 0;

  float o_acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  const float sc = p.scale * kLog2e;

  if (j0 < j1) {
    load_tile_async<HD>(Ks, p.k, p.k_rs, j0 * kBN, p.Tc, kvh * HD);
    load_tile_async<HD>(Vs, p.v, p.v_rs, j0 * kBN, p.Tc, kvh * HD);
  }
  cp_async_commit();

  for (int j = j0; j < j1; ++j) {
    const int buf = (j - j0) & 1;
    if (j + 1 < j1) {
      load_tile_async<HD>(Ks + (buf ^ 1) * kTile, p.k, p.k_rs, (j + 1) * kBN, p.Tc, kvh * HD);
      load_tile_async<HD>(Vs + (buf ^ 1) * kTile, p.v, p.v_rs, (j + 1) * kBN, p.Tc, kvh * HD);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int col0 = j * kBN;
    if (wlo < col0 + kBN && whi > col0) {  // this warp's rows can see this tile
      const __nv_bfloat16* Kt = Ks + buf * kTile;
      const __nv_bfloat16* Vt = Vs + buf * kTile;
      float s[kBN / 8][4];
#pragma unroll
      for (int i = 0; i < kBN / 8; ++i)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) s[i][jj] = 0.f;
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t a[4];
        ldmatrix_x4(a, lda_addr(Qs, LD, warp * 16, kk * 16, lane));
#pragma unroll
        for (int n2 = 0; n2 < kBN / 16; ++n2) {
          uint32_t b[4];
          ldmatrix_x4(b, ldb_nk_addr(Kt, LD, n2 * 16, kk * 16, lane));
          mma_16816(s[2 * n2], a, b[0], b[1]);
          mma_16816(s[2 * n2 + 1], a, b[2], b[3]);
        }
      }
      // mask, scale, row max
      float mx_a = -INFINITY, mx_b = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < kBN / 8; ++nt) {
        const int c = col0 + nt * 8 + 2 * t;
        s[nt][0] = (c >= lo_a && c < hi_a) ? s[nt][0] * sc : -INFINITY;
        s[nt][1] = (c + 1 >= lo_a && c + 1 < hi_a) ? s[nt][1] * sc : -INFINITY;
        s[nt][2] = (c >= lo_b && c < hi_b) ? s[nt][2] * sc : -INFINITY;
        s[nt][3] = (c + 1 >= lo_b && c + 1 < hi_b) ? s[nt][3] * sc : -INFINITY;
        mx_a = fmaxf(mx_a, fmaxf(s[nt][0], s[nt][1]));
        mx_b = fmaxf(mx_b, fmaxf(s[nt][2], s[nt][3]));
      }
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
      mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
      mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
      const float mn_a = fmaxf(m_a, mx_a), mn_b = fmaxf(m_b, mx_b);
      const float mu_a = mn_a == -INFINITY ? 0.f : mn_a, mu_b = mn_b == -INFINITY ? 0.f : mn_b;
      const float al_a = exp2f(m_a - mu_a), al_b = exp2f(m_b - mu_b);
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
      for (int nt = 0; nt < kBN / 8; ++nt) {
        s[nt][0] = exp2f(s[nt][0] - mu_a);
        s[nt][1] = exp2f(s[nt][1] - mu_a);
        s[nt][2] = exp2f(s[nt][2] - mu_b);
        s[nt][3] = exp2f(s[nt][3] - mu_b);
        sum_a += s[nt][0] + s[nt][1];
        sum_b += s[nt][2] + s[nt][3];
      }
      l_a = l_a * al_a + sum_a;  // per-thread partial; quad-reduced at the end
      l_b = l_b * al_b + sum_b;
      m_a = mn_a;
      m_b = mn_b;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        o_acc[i][0] *= al_a;
        o_acc[i][1] *= al_a;
        o_acc[i][2] *= al_b;
        o_acc[i][3] *= al_b;
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < kBN / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int n2 = 0; n2 < HD / 16; ++n2) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, ldb_kn_addr(Vt, LD, kk * 16, n2 * 16, lane));
          mma_16816(o_acc[2 * n2], a, b[0], b[1]);
          mma_16816(o_acc[2 * n2 + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // quad-reduce the partial row sums
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

  // extra keys: per-row dot products in the accumulator layout (cols 8*nt + 2t, +1)
  // (rows of different quads take different branches below, so shuffles name the quad only)
  const unsigned qmask = 0xFu << (lane & 28);
  if (p.E > 0 && p.ext_idx != nullptr) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = half ? rb : ra;
      const int rl = warp * 16 + g + half * 8;
      float& m_r = half ? m_b : m_a;
      float& l_r = half ? l_b : l_a;
#pragma unroll 1
      for (int e = 0; e < p.E; ++e) {
        const int idx = r < p.Tq ? p.ext_idx[(int64_t)r * p.E + e] : -1;  // same for the 4 lanes of a quad
        if (idx < 0 || idx >= p.Te) continue;
        const __nv_bfloat16* kr = p.ke + (int64_t)idx * p.ke_rs + kvh * HD;
        const __nv_bfloat16* vr = p.ve + (int64_t)idx * p.ve_rs + kvh * HD;
        float dot = 0.f;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) {
          const int c = nt * 8 + 2 * t;
          const float2 kv2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kr + c));
          const float2 q2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Qs + rl * LD + c));
          dot += kv2.x * q2.x + kv2.y * q2.y;
        }
        dot += __shfl_xor_sync(qmask, dot, 1);
        dot += __shfl_xor_sync(qmask, dot, 2);
        const float sv = dot * sc;
        const float mn = fmaxf(m_r, sv);
        const float al = exp2f(m_r - mn);
        const float pe = exp2f(sv - mn);
        l_r = l_r * al + pe;
        m_r = mn;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) {
          const int c = nt * 8 + 2 * t;
          const float2 v2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vr + c));
          o_acc[nt][half * 2 + 0] = o_acc[nt][half * 2 + 0] * al + pe * v2.x;
          o_acc[nt][half * 2 + 1] = o_acc[nt][half * 2 + 1] * al + pe * v2.y;
        }
      }
    }
  }

  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
  if (ra < p.Tq) {
    __nv_bfloat16* orow = p.out + (int64_t)ra * p.o_rs + h * HD;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt)
      *reinterpret_cast<__nv_bfloat162*>(orow + nt * 8 + 2 * t) =
          __floats2bfloat162_rn(o_acc[nt][0] * inv_a, o_acc[nt][1] * inv_a);
    if (t == 0) p.lse2[(int64_t)h * p.Tq + ra] = l_a > 0.f ? m_a + log2f(l_a) : INFINITY;
  }
  if (rb < p.Tq) {
    __nv_bfloat16* orow = p.out + (int64_t)rb * p.o_rs + h * HD;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt)
      *reinterpret_cast<__nv_bfloat162*>(orow + nt * 8 + 2 * t) =
          __floats2bfloat162_rn(o_acc[nt][2] * inv_b, o_acc[nt][3] * inv_b);
    if (t == 0) p.lse2[(int64_t)h * p.Tq + rb] = l_b > 0.f ? m_b + log2f(l_b) : INFINITY;
  }
}

// ----------------------------------------------------------------------------------------
// Backward, part 1: dQ (and delta, and the extra keys' dK / dV).
template <int HD>
__global__ void __launch_bounds__(kAttnThreads)
attn_bwd_dq_kernel(const AttnParams p) {
  constexpr int LD = SmemLayout<HD>::LD;
  constexpr int kTile = SmemLayout<HD>::kTile;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* dOs = Qs + kTile;
  __nv_bfloat16* Ks = dOs + kTile;     // 2 buffers
  __nv_bfloat16* Vs = Ks + 2 * kTile;  // 2 buffers
  __shared__ int s_range[2];

  // late query tiles see the most keys under a causal mask: hand them out first
  const int tile_m = gridDim.x - 1 - blockIdx.x, h = blockIdx.y;
  const int kvh = h / (p.nh / p.nkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int row0 = tile_m * kBM;

  load_tile_async<HD>(Qs, p.q, p.q_rs, row0, p.Tq, h * HD);
  load_tile_async<HD>(dOs, p.dout, p.do_rs, row0, p.Tq, h * HD);
  cp_async_commit();

  const int ra = row0 + warp * 16 + g, rb = ra + 8;
  const int lo_a = ra < p.Tq ? p.lo[ra] : 0x7fffffff, hi_a = ra < p.Tq ? min(p.hi[ra], p.Tc) : 0;
  const int lo_b = rb < p.Tq ? p.lo[rb] : 0x7fffffff, hi_b = rb < p.Tq ? min(p.hi[rb], p.Tc) : 0;
  const float lse_a = ra < p.Tq ? p.lse2[(int64_t)h * p.Tq + ra] : INFINITY;
  const float lse_b = rb < p.Tq ? p.lse2[(int64_t)h * p.Tq + rb] : INFINITY;
  int wlo = min(hi_a > lo_a ? lo_a : 0x7fffffff, hi_b > lo_b ? lo_b : 0x7fffffff);
  int whi = max(hi_a > lo_a ? hi_a : 0, hi_b > lo_b ? hi_b : 0);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    wlo = min(wlo, __shfl_xor_sync(0xffffffffu, wlo, o));
    whi = max(whi, __shfl_xor_sync(0xffffffffu, whi, o));
  }
  if (threadIdx.x == 0) {
    s_range[0] = 0x7fffffff;
    s_range[1] = 0;
  }
  __syncthreads();
  if (lane == 0) {
    atomicMin(&s_range[0], wlo);
    atomicMax(&s_range[1], whi);
  }
  __syncthreads();
  const int c_lo = s_range[0], c_hi = s_range[1];
  const int j0 = c_hi > c_lo ? c_lo / kBN : 0;
  const int j1 = c_hi > c_lo ? (c_hi + kBN - 1) / kBN : 0;

  if (j0 < j1) {
    load_tile_async<HD>(Ks, p.k, p.k_rs, j0 * kBN, p.Tc, kvh * HD);
    load_tile_async<HD>(Vs, p.v, p.v_rs, j0 * kBN, p.Tc, kvh * HD);
  }
  cp_async_commit();
  cp_async_wait<1>();  // Q and dO have landed
  __syncthreads();

  // delta = rowsum(dO * O) for the two rows of this thread (quad-reduced)
  float d_a = 0.f, d_b = 0.f;
  {
    const int rla = warp * 16 + g, rlb = rla + 8;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt) {
      const int c = nt * 8 + 2 * t;
      if (ra < p.Tq) {
        const float2 o2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p.out + (int64_t)ra * p.o_rs + h * HD + c));
        const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dOs + rla * LD + c));
        d_a += o2.x * g2.x + o2.y * g2.y;
      }
      if (rb < p.Tq) {
        const float2 o2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p.out + (int64_t)rb * p.o_rs + h * HD + c));
        const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dOs + rlb * LD + c));
        d_b += o2.x * g2.x + o2.y * g2.y;
      }
    }
    d_a += __shfl_xor_sync(0xffffffffu, d_a, 1);
    d_a += __shfl_xor_sync(0xffffffffu, d_a, 2);
    d_b += __shfl_xor_sync(0xffffffffu, d_b, 1);
    d_b += __shfl_xor_sync(0xffffffffu, d_b, 2);
    if (t == 0) {
      if (ra < p.Tq) p.delta[(int64_t)h * p.Tq + ra] = d_a;
      if (rb < p.Tq) p.delta[(int64_t)h * p.Tq + rb] = d_b;
    }
  }

  float dq_acc[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) dq_acc[i][j] = 0.f;
  const float sc = p.scale * kLog2e;

  for (int j = j0; j < j1; ++j) {
    const int buf = (j - j0) & 1;
    if (j + 1 < j1) {
      load_tile_async<HD>(Ks + (buf ^ 1) * kTile, p.k, p.k_rs, (j + 1) * kBN, p.Tc, kvh * HD);
      load_tile_async<HD>(Vs + (buf ^ 1) * kTile, p.v, p.v_rs, (j + 1) * kBN, p.Tc, kvh * HD);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int col0 = j * kBN;
    if (wlo < col0 + kBN && whi > col0) {
      const __nv_bfloat16* Kt = Ks + buf * kTile;
      const __nv_bfloat16* Vt = Vs + buf * kTile;
      float s[kBN / 8][4], dp[kBN / 8][4];
#pragma unroll
      for (int i = 0; i < kBN / 8; ++i)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          s[i][jj] = 0.f;
          dp[i][jj] = 0.f;
        }
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t a[4], ad[4];
        ldmatrix_x4(a, lda_addr(Qs, LD, warp * 16, kk * 16, lane));
        ldmatrix_x4(ad, lda_addr(dOs, LD, warp * 16, kk * 16, lane));
#pragma unroll
        for (int n2 = 0; n2 < kBN / 16; ++n2) {
          uint32_t b[4], bv[4];
          ldmatrix_x4(b, ldb_nk_addr(Kt, LD, n2 * 16, kk * 16, lane));
          ldmatrix_x4(bv, ldb_nk_addr(Vt, LD, n2 * 16, kk * 16, lane));
          mma_16816(s[2 * n2], a, b[0], b[1]);
          mma_16816(s[2 * n2 + 1], a, b[2], b[3]);
          mma_16816(dp[2 * n2], ad, bv[0], bv[1]);
          mma_16816(dp[2 * n2 + 1], ad, bv[2], bv[3]);
        }
      }
#pragma unroll
      for (int nt = 0; nt < kBN / 8; ++nt) {
        const int c = col0 + nt * 8 + 2 * t;
        const float p0 = (c >= lo_a && c < hi_a) ? exp2f(s[nt][0] * sc - lse_a) : 0.f;
        const float p1 = (c + 1 >= lo_a && c + 1 < hi_a) ? exp2f(s[nt][1] * sc - lse_a) : 0.f;
        const float p2 = (c >= lo_b && c < hi_b) ? exp2f(s[nt][2] * sc - lse_b) : 0.f;
        const float p3 = (c + 1 >= lo_b && c + 1 < hi_b) ? exp2f(s[nt][3] * sc - lse_b) : 0.f;
        s[nt][0] = p0 * (dp[nt][0] - d_a);
        s[nt][1] = p1 * (dp[nt][1] - d_a);
        s[nt][2] = p2 * (dp[nt][2] - d_b);
        s[nt][3] = p3 * (dp[nt][3] - d_b);
      }
#pragma unroll
      for (int kk = 0; kk < kBN / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int n2 = 0; n2 < HD / 16; ++n2) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, ldb_kn_addr(Kt, LD, kk * 16, n2 * 16, lane));
          mma_16816(dq_acc[2 * n2], a, b[0], b[1]);
          mma_16816(dq_acc[2 * n2 + 1], a, b[2], b[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  const unsigned qmask = 0xFu << (lane & 28);
  if (p.E > 0 && p.ext_idx != nullptr) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = half ? rb : ra;
      const int rl = warp * 16 + g + half * 8;
      const float lse_r = half ? lse_b : lse_a;
      const float d_r = half ? d_b : d_a;
#pragma unroll 1
      for (int e = 0; e < p.E; ++e) {
        const int idx = r < p.Tq ? p.ext_idx[(int64_t)r * p.E + e] : -1;
        if (idx < 0 || idx >= p.Te) continue;
        const __nv_bfloat16* kr = p.ke + (int64_t)idx * p.ke_rs + kvh * HD;
        const __nv_bfloat16* vr = p.ve + (int64_t)idx * p.ve_rs + kvh * HD;
        float dot = 0.f, dpe = 0.f;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) {
          const int c = nt * 8 + 2 * t;
          const float2 k2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kr + c));
          const float2 v2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(vr + c));
          const float2 q2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Qs + rl * LD + c));
          const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dOs + rl * LD + c));
          dot += k2.x * q2.x + k2.y * q2.y;
          dpe += v2.x * g2.x + v2.y * g2.y;
        }
        dot += __shfl_xor_sync(qmask, dot, 1);
        dot += __shfl_xor_sync(qmask, dot, 2);
        dpe += __shfl_xor_sync(qmask, dpe, 1);
        dpe += __shfl_xor_sync(qmask, dpe, 2);
        const float pe = exp2f(dot * sc - lse_r);
        const float ds = pe * (dpe - d_r);
        float* dkr = p.dke + ((int64_t)idx * p.nkv + kvh) * HD;
        float* dvr = p.dve + ((int64_t)idx * p.nkv + kvh) * HD;
#pragma unroll
        for (int nt = 0; nt < HD / 8; ++nt) {
          const int c = nt * 8 + 2 * t;
          const float2 k2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(kr + c));
          const float2 q2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(Qs + rl * LD + c));
          const float2 g2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(dOs + rl * LD + c));
          dq_acc[nt][half * 2 + 0] += ds * k2.x;
          dq_acc[nt][half * 2 + 1] += ds * k2.y;
          atomicAdd(dkr + c, ds * p.scale * q2.x);
          atomicAdd(dkr + c + 1, ds * p.scale * q2.y);
          atomicAdd(dvr + c, pe * g2.x);
          atomicAdd(dvr + c + 1, pe * g2.y);
        }
      }
    }
  }

  if (ra < p.Tq) {
    __nv_bfloat16* row = p.dq + (int64_t)ra * p.dq_rs + h * HD;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt)
      *reinterpret_cast<__nv_bfloat162*>(row + nt * 8 + 2 * t) =
          __floats2bfloat162_rn(dq_acc[nt][0] * p.scale, dq_acc[nt][1] * p.scale);
  }
  if (rb < p.Tq) {
    __nv_bfloat16* row = p.dq + (int64_t)rb * p.dq_rs + h * HD;
#pragma unroll
    for (int nt = 0; nt < HD / 8; ++nt)
      *reinterpret_cast<__nv_bfloat162*>(row + nt * 8 + 2 * t) =
          __floats2bfloat162_rn(dq_acc[nt][2] * p.scale, dq_acc[nt][3] * p.scale);
  }
}

// For every kv tile: the range of query rows whose interval touches it.  One CTA per
// tile scans all query rows (coalesced) and reduces min / max in the block.
__global__ void __launch_bounds__(256)
kv_tile_range_kernel(const int* __restrict__ lo, const int* __restrict__ hi, int Tq,
                     int Tc, int* __restrict__ qmin, int* __restrict__ qmax) {
  __shared__ int smin[8], smax[8];
  const int k0 = blockIdx.x * kBN, k1 = k0 + kBN;
  int mn = 0x7fffffff, mx = 0;
  for (int i = threadIdx.x; i < Tq; i += blockDim.x) {
    const int l = lo[i], h = min(hi[i], Tc);
    if (l >= 0 && h > l && l < k1 && h > k0) {
      mn = min(mn, i);
      mx = max(mx, i + 1);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  if ((threadIdx.x & 31) == 0) {
    smin[threadIdx.x >> 5] = mn;
    smax[threadIdx.x >> 5] = mx;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
      mn = min(mn, smin[w]);
      mx = max(mx, smax[w]);
    }
    qmin[blockIdx.x] = mn;
    qmax[blockIdx.x] = mx;
  }
}

// ----------------------------------------------------------------------------------------
// Backward, part 2: dK / dV of the context keys.  One CTA per (query head, kv tile); each
// warp owns 16 keys and accumulates over the query tiles that can see them.  Under a
// causal mask the work per kv tile falls linearly with its index, so the grid is ordered
// heaviest tile first and split by query head (1..n_qt iterations per CTA instead of
// group * n_qt): the tail of light CTAs fills the SMs the heavy ones leave.  With grouped
// queries the CTAs of a group write fp32 partials that dkv_reduce_kernel sums in fixed
// order (deterministic), otherwise the bf16 result is written directly.
// At head dim 256 a warp's dK and dV rows would need 256 fp32 accumulators per thread (they spilled: 1.6 KB of
// stores and 2 KB of loads per thread and tile): the head dim of the *outputs* is split over blockIdx.z, each CTA
// recomputes the score tile over the whole head dim and accumulates kDkvCols<HD> of the dK / dV columns.
template <int HD>
constexpr int kDkvCols = HD > 128 ? 128 : HD;

template <int HD>
__global__ void __launch_bounds__(kAttnThreads)
attn_bwd_dkv_kernel(const AttnParams p) {
  constexpr int HDO = kDkvCols<HD>;
  const int c0 = blockIdx.z * HDO;  // first dK / dV column of this CTA
  constexpr int LD = SmemLayout<HD>::LD;
  constexpr int kTile = SmemLayout<HD>::kTile;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Kt = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Vt = Kt + kTile;
  __nv_bfloat16* Qs = Vt + kTile;       // 2 buffers
  __nv_bfloat16* dOs = Qs + 2 * kTile;  // 2 buffers
  float* rowf = reinterpret_cast<float*>(dOs + 2 * kTile);  // [2][2][64]: lse2, delta
  int* rowi = reinterpret_cast<int*>(rowf + 2 * 2 * kBM);   // [2][2][64]: lo, hi

  const int hq = blockIdx.x, tile_n = blockIdx.y;
  const int group = p.nh / p.nkv;
  const int kvh = hq / group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int key0 = tile_n * kBN;
  const int ka = key0 + warp * 16 + g, kb = ka + 8;  // keys owned by this thread's accumulator rows

  const int qmin = p.tile_qmin[tile_n], qmax = p.tile_qmax[tile_n];
  const int i0 = qmax > qmin ? qmin / kBM : 0;
  const int i1 = qmax > qmin ? (qmax + kBM - 1) / kBM : 0;
  const int n_iter = i1 - i0;

  load_tile_async<HD>(Kt, p.k, p.k_rs, key0, p.Tc, kvh * HD);
  load_tile_async<HD>(Vt, p.v, p.v_rs, key0, p.Tc, kvh * HD);
  cp_async_commit();

  auto issue = [&](int it, int buf) {
    const int qrow0 = (i0 + it) * kBM;
    load_tile_async<HD>(Qs + buf * kTile, p.q, p.q_rs, qrow0, p.Tq, hq * HD);
    load_tile_async<HD>(dOs + buf * kTile, p.dout, p.do_rs, qrow0, p.Tq, hq * HD);
    if (threadIdx.x < kBM) {
      const int r = qrow0 + threadIdx.x;
      const bool ok = r < p.Tq;
      rowf[(buf * 2 + 0) * kBM + threadIdx.x] = ok ? p.lse2[(int64_t)hq * p.Tq + r] : INFINITY;
      rowf[(buf * 2 + 1) * kBM + threadIdx.x] = ok ? p.delta[(int64_t)hq * p.Tq + r] : 0.f;
      rowi[(buf * 2 + 0) * kBM + threadIdx.x] = ok ? p.lo[r] : 0x7fffffff;
      rowi[(buf * 2 + 1) * kBM + threadIdx.x] = ok ? min(p.hi[r], p.Tc) : 0;
    }
  };

  float dk_acc[HDO / 8][4], dv_acc[HDO / 8][4];
#pragma unroll
  for (int i = 0; i < HDO / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      dk_acc[i][j] = 0.f;
      dv_acc[i][j] = 0.f;
    }
  const float sc = p.scale * kLog2e;

  if (n_iter > 0) issue(0, 0);
  cp_async_commit();

  for (int it = 0; it < n_iter; ++it) {
    const int buf = it & 1;
    if (it + 1 < n_iter) issue(it + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* Qt = Qs + buf * kTile;
    const __nv_bfloat16* dOt = dOs + buf * kTile;
    const float* lse_s = rowf + (buf * 2 + 0) * kBM;
    const float* del_s = rowf + (buf * 2 + 1) * kBM;
    const int* lo_s = rowi + (buf * 2 + 0) * kBM;
    const int* hi_s = rowi + (buf * 2 + 1) * kBM;
    // does any query of this tile see any of this warp's 16 keys?
    int tlo = min(lo_s[lane], lo_s[lane + 32]);
    int thi = max(hi_s[lane], hi_s[lane + 32]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      tlo = min(tlo, __shfl_xor_sync(0xffffffffu, tlo, o));
      thi = max(thi, __shfl_xor_sync(0xffffffffu, thi, o));
    }
    const int wk0 = key0 + warp * 16;
    if (tlo < wk0 + 16 && thi > wk0) {
      float st[kBM / 8][4], dpt[kBM / 8][4];
#pragma unroll
      for (int i = 0; i < kBM / 8; ++i)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          st[i][jj] = 0.f;
          dpt[i][jj] = 0.f;
        }
      // S^T = K Q^T, dP^T = V dO^T   (rows: keys, cols: queries)
#pragma unroll
      for (int kk = 0; kk < HD / 16; ++kk) {
        uint32_t a[4], av[4];
        ldmatrix_x4(a, lda_addr(Kt, LD, warp * 16, kk * 16, lane));
        ldmatrix_x4(av, lda_addr(Vt, LD, warp * 16, kk * 16, lane));
#pragma unroll
        for (int n2 = 0; n2 < kBM / 16; ++n2) {
          uint32_t b[4], bd[4];
          ldmatrix_x4(b, ldb_nk_addr(Qt, LD, n2 * 16, kk * 16, lane));
          ldmatrix_x4(bd, ldb_nk_addr(dOt, LD, n2 * 16, kk * 16, lane));
          mma_16816(st[2 * n2], a, b[0], b[1]);
          mma_16816(st[2 * n2 + 1], a, b[2], b[3]);
          mma_16816(dpt[2 * n2], av, bd[0], bd[1]);
          mma_16816(dpt[2 * n2 + 1], av, bd[2], bd[3]);
        }
      }
      // P^T and dS^T in place
#pragma unroll
      for (int nt = 0; nt < kBM / 8; ++nt) {
        const int c = nt * 8 + 2 * t;  // local query index of columns c, c+1
        const float l0 = lse_s[c], l1 = lse_s[c + 1], e0 = del_s[c], e1 = del_s[c + 1];
        const int lo0 = lo_s[c], lo1 = lo_s[c + 1], hi0 = hi_s[c], hi1 = hi_s[c + 1];
        const float p0 = (ka >= lo0 && ka < hi0) ? exp2f(st[nt][0] * sc - l0) : 0.f;
        const float p1 = (ka >= lo1 && ka < hi1) ? exp2f(st[nt][1] * sc - l1) : 0.f;
        const float p2 = (kb >= lo0 && kb < hi0) ? exp2f(st[nt][2] * sc - l0) : 0.f;
        const float p3 = (kb >= lo1 && kb < hi1) ? exp2f(st[nt][3] * sc - l1) : 0.f;
        st[nt][0] = p0;
        st[nt][1] = p1;
        st[nt][2] = p2;
        st[nt][3] = p3;
        dpt[nt][0] = p0 * (dpt[nt][0] - e0);
        dpt[nt][1] = p1 * (dpt[nt][1] - e1);
        dpt[nt][2] = p2 * (dpt[nt][2] - e0);
        dpt[nt][3] = p3 * (dpt[nt][3] - e1);
      }
      // dV += P^T dO ; dK += dS^T Q     (contraction over the 64 queries)
#pragma unroll
      for (int kk = 0; kk < kBM / 16; ++kk) {
        uint32_t ap[4], as_[4];
        ap[0] = pack_bf16(st[2 * kk][0], st[2 * kk][1]);
        ap[1] = pack_bf16(st[2 * kk][2], st[2 * kk][3]);
        ap[2] = pack_bf16(st[2 * kk + 1][0], st[2 * kk + 1][1]);
        ap[3] = pack_bf16(st[2 * kk + 1][2], st[2 * kk + 1][3]);
        as_[0] = pack_bf16(dpt[2 * kk][0], dpt[2 * kk][1]);
        as_[1] = pack_bf16(dpt[2 * kk][2], dpt[2 * kk][3]);
        as_[2] = pack_bf16(dpt[2 * kk + 1][0], dpt[2 * kk + 1][1]);
        as_[3] = pack_bf16(dpt[2 * kk + 1][2], dpt[2 * kk + 1][3]);
#pragma unroll
        for (int n2 = 0; n2 < HDO / 16; ++n2) {
          uint32_t bo[4], bq[4];
          ldmatrix_x4_trans(bo, ldb_kn_addr(dOt, LD, kk * 16, c0 + n2 * 16, lane));
          ldmatrix_x4_trans(bq, ldb_kn_addr(Qt, LD, kk * 16, c0 + n2 * 16, lane));
          mma_16816(dv_acc[2 * n2], ap, bo[0], bo[1]);
          mma_16816(dv_acc[2 * n2 + 1], ap, bo[2], bo[3]);
          mma_16816(dk_acc[2 * n2], as_, bq[0], bq[1]);
          mma_16816(dk_acc[2 * n2 + 1], as_, bq[2], bq[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  if (p.dkv_part != nullptr) {
    const int64_t plane = (int64_t)p.Tc * p.nkv * HD;
    float* base = p.dkv_part + (int64_t)(hq - kvh * group) * 2 * plane;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int key = half ? kb : ka;
      if (key >= p.Tc) continue;
      float* rk = base + ((int64_t)key * p.nkv + kvh) * HD + c0;
      float* rv = rk + plane;
#pragma unroll
      for (int nt = 0; nt < HDO / 8; ++nt) {
        *reinterpret_cast<float2*>(rk + nt * 8 + 2 * t) = make_float2(dk_acc[nt][2 * half] * p.scale, dk_acc[nt][2 * half + 1] * p.scale);
        *reinterpret_cast<float2*>(rv + nt * 8 + 2 * t) = make_float2(dv_acc[nt][2 * half], dv_acc[nt][2 * half + 1]);
      }
    }
    return;
  }
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int key = half ? kb : ka;
    if (key >= p.Tc) continue;
    __nv_bfloat16* rk = p.dk + ((int64_t)key * p.nkv + kvh) * HD + c0;
    __nv_bfloat16* rv = p.dv + ((int64_t)key * p.nkv + kvh) * HD + c0;
#pragma unroll
    for (int nt = 0; nt < HDO / 8; ++nt) {
      *reinterpret_cast<__nv_bfloat162*>(rk + nt * 8 + 2 * t) =
          __floats2bfloat162_rn(dk_acc[nt][2 * half] * p.scale, dk_acc[nt][2 * half + 1] * p.scale);
      *reinterpret_cast<__nv_bfloat162*>(rv + nt * 8 + 2 * t) = __floats2bfloat162_rn(dv_acc[nt][2 * half], dv_acc[nt][2 * half + 1]);
    }
  }
}

// Sum the per-query-head partials of a group in head order and round to bf16.
// part: [group, 2, n] fp32 with n = Tc * nkv * HD (n % 8 == 0); dk, dv: [n] bf16.
__global__ void __launch_bounds__(256)
dkv_reduce_kernel(const float* __restrict__ part, int group, int64_t n, __nv_bfloat16* __restrict__ dk, __nv_bfloat16* __restrict__ dv) {
  const int64_t nvec = n >> 3;
  for (int64_t vi = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; vi < 2 * nvec; vi += (int64_t)gridDim.x * blockDim.x) {
    const int which = vi >= nvec;
    const int64_t off = (vi - which * nvec) << 3;
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < group; ++s) {
      const float4* src = reinterpret_cast<const float4*>(part + ((int64_t)s * 2 + which) * n + off);
      const float4 a = src[0], b = src[1];
      acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
      acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
    }
    st8((which ? dv : dk) + off, pack8(acc));
  }
}

// ----------------------------------------------------------------------------------------
template <int HD>
static size_t fwd_smem() { return (size_t)5 * SmemLayout<HD>::kTile * sizeof(__nv_bfloat16); }
template <int HD>
static size_t bwd_smem() {
  return (size_t)6 * SmemLayout<HD>::kTile * sizeof(__nv_bfloat16) + 2 * 2 * kBM * (sizeof(float) + sizeof(int));
}

template <int HD>
static int launch_fwd_t(const AttnParams& p, cudaStream_t stream) {
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fwd_smem<HD>()) != cudaSuccess) return -2;
    configured.mark();
  }
  dim3 grid((p.Tq + kBM - 1) / kBM, p.nh);
  count_launch(1);
  attn_fwd_kernel<HD><<<grid, kAttnThreads, fwd_smem<HD>(), stream>>>(p);
  return 0;
}

template <int HD>
static int launch_bwd_t(const AttnParams& p, int* tile_qmin, int* tile_qmax, cudaStream_t stream) {
  static PerDeviceOnce configured;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(attn_bwd_dq_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bwd_smem<HD>()) != cudaSuccess) return -2;
    if (cudaFuncSetAttribute(attn_bwd_dkv_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bwd_smem<HD>()) != cudaSuccess) return -2;
    configured.mark();
  }
  const int n_kv_tiles = (p.Tc + kBN - 1) / kBN;
  count_launch(3);
  dim3 grid_q((p.Tq + kBM - 1) / kBM, p.nh);
  attn_bwd_dq_kernel<HD><<<grid_q, kAttnThreads, bwd_smem<HD>(), stream>>>(p);
  kv_tile_range_kernel<<<n_kv_tiles, 256, 0, stream>>>(p.lo, p.hi, p.Tq, p.Tc, tile_qmin, tile_qmax);
  dim3 grid_kv(p.nh, n_kv_tiles, HD / kDkvCols<HD>);  // x = head: all heads of the heaviest tile are dispatched first; z = output column part
  attn_bwd_dkv_kernel<HD><<<grid_kv, kAttnThreads, bwd_smem<HD>(), stream>>>(p);
  if (p.dkv_part != nullptr) {
    const int64_t n = (int64_t)p.Tc * p.nkv * HD;
    const int64_t blocks = (2 * (n >> 3) + 255) / 256;
    count_launch(1);
    dkv_reduce_kernel<<<(int)(blocks < 8 * kNumSM ? blocks : 8 * kNumSM), 256, 0, stream>>>(p.dkv_part, p.nh / p.nkv, n, p.dk, p.dv);
  }
  return 0;
}

int launch_kv_tile_range(const AttnParams& p, int* tile_qmin, int* tile_qmax, cudaStream_t stream) {
  const int n_kv_tiles = (p.Tc + kBN - 1) / kBN;
  count_launch(1);
  kv_tile_range_kernel<<<n_kv_tiles, 256, 0, stream>>>(p.lo, p.hi, p.Tq, p.Tc, tile_qmin, tile_qmax);
  return 0;
}

int launch_dkv_reduce(const AttnParams& p, cudaStream_t stream) {
  const int64_t n = (int64_t)p.Tc * p.nkv * 128;
  const int64_t blocks = (2 * (n >> 3) + 255) / 256;
  count_launch(1);
  dkv_reduce_kernel<<<(int)(blocks < 8 * kNumSM ? blocks : 8 * kNumSM), 256, 0, stream>>>(p.dkv_part, p.nh / p.nkv, n, p.dk, p.dv);
  return 0;
}

int launch_attn_fwd(const AttnParams& p, int hd, cudaStream_t stream) {
  if (p.Tq <= 0) return 0;
  if (hd == 64) return launch_fwd_t<64>(p, stream);
  if (hd == 128) return launch_fwd_t<128>(p, stream);
  if (hd == 256) return launch_fwd_t<256>(p, stream);
  return -1;
}

// tile_qmin / tile_qmax: scratch, one int per 64-key tile (fully written here).
int launch_attn_bwd(const AttnParams& p, int hd, int* tile_qmin, int* tile_qmax, cudaStream_t stream) {
  if (p.Tq <= 0) return 0;
  if (hd == 64) return launch_bwd_t<64>(p, tile_qmin, tile_qmax, stream);
  if (hd == 128) return launch_bwd_t<128>(p, tile_qmin, tile_qmax, stream);
  if (hd == 256) return launch_bwd_t<256>(p, tile_qmin, tile_qmax, stream);
  return -1;
}

}  // namespace sb200
