// bf16 GEMM on the 5th-generation tensor cores:  C[M,N] = A[M,K] * B[N,K]^T  (+ epilogue)
//
// This is the nn.Linear forward shape: both operands are K-major (row-major with K
// contiguous), the accumulator is fp32.  Structure of one persistent CTA (192 threads):
//
//   warp 0  TMA producer : cp.async.bulk.tensor (128B-swizzled boxes, no multicast) into a
//                          4-stage shared-memory ring, completion counted on mbarriers
//   warp 1  MMA issuer   : allocates all 512 TMEM columns (two 128x256 fp32 accumulators),
//                          one elected thread issues tcgen05.mma (M=128, N=256, K=16) from
//                          shared-memory descriptors and tcgen05.commit's to free ring slots
//   warps 2-5 epilogue   : tcgen05.ld the finished accumulator (each warp its own 32 TMEM
//                          lanes = 32 output rows), convert to bf16, apply the epilogue and
//                          store; the MMA warp meanwhile fills the other accumulator
//
// Tiles are walked n-major so that CTAs running at the same time share B (weight) tiles in
// L2.  Ragged M / N / K are handled by TMA zero fill and masked stores.
//
// Two kernels share this structure.  gemm_tn_kernel works on 128x256 tiles, one CTA per
// tile.  gemm_tn_2cta_kernel pairs two SMs (a cluster of two CTAs, tcgen05 cta_group::2)
// on a 256x256 tile: each CTA stages its own 128 rows of A and 128 of the tile's 256 rows
// of B (32 KB per stage instead of 48 KB, six stages instead of four), the even CTA's
// elected thread issues M=256 MMAs that read both CTAs' shared memory and write both
// CTAs' TMEM, and completion is multicast to the barriers of both CTAs.  Halving the B
// traffic per SM is what the L2-to-SM path needs to keep the tensor pipe fed.
//
// Operand layouts.  The forward product has both operands K-major (rows of A and of B run
// along the contraction).  The backward products of a linear layer do not:
//   dgrad  dX[T,in]  = dY[T,out] * W[out,in]        B is read as stored, [K, N] with N contiguous
//   wgrad  dW[out,in] (+)= dY[T,out]^T * X[T,in]    A is [K, M] with M contiguous, B is [K, N]
// The CTA-pair kernel therefore takes each operand either K-major or MN-major (template flags):
// an MN-major operand is staged by TMA as boxes of 64 MN-elements x 128 contraction rows (the
// same 16 KB, 128-byte swizzle) and described to the tensor core with an MN-major shared-memory
// descriptor plus the transpose bit of the instruction descriptor, so no operand is ever
// transposed in memory.
//
// Every wait is bounded: a thread that exhausts its poll budget records a code in the
// caller's status word and leaves its loop; the other roles then run out of budget (or
// see the status word) too, the CTA meets at the final barrier, frees its TMEM and
// returns.  Nothing traps and nothing spins forever.
#include "loss_stats.cuh"
#include "tcgen05_utils.cuh"

namespace sb200 {

namespace tc {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int kDefaultPairVariant = 3;

// kSwiGLU: the weight is the stack [gate rows | up rows] of a gated MLP (N = 2 I).  A tile pairs 128 gate columns
// with the same 128 up columns (the leader CTA loads the gate rows, its peer the up rows, so the accumulator holds
// gate in columns 0..127 and up in 128..255); the epilogue stores both halves into C[M, 2 I] (kept for the backward
// pass) and silu(gate) * up into h[M, I].
enum Epilogue : int { kStore = 0, kAccumulate = 1, kAddResidual = 2, kSwiGLU = 3 };
enum Status : int { kOk = kStatusOk, kTimeoutProducer = 1, kTimeoutMma = 2, kTimeoutEpilogue = 3 };

// Row statistics in the epilogue (the lm_head product fused with the row loss): next to
// storing the logits tile, every thread reduces its row's 256 columns of the tile, together with
// the same columns of the target logits row `row + shift`, to the online-softmax statistics of
// both and the cross term of the KL divergence, and writes them as one record of kStatWords
// floats at partial[(row * tiles_n + tile_n) * kStatWords].  A second kernel merges a row's
// records.  The statistics are taken from the bf16-rounded logits, i.e. from the values the
// backward pass reads back.
constexpr int kStatWords = 12;  // m_d z_d best_d idx_d | m_t z_t A best_t | idx_t - - -   (one record per row and 128-column half tile)
struct RowStatsOut {
  const __nv_bfloat16* targets;  // nullptr: plain GEMM
  int64_t ldt;
  int t_rows;   // rows of the target matrix
  int shift;    // logits row r pairs with target row r + shift
  float* partial;
};

// Grouped products (mixture-of-experts): rows sorted by expert, expert e owning the rows
// seg[e] .. seg[e+1] of the activation matrices, every seg[e] a multiple of 128 (the rows
// between an expert's last token and the next boundary are zero).  All sizes that depend on the
// routing are read from device memory, so the launch is fixed-shape and can be captured.
//   kGroupRows  C[r, :] = A[r, :] . B_e^T for r in expert e (forward and input gradient): tiles are
//               enumerated per expert through tile_start (prefix sum of ceil(rows_e / 256) * tiles_n);
//               B is the stack of the experts' matrices ([E * N, K] K-major or [E * K, N] MN-major).
//   kGroupK     C_e (+)= A[seg_e, :]^T . B[seg_e, :] (weight gradient): the contraction runs over
//               expert e's rows, C is the stack [E * M, N]; an expert without rows yields zeros.
enum GroupMode : int { kGroupNone = 0, kGroupRows = 1, kGroupK = 2 };
struct Grouping {
  int mode;
  int num_groups;
  const int* seg;         // [num_groups + 1] padded row offsets
  const int* tile_start;  // [num_groups + 1] prefix sum of ceil(rows_e / 256) (kGroupRows); tiles of expert e: that x tiles_n
};

// Row-parallel product of a tensor-parallel layer: the ranks hold slices of the contraction, so
// every rank's product is a partial sum of the whole [M, N] output.  Rank `owner = column /
// cols` reduces the columns owner * cols .. + cols - 1; instead of storing its partial tile at home
// and handing the buffer to a collective, the epilogue stores each tile straight into the owner's
// staging area over NVLink (plain stores to peer-mapped memory, issued while the tensor core works
// on the next tile): stage of rank o = [world][M][cols], slot `rank` written by this rank.
// cols is a multiple of 256, so a tile has one owner.
constexpr int kMaxScatterRanks = 8;
struct Scatter {
  int world;  // 0: off
  int rank;
  int cols;   // N / world
  __nv_bfloat16* stage[kMaxScatterRanks];
};

struct Params {
  __nv_bfloat16* c;
  const __nv_bfloat16* residual;
  int M, N, K;
  int64_t ldc, ldr;
  int epilogue;
  int* status;
  RowStatsOut rs;
  Grouping grp;
  Scatter sc;
  __nv_bfloat16* h;  // kSwiGLU: [M, N / 2] output, row stride ldh
  int64_t ldh;
};

// First element of the W-column chunk at (row, n0) of the output.
__device__ __forceinline__ __nv_bfloat16* c_chunk(const Params& p, int row, int n0) {
  if (p.sc.world > 0) {
    const int owner = n0 / p.sc.cols;
    return p.sc.stage[owner] + ((int64_t)p.sc.rank * p.M + row) * p.sc.cols + (n0 - owner * p.sc.cols);
  }
  return p.c + (int64_t)row * p.ldc + n0;
}

// Where one 256x256 tile (or this CTA's half of it) sits in the operands.
struct TileInfo {
  int a_m, a_k0;   // A: first MN index of this CTA's 128, first contraction index
  int b_n, b_k0;   // B: the same
  int num_kb;      // 128-wide contraction steps
  int c_row0;      // C row of this CTA's first accumulator row
  int row_end;     // C rows >= row_end do not exist (for this tile)
  int n0;          // first C column
  int tile_n;      // column-tile index (row statistics)
};

constexpr int kBandRows = 8;

template <bool B_MN>
__device__ __forceinline__ TileInfo decode_tile(const Params& p, int tile, int tiles_m, int tiles_n, int num_kb, int rank) {
  TileInfo t;
  if (p.grp.mode == kGroupNone) {
    // Tiles run down a band of kBandRows tile rows, column after column, then the next band: the
    // CTA pairs working at the same time cover a near-square patch of C (8 x 9 tiles on 74 pairs),
    // so a wave touches about 17 operand panels instead of 75 and a tall output (a weight
    // gradient of a wide layer) no longer re-reads its whole A operand once per tile column.
    const int band = tile / (kBandRows * tiles_n), first = band * kBandRows;
    const int rows = min(kBandRows, tiles_m - first), local = tile - band * kBandRows * tiles_n;
    const int m0 = (first + local % rows) * 256 + rank * 128;
    t.tile_n = local / rows;
    t.n0 = t.tile_n * 256;
    t.a_m = m0; t.a_k0 = 0; t.b_n = t.n0 + rank * 128; t.b_k0 = 0; t.num_kb = num_kb; t.c_row0 = m0; t.row_end = p.M;
    if (p.epilogue == kSwiGLU) {  // 128 gate rows for the leader, the matching up rows for its peer
      t.n0 = t.tile_n * 128;
      t.b_n = t.n0 + rank * (p.N >> 1);
    }
  } else if (p.grp.mode == kGroupRows) {
    int lo = 0, hi = p.grp.num_groups - 1;  // last e with tile_start[e] <= tile
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.grp.tile_start[mid] * tiles_n <= tile) lo = mid; else hi = mid - 1;
    }
    const int e = lo, s0 = p.grp.seg[e], s1 = p.grp.seg[e + 1];
    const int tm = (s1 - s0 + 255) >> 8, local = tile - p.grp.tile_start[e] * tiles_n;
    const int m0 = s0 + (local % tm) * 256 + rank * 128;
    t.tile_n = local / tm;
    t.n0 = t.tile_n * 256;
    t.a_m = m0; t.a_k0 = 0; t.num_kb = num_kb; t.c_row0 = m0; t.row_end = s1;
    t.b_n = (B_MN ? 0 : e * p.N) + t.n0 + rank * 128;
    t.b_k0 = B_MN ? e * p.K : 0;
  } else {
    const int per = tiles_m * tiles_n, e = tile / per, local = tile % per;
    const int m0 = (local % tiles_m) * 256 + rank * 128, s0 = p.grp.seg[e];
    t.tile_n = local / tiles_m;
    t.n0 = t.tile_n * 256;
    t.a_m = m0; t.a_k0 = s0; t.b_n = t.n0 + rank * 128; t.b_k0 = s0; t.num_kb = (p.grp.seg[e + 1] - s0) >> 7;
    t.c_row0 = e * p.M + m0; t.row_end = e * p.M + p.M;
  }
  return t;
}

// 32-byte store (one full sector) of sixteen bf16; ptr must be 32-byte aligned.
__device__ __forceinline__ void st32(__nv_bfloat16* ptr, const bf16x8& a, const bf16x8& b) {
  const uint4 x = *reinterpret_cast<const uint4*>(&a), y = *reinterpret_cast<const uint4*>(&b);
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"l"(ptr), "r"(x.x), "r"(x.y), "r"(x.z), "r"(x.w), "r"(y.x), "r"(y.y), "r"(y.z), "r"(y.w)
               : "memory");
}

// Epilogue of one thread: TMEM lane `taddr` (its 256 fp32 columns) -> row `row`, columns
// n0 .. n0+255 of C, with the configured epilogue.
template <int W>
__device__ __forceinline__ void store_accumulator(const Params& p, uint32_t taddr, int row, int n0, int row_end, bool zero) {
  __nv_bfloat16* crow = c_chunk(p, row, n0);
  const __nv_bfloat16* rrow = p.residual ? p.residual + (int64_t)row * p.ldr + n0 : nullptr;
  const bool vec_ok = ((p.ldc & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) &&
                      (p.epilogue != kAddResidual || (((p.ldr & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0)));
  const bool wide_ok = vec_ok && ((p.ldc & 15) == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 31) == 0);
#pragma unroll 1
  for (int c = 0; c < W / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait();
    if (zero) {  // no contraction step ran (an expert without rows): the accumulator holds nothing
#pragma unroll
      for (int j = 0; j < 32; ++j) r[j] = 0u;
    }
    if (row < row_end) {
      const int col0 = n0 + c * 32;
      if (vec_ok && col0 + 32 <= p.N) {
        bf16x8 packed[4];
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
          if (p.epilogue == kAccumulate) {
            float o[8];
            unpack8(ld8(crow + c * 32 + v * 8), o);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] += o[j];
          } else if (p.epilogue == kAddResidual) {
            float o[8];
            unpack8(ld8(rrow + c * 32 + v * 8), o);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] += o[j];
          }
          packed[v] = pack8(f);
        }
        if (wide_ok) {  // full 32-byte sectors per store
          st32(crow + c * 32, packed[0], packed[1]);
          st32(crow + c * 32 + 16, packed[2], packed[3]);
        } else {
#pragma unroll
          for (int v = 0; v < 4; ++v) st8(crow + c * 32 + v * 8, packed[v]);
        }
      } else {
        for (int j = 0; j < 32; ++j) {
          if (col0 + j < p.N) {
            float f = __uint_as_float(r[j]);
            if (p.epilogue == kAccumulate) f += __bfloat162float(crow[c * 32 + j]);
            else if (p.epilogue == kAddResidual) f += __bfloat162float(rrow[c * 32 + j]);
            crow[c * 32 + j] = __float2bfloat16(f);
          }
        }
      }
    }
  }
}

// ---- gated MLP: gate | up product with silu(gate) * up formed in the epilogue -------------------
// One thread = one row; `tlane` = TMEM address of its lane at the first of the 64 gate columns it handles
// (the matching up columns sit 128 columns further), col0 = their column in [0, I).  The activation is
// taken from the bf16-rounded gate and up (what the backward pass reads back), in the element-wise
// kernel's order: silu(gate) rounded to bf16, times up.  Needs I % 128 == 0, ldc / ldh multiples of 16
// and 32-byte aligned bases (checked on the host).
__device__ __forceinline__ void store_accumulator_swiglu(const Params& p, uint32_t tlane, int row, int col0, int row_end) {
  const int I = p.N >> 1;
  __nv_bfloat16* grow = p.c + (int64_t)row * p.ldc + col0;
  __nv_bfloat16* hrow = p.h + (int64_t)row * p.ldh + col0;
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    uint32_t g[32], u[32];
    tmem_ld32(tlane + c * 32, g);
    tmem_ld32(tlane + 128 + c * 32, u);
    tmem_ld_wait();
    if (row >= row_end) continue;
    bf16x8 gp[4], up[4], hp[4];
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      float gf[8], uf[8], o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { gf[j] = __uint_as_float(g[v * 8 + j]); uf[j] = __uint_as_float(u[v * 8 + j]); }
      gp[v] = pack8(gf);
      up[v] = pack8(uf);
      unpack8(gp[v], gf);
      unpack8(up[v], uf);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float sg = 1.f / (1.f + __expf(-gf[j]));
        o[j] = __bfloat162float(__float2bfloat16(gf[j] * sg)) * uf[j];
      }
      hp[v] = pack8(o);
    }
    st32(grow + c * 32, gp[0], gp[1]);
    st32(grow + c * 32 + 16, gp[2], gp[3]);
    st32(grow + I + c * 32, up[0], up[1]);
    st32(grow + I + c * 32 + 16, up[2], up[3]);
    st32(hrow + c * 32, hp[0], hp[1]);
    st32(hrow + c * 32 + 16, hp[2], hp[3]);
  }
}

// ---- epilogues that read memory (C += result, result + residual) ---------------------------
// The addend row (256 bf16 = 512 bytes per thread) is fetched into registers *before* the
// thread waits for the accumulator, so the loads' latency is spent while the tensor core still
// works on the tile.  With a short contraction (weight gradients: K = tokens of one step) the
// time per tile is otherwise set by eight dependent load round trips per thread.
template <int W>
struct RowPrefetch {
  uint4 v[W / 8];
  bool tile_ok;  // the same for every thread of the warp: selects the epilogue (its tcgen05.ld is warp-collective)
  bool valid;    // this thread's row exists (its loads were issued, its stores may be)
};

template <int W>
__device__ __forceinline__ bool tile_reads_vectorised(const Params& p, int n0) {
  if (p.epilogue == kStore || n0 + W > p.N || (p.ldc & 7) || (reinterpret_cast<uintptr_t>(p.c) & 15)) return false;
  if (p.epilogue == kAddResidual && ((p.ldr & 7) || (reinterpret_cast<uintptr_t>(p.residual) & 15))) return false;
  return true;
}

template <int W>
__device__ __forceinline__ void prefetch_addend(const Params& p, int row, int n0, int row_end, RowPrefetch<W>& pre) {
  pre.tile_ok = tile_reads_vectorised<W>(p, n0);
  pre.valid = pre.tile_ok && row < row_end;
  if (pre.valid) {
    const __nv_bfloat16* src = p.epilogue == kAccumulate ? p.c + (int64_t)row * p.ldc + n0 : p.residual + (int64_t)row * p.ldr + n0;
#pragma unroll
    for (int i = 0; i < W / 8; ++i) pre.v[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
  }
}

// Same result as store_accumulator for a tile whose addend rows are already in registers.  Called
// by whole warps (pre.tile_ok); a thread whose row does not exist takes part in the tensor-memory
// loads and stores nothing.
template <int W>
__device__ __forceinline__ void store_accumulator_prefetched(const Params& p, uint32_t taddr, int row, int n0, const RowPrefetch<W>& pre, bool zero) {
  __nv_bfloat16* crow = p.c + (int64_t)row * p.ldc + n0;
  const bool wide_ok = ((p.ldc & 15) == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 31) == 0);
#pragma unroll
  for (int c = 0; c < W / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait();
    bf16x8 packed[4];
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      float f[8], o[8];
      unpack8(*reinterpret_cast<const bf16x8*>(&pre.v[c * 4 + v]), o);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = (zero ? 0.f : __uint_as_float(r[v * 8 + j])) + o[j];
      packed[v] = pack8(f);
    }
    if (!pre.valid) continue;
    if (wide_ok) {
      st32(crow + c * 32, packed[0], packed[1]);
      st32(crow + c * 32 + 16, packed[2], packed[3]);
    } else {
#pragma unroll
      for (int v = 0; v < 4; ++v) st8(crow + c * 32 + v * 8, packed[v]);
    }
  }
}

// ---- logits tile + row statistics ------------------------------------------------------------
template <int W>
__device__ __forceinline__ void prefetch_targets(const Params& p, int row, int n0, RowPrefetch<W>& pre) {
  const int trow = row + p.rs.shift;
  pre.tile_ok = true;
  pre.valid = row < p.M && trow < p.rs.t_rows;
  const __nv_bfloat16* src = p.rs.targets + (int64_t)trow * p.rs.ldt + n0;
#pragma unroll
  for (int i = 0; i < W / 8; ++i) {
    if (pre.valid && n0 + i * 8 + 8 <= p.N) pre.v[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
    else pre.v[i] = make_uint4(0u, 0u, 0u, 0u);
  }
}

// Requires N % 8 == 0, ldc % 8 == 0 and 16-byte aligned C / target rows (checked on the host).
template <int W>
__device__ __forceinline__ void store_accumulator_with_stats(const Params& p, uint32_t taddr, int row, int n0, int record, int records_per_row,
                                                             const RowPrefetch<W>& pre) {
  __nv_bfloat16* crow = p.c + (int64_t)row * p.ldc + n0;
  RowStats sd{-INFINITY, 0.f, -INFINITY, 0x7fffffff}, st{-INFINITY, 0.f, -INFINITY, 0x7fffffff};
  float A = 0.f;
#pragma unroll
  for (int c = 0; c < W / 32; ++c) {
    uint32_t r[32];
    tmem_ld32(taddr + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const int col0 = n0 + c * 32 + v * 8;
      float f[8], x[8], t[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
      const bf16x8 packed = pack8(f);
      if (col0 + 8 <= p.N) {
        unpack8(packed, x);
        unpack8(*reinterpret_cast<const bf16x8*>(&pre.v[c * 4 + v]), t);
        online_update(sd, x, col0);
        online_update_kl(st, A, t, x, col0);
        if (row < p.M) st8(crow + c * 32 + v * 8, packed);
      }
    }
  }
  if (pre.valid) {
    float4* out = reinterpret_cast<float4*>(p.rs.partial + ((int64_t)row * records_per_row + record) * kStatWords);
    out[0] = make_float4(sd.m, sd.z, sd.best, __int_as_float(sd.best_idx));
    out[1] = make_float4(st.m, st.z, A, st.best);
    out[2] = make_float4(__int_as_float(st.best_idx), 0.f, 0.f, 0.f);
  }
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  // 1024-byte alignment for the swizzled tiles
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ __align__(8) uint64_t bar_full[STAGES], bar_empty[STAGES], bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (p.M + BM - 1) / BM, tiles_n = (p.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_addr(&bar_full[s]), 1);
      mbar_init(smem_addr(&bar_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_addr(&bar_acc_full[a]), 1);
      mbar_init(smem_addr(&bar_acc_empty[a]), 128);
    }
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(smem_addr(&bar_empty[stage]), phase ^ 1, p.status, kTimeoutProducer))) break;
          const uint32_t full = smem_addr(&bar_full[stage]);
          mbar_expect_tx(full, STAGE_BYTES);
          const uint32_t sa = smem_addr(smem + stage * STAGE_BYTES);
          tma_load_2d(sa, &map_a, full, kb * BK, m0);
          tma_load_2d(sa + A_BYTES, &map_b, full, kb * BK, n0);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_bf16(BM, BN);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        if (!(ok = mbar_wait(smem_addr(&bar_acc_empty[acc]), ((local >> 1) & 1) ^ 1, p.status, kTimeoutMma))) break;
        fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(smem_addr(&bar_full[stage]), phase, p.status, kTimeoutMma))) break;
          fence_after_sync();
          const uint32_t sa = smem_addr(smem + stage * STAGE_BYTES);
          const uint64_t adesc = smem_desc_kmajor_sw128(sa), bdesc = smem_desc_kmajor_sw128(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // advancing 16 K-elements = 32 bytes inside the 128-byte swizzled row: +2 in 16-byte units
            umma_bf16(tmem_d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
          }
          umma_commit(smem_addr(&bar_empty[stage]));  // frees the ring slot once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(smem_addr(&bar_acc_full[acc]));
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;  // TMEM lanes this warp may touch: 32*quarter .. +31
    bool ok = true;
    int local = 0;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * BN;
      RowPrefetch<BN> pre;
      prefetch_addend<BN>(p, m0 + quarter * 32 + lane, n0, p.M, pre);
      ok = mbar_wait(smem_addr(&bar_acc_full[acc]), (local >> 1) & 1, p.status, kTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      fence_after_sync();
      if (pre.tile_ok) store_accumulator_prefetched<BN>(p, tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN, m0 + quarter * 32 + lane, n0, pre, false);
      else store_accumulator<BN>(p, tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN, m0 + quarter * 32 + lane, n0, p.M, false);
      fence_before_sync();
      mbar_arrive(smem_addr(&bar_acc_empty[acc]));
    }
  }

  // A role that gave up did so after seconds of polling, far beyond the lifetime of any
  // bulk copy it had issued, so no copy is still writing shared memory at this point.
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- 256x256 tiles on CTA pairs ----------------------------------------------------------
// A pipeline stage holds KSUB sub-tiles of 64 K-elements (KSUB x 32 KB per CTA); the ring
// always spans 192 KB.  KSUB = 2 halves the number of barrier waits / commits the MMA
// thread executes per unit of tensor work (its instruction stream, not the tensor pipe,
// is what paces the loop at KSUB = 1).
constexpr int P_HALF = 128;                                    // rows of A and of B staged per CTA
constexpr int P_A_BYTES = P_HALF * BK * 2, P_B_BYTES = P_HALF * BK * 2, P_SUB_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_TILE_M = 2 * P_HALF, P_TILE_N = 2 * P_HALF;
constexpr int P_RING_BYTES = 6 * P_SUB_BYTES;
// The pair kernel runs eight epilogue warps: warps w and w + 4 reach the same 32 TMEM lanes (rows) and take 128 of the
// tile's 256 columns each, so two warps per scheduler share the epilogue's instruction stream (with four warps the row
// statistics of the lm_head epilogue, and the addend of short-contraction weight gradients, set the pace of the tile).
constexpr int P_THREADS = 320, P_EPI_COLS = 128;

template <int KSUB, bool A_MN = false, bool B_MN = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(P_THREADS, 1)
gemm_tn_2cta_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Params p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  static_assert(KSUB == 2 || (!A_MN && !B_MN), "MN-major operands are staged as 128-row boxes: KSUB must be 2");
  constexpr int P_STAGES = 6 / KSUB;
  constexpr int P_STAGE_BYTES = KSUB * P_SUB_BYTES;
  constexpr int STAGE_K = KSUB * BK;
  __shared__ __align__(8) uint64_t bar_full[P_STAGES], bar_empty[P_STAGES], bar_acc_full[2], bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  const int tiles_m = (p.M + P_TILE_M - 1) / P_TILE_M, tiles_n = (p.N + P_TILE_N - 1) / P_TILE_N;
  const int num_tiles = p.grp.mode == kGroupRows ? p.grp.tile_start[p.grp.num_groups] * tiles_n
                        : p.grp.mode == kGroupK  ? p.grp.num_groups * tiles_m * tiles_n
                                                 : tiles_m * tiles_n;
  const int num_kb = (p.K + STAGE_K - 1) / STAGE_K;

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(smem_addr(&bar_full[s]), 1);   // the leader's expect_tx arrival; bytes come from both CTAs' copies
      mbar_init(smem_addr(&bar_empty[s]), 1);  // one multicast commit per use
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_addr(&bar_acc_full[a]), 1);
      mbar_init(smem_addr(&bar_acc_empty[a]), 512);  // the epilogue threads of both CTAs (used in the leader only)
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // collective over the pair: the same warp of both CTAs
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  fence_before_sync();
  cluster_sync_all();  // barriers of both CTAs are initialised before any remote signal
  fence_after_sync();
  const uint32_t tmem_base = tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const TileInfo ti = decode_tile<B_MN>(p, tile, tiles_m, tiles_n, num_kb, (int)rank);
        for (int kb = 0; kb < ti.num_kb; ++kb) {
          if (!(ok = mbar_wait(smem_addr(&bar_empty[stage]), phase ^ 1, p.status, kTimeoutProducer))) break;
          const uint32_t full_local = smem_addr(&bar_full[stage]);
          if (leader) mbar_expect_tx(full_local, 2 * P_STAGE_BYTES);
          const uint32_t full_leader = map_to_cta(full_local, 0);
          const uint32_t sa = smem_addr(smem + stage * P_STAGE_BYTES);
          // Elements outside the matrices read as zeros (TMA fill).  K-major operand: sub-tile u =
          // 128 rows x 64 contraction columns.  MN-major operand: sub-tile u = 128 contraction rows x
          // 64 MN-columns (MN-elements 64u .. 64u+63 of this CTA's 128).  Either way 16 KB at the same place.
#pragma unroll
          for (int u = 0; u < KSUB; ++u) {
            if (A_MN) tma_load_2d_pair(sa + u * P_SUB_BYTES, &map_a, full_leader, ti.a_m + u * 64, ti.a_k0 + kb * STAGE_K);
            else tma_load_2d_pair(sa + u * P_SUB_BYTES, &map_a, full_leader, ti.a_k0 + kb * STAGE_K + u * BK, ti.a_m);
            if (B_MN) tma_load_2d_pair(sa + u * P_SUB_BYTES + P_A_BYTES, &map_b, full_leader, ti.b_n + u * 64, ti.b_k0 + kb * STAGE_K);
            else tma_load_2d_pair(sa + u * P_SUB_BYTES + P_A_BYTES, &map_b, full_leader, ti.b_k0 + kb * STAGE_K + u * BK, ti.b_n);
          }
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
      }
      // tail: stay until the MMAs that read this CTA's last slots have retired (their
      // completion is signalled into this CTA's shared memory)
      for (int s = 0; s < P_STAGES && ok; ++s) {
        ok = mbar_wait(smem_addr(&bar_empty[stage]), phase ^ 1, p.status, kTimeoutProducer);
        if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = instr_desc_ab(P_TILE_M, P_TILE_N, A_MN, B_MN);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      int local = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
        const int acc = local & 1;
        if (!(ok = mbar_wait(smem_addr(&bar_acc_empty[acc]), ((local >> 1) & 1) ^ 1, p.status, kTimeoutMma))) break;
        fence_after_sync();
        const uint32_t tmem_d = tmem_base + acc * BN;
        const int tile_kb = decode_tile<B_MN>(p, tile, tiles_m, tiles_n, num_kb, 0).num_kb;
        for (int kb = 0; kb < tile_kb; ++kb) {
          if (!(ok = mbar_wait(smem_addr(&bar_full[stage]), phase, p.status, kTimeoutMma))) break;
          fence_after_sync();
          const uint32_t sa = smem_addr(smem + stage * P_STAGE_BYTES);
          // MN-major: the two 64-element column blocks are P_SUB_BYTES apart (leading byte offset)
          const uint64_t adesc = A_MN ? smem_desc_mnmajor_sw128(sa, P_SUB_BYTES) : smem_desc_kmajor_sw128(sa);
          const uint64_t bdesc = B_MN ? smem_desc_mnmajor_sw128(sa + P_A_BYTES, P_SUB_BYTES) : smem_desc_kmajor_sw128(sa + P_A_BYTES);
#pragma unroll
          for (int u = 0; u < KSUB; ++u) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) {
              // K-major: next sub-tile + P_SUB_BYTES, next 16 K-elements inside a 128-byte swizzled row + 32 bytes;
              // MN-major: 16 contraction rows of 128 bytes = 2048 bytes per step (all in 16-byte units)
              const uint32_t off_k = u * (P_SUB_BYTES >> 4) + 2 * k, off_mn = (u * (BK / 16) + k) * (2048 >> 4);
              umma_bf16_pair(tmem_d, adesc + (A_MN ? off_mn : off_k), bdesc + (B_MN ? off_mn : off_k), idesc, (kb | u | k) != 0);
            }
          }
          umma_commit_pair(smem_addr(&bar_empty[stage]));  // frees the slot in both CTAs
          if (++stage == P_STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit_pair(smem_addr(&bar_acc_full[acc]));  // wakes the epilogues of both CTAs
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue (warps 2..9, both CTAs)
    const int quarter = warp & 3;         // TMEM lanes 32 * quarter .. + 31
    const int chalf = (warp - 2) >> 2;    // columns 128 * chalf .. + 127 of the tile
    const uint32_t acc_empty_leader[2] = {map_to_cta(smem_addr(&bar_acc_empty[0]), 0), map_to_cta(smem_addr(&bar_acc_empty[1]), 0)};
    bool ok = true;
    int local = 0;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++local) {
      const int acc = local & 1;
      const TileInfo ti = decode_tile<B_MN>(p, tile, tiles_m, tiles_n, num_kb, (int)rank);
      const int row = ti.c_row0 + quarter * 32 + lane, n0 = ti.n0 + chalf * P_EPI_COLS;
      const bool zero = ti.num_kb == 0;
      RowPrefetch<P_EPI_COLS> pre;
      const bool with_stats = p.rs.targets != nullptr, gated = p.epilogue == kSwiGLU;
      if (with_stats) prefetch_targets<P_EPI_COLS>(p, row, n0, pre);
      else if (!gated) prefetch_addend<P_EPI_COLS>(p, row, n0, ti.row_end, pre);
      ok = mbar_wait(smem_addr(&bar_acc_full[acc]), (local >> 1) & 1, p.status, kTimeoutEpilogue);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      fence_after_sync();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + chalf * P_EPI_COLS;
      if (gated)  // this warp: gate columns 64 * chalf .. + 63 of the tile and the same up columns
        store_accumulator_swiglu(p, tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN + chalf * 64, row, ti.n0 + chalf * 64, ti.row_end);
      else if (with_stats) store_accumulator_with_stats<P_EPI_COLS>(p, taddr, row, n0, ti.tile_n * 2 + chalf, tiles_n * 2, pre);
      else if (pre.tile_ok) store_accumulator_prefetched<P_EPI_COLS>(p, taddr, row, n0, pre, zero);
      else store_accumulator<P_EPI_COLS>(p, taddr, row, n0, ti.row_end, zero);
      fence_before_sync();
      mbar_arrive_cluster(acc_empty_leader[acc]);
    }
  }

  // Both CTAs stay until the pair is done: the peer's copies signal the leader's barriers,
  // the leader's MMAs read the peer's shared memory and write its TMEM.
  fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    fence_after_sync();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

// ---- host side ---------------------------------------------------------------------------
}  // namespace tc

// C[M,N] = op(A) * op(B)^T with epilogue (0 store, 1 C += result, 2 result + residual).
//   a_mn == 0: A is [M, K] row-major (K-major), lda = row stride;  a_mn == 1: A is [K, M] row-major (M contiguous)
//   b_mn == 0: B is [N, K] row-major (K-major), ldb = row stride;  b_mn == 1: B is [K, N] row-major (N contiguous)
// lda / ldb / ldc / ldr in elements; operand rows must be 16-byte aligned (ld multiple of 8).
// `status` is a device int the kernel writes a non-zero code to if a bounded wait ran out.
// variant: 0 = choose (CTA pairs when M > 128 or an operand is MN-major), 1 = one CTA per 128x256 tile (K-major
// only), 2 = CTA pairs with 64-wide K stages (K-major only), 3 = CTA pairs with 128-wide K stages.
static int launch_gemm_impl(const void* a, const void* b, void* c, const void* residual, int M, int N, int K, int64_t lda,
                            int64_t ldb, int64_t ldc, int64_t ldr, int epilogue, int a_mn, int b_mn, int* status, int variant,
                            const void* stats_targets, int64_t stats_ldt, int stats_t_rows, int stats_shift, float* stats_partial,
                            const tc::Grouping* grp, cudaStream_t stream, const tc::Scatter* scatter = nullptr, void* gated_h = nullptr,
                            int64_t gated_ldh = 0) {
  using namespace tc;
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return -1;
  const bool mn = a_mn || b_mn;
  if (variant == 0) variant = (M > BM || mn) ? kDefaultPairVariant : 1;
  if (mn && variant != 3) return -4;
  const bool pairs = variant >= 2;
  CUtensorMap map_a, map_b;
  int rc = a_mn ? make_map_bf16(&map_a, a, K, M, lda, 2 * BK) : make_map_bf16(&map_a, a, M, K, lda, BM);
  if (rc) return rc;
  // grouped by rows: B is the stack of the experts' matrices
  const int64_t b_stack = (grp != nullptr && grp->mode == kGroupRows) ? grp->num_groups : 1;
  rc = b_mn ? make_map_bf16(&map_b, b, b_stack * K, N, ldb, 2 * BK) : make_map_bf16(&map_b, b, b_stack * N, K, ldb, pairs ? P_HALF : BN);
  if (rc) return rc;
  Params p{(__nv_bfloat16*)c, (const __nv_bfloat16*)residual, M, N, K, ldc, ldr, epilogue, status, RowStatsOut{nullptr, 0, 0, 0, nullptr},
           Grouping{kGroupNone, 0, nullptr, nullptr}, Scatter{}, (__nv_bfloat16*)gated_h, gated_ldh};
  if (epilogue == kSwiGLU) {
    if (!pairs || a_mn || b_mn || grp != nullptr || stats_targets != nullptr || scatter != nullptr || gated_h == nullptr || (N & 255) || (ldc & 15) ||
        (gated_ldh & 15) || (reinterpret_cast<uintptr_t>(c) & 31) || (reinterpret_cast<uintptr_t>(gated_h) & 31))
      return -8;
  }
  if (scatter != nullptr) {
    if (!pairs || grp != nullptr || stats_targets != nullptr || epilogue != kStore || scatter->world < 1 || scatter->world > kMaxScatterRanks ||
        scatter->cols * scatter->world != N || (scatter->cols & 255))
      return -7;
    p.sc = *scatter;
    p.c = scatter->stage[scatter->rank];  // alignment checks of the store path look at c / ldc
    p.ldc = scatter->cols;
    for (int q = 0; q < scatter->world; ++q)
      if (reinterpret_cast<uintptr_t>(scatter->stage[q]) & 31) return -7;
  }
  if (grp != nullptr) {
    if (!pairs || variant != 3 || stats_targets != nullptr || residual != nullptr) return -6;
    if (grp->mode == kGroupRows && (a_mn || (K & 127) || (N & 255))) return -6;  // experts' matrices must not share a box
    if (grp->mode == kGroupK && !(a_mn && b_mn)) return -6;
    p.grp = *grp;
  }
  if (stats_targets != nullptr) {
    if (!pairs || a_mn || b_mn || epilogue != kStore || (N & 7) || (ldc & 7) || (stats_ldt & 7) || (reinterpret_cast<uintptr_t>(c) & 15) ||
        (reinterpret_cast<uintptr_t>(stats_targets) & 15))
      return -5;
    p.rs = RowStatsOut{(const __nv_bfloat16*)stats_targets, stats_ldt, stats_t_rows, stats_shift, stats_partial};
  }
  count_launch(1);
  if (pairs) {
    static PerDeviceOnce configured2;
    constexpr int smem2 = P_RING_BYTES + 1024;
    if (configured2.needed()) {
      bool ok = cudaFuncSetAttribute(gemm_tn_2cta_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) == cudaSuccess;
      ok = ok && cudaFuncSetAttribute(gemm_tn_2cta_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) == cudaSuccess;
      ok = ok && cudaFuncSetAttribute(gemm_tn_2cta_kernel<2, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) == cudaSuccess;
      ok = ok && cudaFuncSetAttribute(gemm_tn_2cta_kernel<2, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) == cudaSuccess;
      ok = ok && cudaFuncSetAttribute(gemm_tn_2cta_kernel<2, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) == cudaSuccess;
      if (!ok) return -2;
      configured2.mark();
    }
    const int max_pairs = kNumSM / 2;
    // grouped: the number of tiles is known on the device only; every pair looks for work
    const int tiles = grp != nullptr ? max_pairs : ((M + P_TILE_M - 1) / P_TILE_M) * ((N + P_TILE_N - 1) / P_TILE_N);
    const int grid = 2 * (tiles < max_pairs ? tiles : max_pairs);
    if (a_mn && b_mn) gemm_tn_2cta_kernel<2, true, true><<<grid, P_THREADS, smem2, stream>>>(map_a, map_b, p);
    else if (a_mn) gemm_tn_2cta_kernel<2, true, false><<<grid, P_THREADS, smem2, stream>>>(map_a, map_b, p);
    else if (b_mn) gemm_tn_2cta_kernel<2, false, true><<<grid, P_THREADS, smem2, stream>>>(map_a, map_b, p);
    else if (variant == 3) gemm_tn_2cta_kernel<2><<<grid, P_THREADS, smem2, stream>>>(map_a, map_b, p);
    else gemm_tn_2cta_kernel<1><<<grid, P_THREADS, smem2, stream>>>(map_a, map_b, p);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
  }
  static PerDeviceOnce configured;
  constexpr int smem_bytes = STAGES * STAGE_BYTES + 1024;
  if (configured.needed()) {
    if (cudaFuncSetAttribute(gemm_tn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return -2;
    configured.mark();
  }
  const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  const int grid = tiles < kNumSM ? tiles : kNumSM;
  gemm_tn_kernel<<<grid, THREADS, smem_bytes, stream>>>(map_a, map_b, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int launch_gemm_tcgen05(const void* a, const void* b, void* c, const void* residual, int M, int N, int K, int64_t lda,
                        int64_t ldb, int64_t ldc, int64_t ldr, int epilogue, int a_mn, int b_mn, int* status, int variant,
                        cudaStream_t stream) {
  return launch_gemm_impl(a, b, c, residual, M, N, K, lda, ldb, ldc, ldr, epilogue, a_mn, b_mn, status, variant, nullptr, 0, 0, 0, nullptr, nullptr, stream);
}

int launch_gemm_tn_tcgen05(const void* a, const void* b, void* c, const void* residual, int M, int N, int K, int64_t lda,
                           int64_t ldb, int64_t ldc, int64_t ldr, int epilogue, int* status, int variant, cudaStream_t stream) {
  return launch_gemm_tcgen05(a, b, c, residual, M, N, K, lda, ldb, ldc, ldr, epilogue, 0, 0, status, variant, stream);
}

// ---- row-parallel product with the reduce-scatter's transfer in the epilogue -----------------
// partial[M, N] = a[M, K] . b[N, K]^T, tile columns stored into slot `rank` of their owner's staging
// area stage[owner] = [world][M][N / world] (addresses valid on this device: peer-mapped for the
// other ranks).  N / world must be a multiple of 256.
int launch_gemm_scatter(const void* a, const void* b, void* const* stage, int world, int rank, int M, int N, int K, int64_t lda, int64_t ldb,
                        int* status, cudaStream_t stream) {
  if (world < 1 || world > tc::kMaxScatterRanks || rank < 0 || rank >= world || N % world) return -7;
  tc::Scatter sc{world, rank, N / world, {}};
  for (int q = 0; q < world; ++q) sc.stage[q] = static_cast<__nv_bfloat16*>(stage[q]);
  return launch_gemm_impl(a, b, stage[rank], nullptr, M, N, K, lda, ldb, N / world, 0, tc::kStore, 0, 0, status, 3, nullptr, 0, 0, 0, nullptr, nullptr,
                          stream, &sc);
}

// ---- gate | up product of a gated MLP with the activation in the epilogue ---------------------
// gate_up[M, 2 I] = x[M, K] . w[2 I, K]^T (gate rows first) and h[M, I] = silu(gate) * up.  I % 128 == 0.
int launch_gemm_swiglu(const void* x, const void* w, void* gate_up, void* h, int M, int I, int K, int64_t ldx, int64_t ldw, int64_t ldc, int64_t ldh,
                       int* status, cudaStream_t stream) {
  return launch_gemm_impl(x, w, gate_up, nullptr, M, 2 * I, K, ldx, ldw, ldc, 0, tc::kSwiGLU, 0, 0, status, 3, nullptr, 0, 0, 0, nullptr, nullptr, stream,
                          nullptr, h, ldh);
}

// ---- grouped products for mixture-of-experts layers -----------------------------------------
// counts[e] rows belong to expert e.  seg[e] = offset of its (128-row aligned) segment in the padded
// row order, mtile_start[e] = prefix sum of ceil(segment rows / 256).  One block; E <= 4096.
__global__ void moe_group_plan_kernel(const int* __restrict__ counts, int num_groups, int* __restrict__ seg, int* __restrict__ mtile_start) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int off = 0, tiles = 0;
  for (int e = 0; e < num_groups; ++e) {
    seg[e] = off;
    mtile_start[e] = tiles;
    const int padded = (counts[e] + 127) & ~127;
    off += padded;
    tiles += (padded + 255) >> 8;
  }
  seg[num_groups] = off;
  mtile_start[num_groups] = tiles;
}

void launch_moe_group_plan(const int* counts, int num_groups, int* seg, int* mtile_start, cudaStream_t stream) {
  count_launch(1);
  moe_group_plan_kernel<<<1, 32, 0, stream>>>(counts, num_groups, seg, mtile_start);
}

// mode 1 (rows grouped): c[R, N] = a[R, K] . b_e^T, b the stack [E, N, K] (b_mn 0) or, for the input
//   gradient, c[R, N] = a[R, K] . b_e with b = [E, K, N] (b_mn 1).  R = rows of the padded order.
// mode 2 (contraction grouped): c_e[M, N] (=, +=) a[seg_e, M]^T . b[seg_e, N], c the stack [E, M, N]; K = R.
int launch_gemm_grouped(const void* a, const void* b, void* c, int M, int N, int K, int64_t lda, int64_t ldb, int64_t ldc, int epilogue,
                        int mode, int b_mn, const int* seg, const int* mtile_start, int num_groups, int* status, cudaStream_t stream) {
  if (mode != tc::kGroupRows && mode != tc::kGroupK) return -6;
  const tc::Grouping grp{mode, num_groups, seg, mtile_start};
  const int a_mn = mode == tc::kGroupK ? 1 : 0;
  return launch_gemm_impl(a, b, c, nullptr, M, N, K, lda, ldb, ldc, 0, epilogue, a_mn, mode == tc::kGroupK ? 1 : b_mn, status, 3, nullptr, 0, 0, 0,
                          nullptr, &grp, stream);
}

// ---- lm_head product fused with the row loss (KL divergence / cross-entropy on the argmax) -----
int lmhead_stat_words() { return tc::kStatWords; }
// records per logits row: two per 256-column tile (one per 128-column epilogue half)
int lmhead_tiles_n(int N) { return 2 * ((N + tc::P_TILE_N - 1) / tc::P_TILE_N); }

// logits[M,N] = x[M,K] * w[N,K]^T (stored, bf16) and, per (row, 256-column tile), the statistics of the logits
// row and of targets[row + shift] over those columns into partial[M, tiles_n, kStatWords].
int launch_lmhead_logits_stats(const void* x, const void* w, void* logits, const void* targets, int M, int N, int K, int64_t ldx,
                               int64_t ldw, int64_t ldc, int64_t ldt, int t_rows, int shift, float* partial, int* status,
                               cudaStream_t stream) {
  return launch_gemm_impl(x, w, logits, nullptr, M, N, K, ldx, ldw, ldc, 0, tc::kStore, 0, 0, status, 3, targets, ldt, t_rows, shift, partial, nullptr, stream);
}

// One warp per row: merge the row's tile records and write what the row-loss forward kernel writes
// (loss, the five saved statistics, both argmaxes); rows with active[r] == 0 get the same sentinels.
// op: 0 = KL(target || draft), 3 = cross-entropy against the target row's argmax.
__global__ void __launch_bounds__(128)
lmhead_combine_kernel(const float* __restrict__ partial, const __nv_bfloat16* __restrict__ logits, const uint8_t* __restrict__ active,
                      float* __restrict__ loss, float* __restrict__ stats, int* __restrict__ argmax_d, int* __restrict__ argmax_t,
                      int rows, int tiles_n, int64_t ld_logits, int op) {
  const int r = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  float* st = stats + r;
  if (active && !active[r]) {
    if (lane == 0) {
      loss[r] = 0.f;
      for (int k = 0; k < 5; ++k) st[(int64_t)k * rows] = 0.f;
      if (argmax_d) argmax_d[r] = -1;
      if (argmax_t) argmax_t[r] = -2;
    }
    return;
  }
  RowStats sd{-INFINITY, 0.f, -INFINITY, 0x7fffffff}, stt{-INFINITY, 0.f, -INFINITY, 0x7fffffff};
  float A = 0.f;
  for (int t = lane; t < tiles_n; t += 32) {
    const float4* rec = reinterpret_cast<const float4*>(partial + ((int64_t)r * tiles_n + t) * tc::kStatWords);
    const float4 a = rec[0], b = rec[1], c = rec[2];
    merge_stats(sd, RowStats{a.x, a.y, a.z, __float_as_int(a.w)});
    merge_stats_kl(stt, A, RowStats{b.x, b.y, b.w, __float_as_int(c.x)}, b.z);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    RowStats od{__shfl_xor_sync(0xffffffffu, sd.m, o), __shfl_xor_sync(0xffffffffu, sd.z, o), __shfl_xor_sync(0xffffffffu, sd.best, o),
                __shfl_xor_sync(0xffffffffu, sd.best_idx, o)};
    RowStats ot{__shfl_xor_sync(0xffffffffu, stt.m, o), __shfl_xor_sync(0xffffffffu, stt.z, o), __shfl_xor_sync(0xffffffffu, stt.best, o),
                __shfl_xor_sync(0xffffffffu, stt.best_idx, o)};
    const float oA = __shfl_xor_sync(0xffffffffu, A, o);
    merge_stats(sd, od);
    merge_stats_kl(stt, A, ot, oA);
  }
  if (lane == 0) {
    const float lse_d = sd.m + __logf(sd.z), lse_t = stt.m + __logf(stt.z);
    float L, extra;
    if (op == 3) {
      L = lse_d - __bfloat162float(logits[(int64_t)r * ld_logits + stt.best_idx]);
      extra = (float)stt.best_idx;
    } else {
      L = A / stt.z + lse_d - lse_t;
      extra = L;
    }
    loss[r] = L;
    st[0] = sd.m;
    st[(int64_t)rows] = sd.z;
    st[(int64_t)2 * rows] = stt.m;
    st[(int64_t)3 * rows] = stt.z;
    st[(int64_t)4 * rows] = extra;
    if (argmax_d) argmax_d[r] = sd.best_idx;
    if (argmax_t) argmax_t[r] = stt.best_idx;
  }
}

int launch_lmhead_combine(const float* partial, const void* logits, const uint8_t* active, float* loss, float* stats, int* argmax_d,
                          int* argmax_t, int rows, int tiles_n, int64_t ld_logits, int op, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (op != 0 && op != 3) return -1;
  count_launch(1);
  lmhead_combine_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(partial, (const __nv_bfloat16*)logits, active, loss, stats, argmax_d, argmax_t, rows,
                                                          tiles_n, ld_logits, op);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace sb200
