// RMSNorm forward / backward for bf16 activations (fp32 statistics).
//
// Forward:  y[r, :] = x[src(r), :] * rsqrt(mean(x^2) + eps) * w
//   * `row_index` (optional) gathers the input row, which turns the kernel into
//     "embedding lookup + RMSNorm" for the EAGLE-3 first layer;
//   * separate row strides for x and y let the caller write straight into one half
//     of a [T, 2H] buffer, so the concat of normalised embeddings and normalised
//     hidden states never exists as a separate copy.
// Backward: dx = rstd * (g - xhat * mean(g * xhat)),  g = dy * w,  xhat = x * rstd
//           dw[c] = sum_r dy[r, c] * xhat[r, c]   (two-stage: per-CTA partials,
//           then a column reduce; the partial buffer is caller-provided scratch).
#include "common.cuh"

namespace sb200 {

constexpr int kNormThreads = 256;
// Vectors (8 x bf16) handled per thread are a template parameter NV in {2, 4, 8}:
// H <= 256 * 8 * NV, i.e. 4096 / 8192 / 16384 columns.

SB200_BOUNDS_RECORD

template <int NV>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                   const int64_t* __restrict__ row_index, __nv_bfloat16* __restrict__ y,
                   float* __restrict__ rstd_out, int rows, int H, int64_t x_stride,
                   int64_t y_stride, float eps, int64_t src_rows) {
  __shared__ float scratch[33];
  const int nvec = H >> 3;
  for (int r = blockIdx.x; r < rows; r += gridDim.x) {
    const int64_t src = row_index ? row_index[r] : (int64_t)r;
    if (!SB200_IN_RANGE(src, src_rows, 1)) continue;  // debug build only
    const __nv_bfloat16* xr = x + src * x_stride;
    float cache[NV][8];
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        unpack8(ld8(xr + (v << 3)), cache[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += cache[i][j] * cache[i][j];
      }
    }
    ss = block_sum(ss, scratch);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[r] = rstd;
    __nv_bfloat16* yr = y + (int64_t)r * y_stride;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float wv[8], o[8];
        unpack8(ld8(w + (v << 3)), wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          // match the eager module: normalise in fp32, round to bf16, then scale
          o[j] = __bfloat162float(__float2bfloat16(cache[i][j] * rstd)) * wv[j];
        }
        st8(yr + (v << 3), pack8(o));
      }
    }
  }
}

// One CTA walks rows blockIdx.x, +gridDim.x, ... and keeps its dw partial in registers.
// A row's x and dy stay in registers (packed bf16) between the reduction and the dx pass,
// and the next row is fetched before the block-wide reduction of the current one, so the
// loads of one row overlap the synchronisation of the previous row.
template <int NV>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x,
                   const __nv_bfloat16* __restrict__ w, const float* __restrict__ rstd_in,
                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int rows, int H,
                   int64_t dy_stride, int64_t x_stride, int64_t dx_stride, int accumulate_dx) {
  __shared__ float scratch[33];
  const int nvec = H >> 3;
  float dwacc[NV][8];
  bf16x8 wreg[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int v = threadIdx.x + i * kNormThreads;
    if (v < nvec) wreg[i] = ld8(w + (v << 3));
#pragma unroll
    for (int j = 0; j < 8; ++j) dwacc[i][j] = 0.f;
  }

  constexpr bool kPrefetch = NV <= 4;  // wider rows would spill: fetch each row when it is due
  constexpr int NB = kPrefetch ? NV : 1;
  bf16x8 xa[NV], da[NV], xb[NB], db[NB];
  auto fetch = [&](int r, bf16x8* xr_, bf16x8* dr_) {
    const __nv_bfloat16* xr = x + (int64_t)r * x_stride;
    const __nv_bfloat16* dyr = dy + (int64_t)r * dy_stride;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        xr_[i] = ld8(xr + (v << 3));
        dr_[i] = ld8(dyr + (v << 3));
      }
    }
  };
  int r = blockIdx.x;
  if (kPrefetch && r < rows) fetch(r, xa, da);
  for (; r < rows; r += gridDim.x) {
    if constexpr (kPrefetch) {
      const int rn = r + gridDim.x;
      if (rn < rows) fetch(rn, xb, db);
    } else {
      fetch(r, xa, da);
    }
    const float rstd = rstd_in[r];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float xv[8], dv[8], wv[8];
        unpack8(xa[i], xv);
        unpack8(da[i], dv);
        unpack8(wreg[i], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float xh = xv[j] * rstd;
          dot += dv[j] * wv[j] * xh;
          dwacc[i][j] += dv[j] * xh;
        }
      }
    }
    dot = block_sum(dot, scratch) / (float)H;
    __nv_bfloat16* dxr = dx + (int64_t)r * dx_stride;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float xv[8], dv[8], wv[8], o[8];
        unpack8(xa[i], xv);
        unpack8(da[i], dv);
        unpack8(wreg[i], wv);
        if (accumulate_dx) unpack8(ld8(dxr + (v << 3)), o);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = rstd * (dv[j] * wv[j] - xv[j] * rstd * dot);
          o[j] = accumulate_dx ? o[j] + d : d;
        }
        st8(dxr + (v << 3), pack8(o));
      }
    }
    if constexpr (kPrefetch) {
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        xa[i] = xb[i];
        da[i] = db[i];
      }
    }
  }
  if (dw_partial) {
    float* out = dw_partial + (int64_t)blockIdx.x * H;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int v = threadIdx.x + i * kNormThreads;
      if (v < nvec) {
        float4* o4 = reinterpret_cast<float4*>(out + (v << 3));
        o4[0] = make_float4(dwacc[i][0], dwacc[i][1], dwacc[i][2], dwacc[i][3]);
        o4[1] = make_float4(dwacc[i][4], dwacc[i][5], dwacc[i][6], dwacc[i][7]);
      }
    }
  }
}

// ---- narrow rows (H <= 256: per-head q / k norms) ---------------------------------------------
// One warp per row, lane v holds the row's v-th vector of eight: no shared memory and no block
// barrier per row.  The block-per-row kernels above spend a 256-thread CTA and two barriers on a
// 128-element row (16 active lanes); for the [tokens x heads, head_dim] norms of Qwen3-style
// attention that was 0.3-1.2 ms per launch against about 20 us of memory traffic.
constexpr int kNarrowMaxH = 256;
constexpr int kNarrowWarps = kNormThreads / 32;

__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_narrow_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ y,
                          float* __restrict__ rstd_out, int rows, int H, int64_t x_stride, int64_t y_stride, float eps) {
  const int lane = threadIdx.x & 31, nvec = H >> 3;
  const bool on = lane < nvec;
  float wv[8];
  if (on) unpack8(ld8(w + (lane << 3)), wv);
  const int warps = gridDim.x * kNarrowWarps;
  for (int r = blockIdx.x * kNarrowWarps + (threadIdx.x >> 5); r < rows; r += warps) {
    float xv[8], ss = 0.f;
    if (on) {
      unpack8(ld8(x + (int64_t)r * x_stride + (lane << 3)), xv);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += xv[j] * xv[j];
    }
    ss = warp_sum(ss);
    const float rstd = rsqrtf(ss / (float)H + eps);
    if (lane == 0 && rstd_out) rstd_out[r] = rstd;
    if (on) {
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = __bfloat162float(__float2bfloat16(xv[j] * rstd)) * wv[j];
      st8(y + (int64_t)r * y_stride + (lane << 3), pack8(o));
    }
  }
}

// dw partials: one row of H floats per warp of the grid (summed by colsum_kernel).
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_narrow_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                          const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, int rows, int H,
                          int64_t dy_stride, int64_t x_stride, int64_t dx_stride, int accumulate_dx) {
  const int lane = threadIdx.x & 31, nvec = H >> 3;
  const bool on = lane < nvec;
  float wv[8], dwacc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { wv[j] = 0.f; dwacc[j] = 0.f; }
  if (on) unpack8(ld8(w + (lane << 3)), wv);
  const int warps = gridDim.x * kNarrowWarps, warp_id = blockIdx.x * kNarrowWarps + (threadIdx.x >> 5);
  for (int r = warp_id; r < rows; r += warps) {
    float xv[8], dv[8], dot = 0.f;
    const float rstd = rstd_in[r];
    if (on) {
      unpack8(ld8(x + (int64_t)r * x_stride + (lane << 3)), xv);
      unpack8(ld8(dy + (int64_t)r * dy_stride + (lane << 3)), dv);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float xh = xv[j] * rstd;
        dot += dv[j] * wv[j] * xh;
        dwacc[j] += dv[j] * xh;
      }
    }
    dot = warp_sum(dot) / (float)H;
    if (on) {
      float o[8];
      __nv_bfloat16* dxr = dx + (int64_t)r * dx_stride + (lane << 3);
      if (accumulate_dx) unpack8(ld8(dxr), o);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float d = rstd * (dv[j] * wv[j] - xv[j] * rstd * dot);
        o[j] = accumulate_dx ? o[j] + d : d;
      }
      st8(dxr, pack8(o));
    }
  }
  if (dw_partial && on) {
    float4* o4 = reinterpret_cast<float4*>(dw_partial + (int64_t)warp_id * H + (lane << 3));
    o4[0] = make_float4(dwacc[0], dwacc[1], dwacc[2], dwacc[3]);
    o4[1] = make_float4(dwacc[4], dwacc[5], dwacc[6], dwacc[7]);
  }
}

static int narrow_grid(int rows) {
  const int blocks = (rows + kNarrowWarps - 1) / kNarrowWarps;
  return blocks < 4 * kNumSM ? blocks : 4 * kNumSM;
}

// dw[c] (+)= sum_p partial[p, c].  Block = 32 columns x 32 row-groups; the row-groups
// split P (a handful of independent loads per thread) and meet in shared memory, so
// each column is summed in a fixed order (deterministic) by H/32 CTAs.
constexpr int kColsumGroups = 32;
__global__ void __launch_bounds__(32 * kColsumGroups)
colsum_kernel(const float* __restrict__ partial, float* __restrict__ dw, int P, int H, int accumulate) {
  __shared__ float tile[kColsumGroups][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  float s = 0.f;
  if (c < H) {
#pragma unroll 4
    for (int p = threadIdx.y; p < P; p += kColsumGroups) s += partial[(int64_t)p * H + c];
  }
  tile[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < H) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < kColsumGroups; ++i) t += tile[i][threadIdx.x];
    dw[c] = accumulate ? dw[c] + t : t;
  }
}

int rmsnorm_bwd_partial_rows(int rows, int H) {
  if (H <= kNarrowMaxH) return narrow_grid(rows) * kNarrowWarps;  // one partial row per warp
  int g = 2 * kNumSM;
  return rows < g ? rows : g;
}

SB200_BOUNDS_READER(read_bounds_norm)

// src_rows: number of rows of `x` (what `row_index` may address).
void launch_rmsnorm_fwd(const void* x, const void* w, const int64_t* row_index, void* y,
                        float* rstd, int rows, int H, int64_t x_stride, int64_t y_stride, float eps,
                        int64_t src_rows, cudaStream_t stream) {
  if (rows <= 0) return;
  if (H <= kNarrowMaxH && row_index == nullptr) {
    count_launch(1);
    rmsnorm_fwd_narrow_kernel<<<narrow_grid(rows), kNormThreads, 0, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                                                             (__nv_bfloat16*)y, rstd, rows, H, x_stride, y_stride, eps);
    return;
  }
  int grid = rows < 8 * kNumSM ? rows : 8 * kNumSM;
#define SB200_FWD(NVV)                                                                         \
  rmsnorm_fwd_kernel<NVV><<<grid, kNormThreads, 0, stream>>>(                                    \
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, row_index, (__nv_bfloat16*)y, rstd, rows, \
      H, x_stride, y_stride, eps, src_rows)
  count_launch(1);
  if (H <= 4096) SB200_FWD(2);
  else if (H <= 8192) SB200_FWD(4);
  else SB200_FWD(8);
#undef SB200_FWD
}

void launch_rmsnorm_bwd(const void* dy, const void* x, const void* w, const float* rstd, void* dx,
                        float* dw_partial, float* dw, int rows, int H, int64_t dy_stride,
                        int64_t x_stride, int64_t dx_stride, int accumulate_dx, int accumulate_dw,
                        cudaStream_t stream) {
  if (rows <= 0) return;
  if (H <= kNarrowMaxH) {
    const int g = narrow_grid(rows);
    count_launch(1);
    rmsnorm_bwd_narrow_kernel<<<g, kNormThreads, 0, stream>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,
                                                            (__nv_bfloat16*)dx, dw_partial, rows, H, dy_stride, x_stride, dx_stride,
                                                            accumulate_dx);
    if (dw_partial && dw) {
      count_launch(1);
      colsum_kernel<<<(H + 31) / 32, dim3(32, kColsumGroups), 0, stream>>>(dw_partial, dw, g * kNarrowWarps, H, accumulate_dw);
    }
    return;
  }
  const int grid = rmsnorm_bwd_partial_rows(rows, H);
#define SB200_BWD(NVV)                                                                       \
  rmsnorm_bwd_kernel<NVV><<<grid, kNormThreads, 0, stream>>>(                                  \
      (const __nv_bfloat16*)dy, (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, rstd,         \
      (__nv_bfloat16*)dx, dw_partial, rows, H, dy_stride, x_stride, dx_stride, accumulate_dx)
  count_launch(1);
  if (H <= 4096) SB200_BWD(2);
  else if (H <= 8192) SB200_BWD(4);
  else SB200_BWD(8);
#undef SB200_BWD
  if (dw_partial && dw) count_launch(1);
  if (dw_partial && dw)
    colsum_kernel<<<(H + 31) / 32, dim3(32, kColsumGroups), 0, stream>>>(dw_partial, dw, grid, H, accumulate_dw);
}

}  // namespace sb200
