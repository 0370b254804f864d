// SwiGLU and rotary-embedding kernels (bf16 in/out, fp32 math).
#include "common.cuh"

namespace sb200 {

// gate_up is [rows, 2*I] with the gate in columns [0, I) and up in [I, 2I)
// (the gate and up projections run as one GEMM).  h = silu(gate) * up.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ gate_up,
                                  __nv_bfloat16* __restrict__ h, int64_t rows, int I) {
  const int nvec = I >> 3;
  const int64_t total = rows * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx - r * nvec) << 3;
    const __nv_bfloat16* base = gate_up + r * 2 * (int64_t)I;
    float g[8], u[8], o[8];
    unpack8(ld8(base + c), g);
    unpack8(ld8(base + I + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      // eager order: act(gate) rounded to bf16, then times up
      o[j] = __bfloat162float(__float2bfloat16(g[j] * s)) * u[j];
    }
    st8(h + r * (int64_t)I + c, pack8(o));
  }
}

// d(gate_up) from dh: dgate = dh * up * (s + g*s*(1-s)), dup = dh * silu(g)
__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ dh,
                                  const __nv_bfloat16* __restrict__ gate_up,
                                  __nv_bfloat16* __restrict__ dgate_up, int64_t rows, int I) {
  const int nvec = I >> 3;
  const int64_t total = rows * nvec;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = idx / nvec;
    const int c = (int)(idx - r * nvec) << 3;
    const __nv_bfloat16* base = gate_up + r * 2 * (int64_t)I;
    __nv_bfloat16* obase = dgate_up + r * 2 * (int64_t)I;
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(ld8(base + c), g);
    unpack8(ld8(base + I + c), u);
    unpack8(ld8(dh + r * (int64_t)I + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float s = 1.f / (1.f + __expf(-g[j]));
      dg[j] = d[j] * u[j] * (s + g[j] * s * (1.f - s));
      du[j] = d[j] * g[j] * s;
    }
    st8(obase + c, pack8(dg));
    st8(obase + I + c, pack8(du));
  }
}

// In-place neox rotary embedding on `heads` consecutive heads of width `hd`
// inside a row of `row_stride` elements (q and k live side by side in the fused
// qkv projection output, so one launch rotates both).  Only the first `rot`
// channels of a head rotate (partial rotary).  cos/sin tables are fp32
// [max_pos, rot/2]; `positions` selects the table row per token.  `sign` = +1
// forward, -1 backward (the transpose of a rotation is the inverse rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ x, const int64_t* __restrict__ positions,
                            const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                            int64_t tokens, int heads, int hd, int rot, int64_t row_stride,
                            int64_t max_pos, float sign) {
  const int half = rot >> 1;
  const int64_t total = tokens * heads * half;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % half);
    const int64_t th = idx / half;
    const int h = (int)(th % heads);
    const int64_t t = th / heads;
    int64_t pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float c = cos_t[pos * half + i];
    const float s = sign * sin_t[pos * half + i];
    __nv_bfloat16* p = x + t * row_stride + (int64_t)h * hd;
    const float x1 = __bfloat162float(p[i]);
    const float x2 = __bfloat162float(p[i + half]);
    p[i] = __float2bfloat16(x1 * c - x2 * s);
    p[i + half] = __float2bfloat16(x2 * c + x1 * s);
  }
}

// Same rotation, eight channel pairs per thread (16-byte accesses); needs rot/2 % 8 == 0
// and 16-byte aligned rows/heads (row_stride % 8 == 0, hd % 8 == 0, aligned base).
__global__ void rope_vec8_kernel(__nv_bfloat16* __restrict__ x, const int64_t* __restrict__ positions,
                                 const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                 int64_t tokens, int heads, int hd, int rot, int64_t row_stride,
                                 int64_t max_pos, float sign) {
  const int half = rot >> 1;
  const int hv = half >> 3;
  const int64_t total = tokens * heads * hv;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int i = (int)(idx % hv) << 3;
    const int64_t th = idx / hv;
    const int h = (int)(th % heads);
    const int64_t t = th / heads;
    int64_t pos = positions[t];
    pos = pos < 0 ? 0 : (pos >= max_pos ? max_pos - 1 : pos);
    const float4* c4 = reinterpret_cast<const float4*>(cos_t + pos * half + i);
    const float4* s4 = reinterpret_cast<const float4*>(sin_t + pos * half + i);
    const float4 ca = c4[0], cb = c4[1], sa = s4[0], sb = s4[1];
    const float c[8] = {ca.x, ca.y, ca.z, ca.w, cb.x, cb.y, cb.z, cb.w};
    const float sn[8] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w};
    __nv_bfloat16* p = x + t * row_stride + (int64_t)h * hd + i;
    float x1[8], x2[8], y1[8], y2[8];
    unpack8(ld8(p), x1);
    unpack8(ld8(p + half), x2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sj = sign * sn[j];
      y1[j] = x1[j] * c[j] - x2[j] * sj;
      y2[j] = x2[j] * c[j] + x1[j] * sj;
    }
    st8(p, pack8(y1));
    st8(p + half, pack8(y2));
  }
}

static inline int grid_for(int64_t total, int threads) {
  int64_t g = (total + threads - 1) / threads;
  const int64_t cap = (int64_t)kNumSM * 16;
  return (int)(g < cap ? (g > 0 ? g : 1) : cap);
}

void launch_swiglu_fwd(const void* gate_up, void* h, int64_t rows, int I, cudaStream_t stream) {
  if (rows <= 0) return;
  count_launch(1);
  swiglu_fwd_kernel<<<grid_for(rows * (I >> 3), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)h, rows, I);
}
void launch_swiglu_bwd(const void* dh, const void* gate_up, void* dgate_up, int64_t rows, int I,
                       cudaStream_t stream) {
  if (rows <= 0) return;
  count_launch(1);
  swiglu_bwd_kernel<<<grid_for(rows * (I >> 3), 256), 256, 0, stream>>>(
      (const __nv_bfloat16*)dh, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)dgate_up, rows, I);
}
void launch_rope(void* x, const int64_t* positions, const float* cos_t, const float* sin_t,
                 int64_t tokens, int heads, int hd, int rot, int64_t row_stride, int64_t max_pos,
                 float sign, cudaStream_t stream) {
  if (tokens <= 0) return;
  count_launch(1);
  const int half = rot >> 1;
  const bool vec = (half % 8 == 0) && (hd % 8 == 0) && (row_stride % 8 == 0) && ((uintptr_t)x % 16 == 0) &&
                   ((uintptr_t)cos_t % 16 == 0) && ((uintptr_t)sin_t % 16 == 0);
  if (vec) {
    rope_vec8_kernel<<<grid_for(tokens * heads * (half >> 3), 256), 256, 0, stream>>>(
        (__nv_bfloat16*)x, positions, cos_t, sin_t, tokens, heads, hd, rot, row_stride, max_pos, sign);
    return;
  }
  rope_kernel<<<grid_for(tokens * heads * half, 256), 256, 0, stream>>>(
      (__nv_bfloat16*)x, positions, cos_t, sin_t, tokens, heads, hd, rot, row_stride, max_pos, sign);
}

}  // namespace sb200
