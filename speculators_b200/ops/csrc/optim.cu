// Flat-buffer optimizer kernels: squared-norm reduction and fused AdamW.
//
// The trainable parameters of a model live in one contiguous bf16 buffer (the
// compute weights) with a parallel bf16 gradient buffer; the optimizer keeps fp32
// master weights and both moments for the slice of that buffer this rank owns.
// One AdamW launch therefore updates every parameter: read grad (+ clip scale),
// master, m, v; write master, m, v and the bf16 compute weight.  All scalar
// inputs that change from step to step (learning rate, bias corrections, the
// gradient norm) are read from device memory so the launch can sit inside a
// captured CUDA graph.
#include "common.cuh"

namespace sb200 {

constexpr int kOptThreads = 256;

// hyper layout (fp32): [0] lr  [1] beta1  [2] beta2  [3] eps  [4] weight_decay
//                      [5] bias_correction1  [6] bias_correction2  [7] max_grad_norm (<=0: off)
//                      [8] grad_scale (multiplied into every gradient, e.g. 1/world_size)
constexpr int kHyperLen = 16;

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Stage 1: per-CTA partial sums of squares into partial[blockIdx.x].
template <typename T>
__global__ void __launch_bounds__(kOptThreads)
sumsq_partial_kernel(const T* __restrict__ g, int64_t n, float* __restrict__ partial) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float v = to_f<T>(g[i]);
    acc += v * v;
  }
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

template <>
__global__ void __launch_bounds__(kOptThreads)
sumsq_partial_kernel<__nv_bfloat16>(const __nv_bfloat16* __restrict__ g, int64_t n,
                                     float* __restrict__ partial) {
  __shared__ float scratch[33];
  float acc = 0.f;
  const int64_t nvec = n >> 3;  // buffer base is 16-byte aligned by construction
  for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec;
       v += (int64_t)gridDim.x * blockDim.x) {
    float f[8];
    unpack8(ld8(g + (v << 3)), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += f[j] * f[j];
  }
  for (int64_t i = (nvec << 3) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(g[i]);
    acc += v * v;
  }
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

// Stage 2: out[0] (+)= sum(partial[0:P]) in a fixed order (deterministic).
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int P, float* __restrict__ out,
                                   int accumulate) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int i = threadIdx.x; i < P; i += blockDim.x) acc += partial[i];
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + acc : acc;
}

// norm_sq: device scalar holding the (already all-reduced) sum of squares of the
// *unscaled* gradients; clip coefficient = min(1, max_norm / (grad_scale*sqrt(norm_sq) + 1e-6)).
template <typename G>
__global__ void __launch_bounds__(kOptThreads)
adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
             const G* __restrict__ grad, __nv_bfloat16* __restrict__ w16, int64_t n,
             const float* __restrict__ hyper, const float* __restrict__ norm_sq) {
  const float lr = hyper[0], b1 = hyper[1], b2 = hyper[2], eps = hyper[3], wd = hyper[4];
  const float bc1 = hyper[5], bc2 = hyper[6], max_norm = hyper[7];
  float gscale = hyper[8];
  if (max_norm > 0.f && norm_sq) {
    const float total = gscale * sqrtf(norm_sq[0]);
    const float coef = max_norm / (total + 1e-6f);
    if (coef < 1.f) gscale *= coef;
  }
  const float step_size = lr / bc1;
  const float inv_sqrt_bc2 = rsqrtf(bc2);
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    const float g = to_f<G>(grad[i]) * gscale;
    float p = master[i];
    float mi = m[i], vi = v[i];
    p *= (1.f - lr * wd);
    mi = b1 * mi + (1.f - b1) * g;
    vi = b2 * vi + (1.f - b2) * g * g;
    const float denom = sqrtf(vi) * inv_sqrt_bc2 + eps;
    p -= step_size * (mi / denom);
    master[i] = p;
    m[i] = mi;
    v[i] = vi;
    if (w16) w16[i] = __float2bfloat16(p);
  }
}

// ---- Muon ------------------------------------------------------------------------------
// Matrix update of Muon around its Newton-Schulz iteration (which runs as GEMMs):
//   muon_momentum: g' = g * grad_scale * clip;  buf = lerp(buf, g', 1 - momentum);
//                  u = nesterov ? lerp(g', buf, momentum) : buf;  out = bf16(u)
//                  plus the per-CTA sums of u^2 (for the Frobenius normalisation that
//                  opens the iteration), one launch for both;
//   muon_apply:    w = w * (1 - lr * wd) - lr * adjust * o;  w16 = bf16(w)
// with lr = hyper[0] * lr_ratio (the matrix group follows the schedule of the AdamW group),
// read from device memory so that the launches can be captured.
template <typename G>
__global__ void __launch_bounds__(kOptThreads)
muon_momentum_kernel(const G* __restrict__ grad, float* __restrict__ buf, __nv_bfloat16* __restrict__ out, int64_t n,
                     const float* __restrict__ hyper, const float* __restrict__ norm_sq, float momentum, int nesterov,
                     float* __restrict__ partial) {
  __shared__ float scratch[33];
  const float max_norm = hyper[7];
  float gscale = hyper[8];
  if (max_norm > 0.f && norm_sq) {
    const float coef = max_norm / (gscale * sqrtf(norm_sq[0]) + 1e-6f);
    if (coef < 1.f) gscale *= coef;
  }
  float acc = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float g = to_f<G>(grad[i]) * gscale;
    float b = buf[i];
    b += (g - b) * (1.f - momentum);
    buf[i] = b;
    const float u = nesterov ? g + (b - g) * momentum : b;
    const __nv_bfloat16 r = __float2bfloat16(u);
    out[i] = r;
    const float ur = __bfloat162float(r);
    acc += ur * ur;
  }
  acc = block_sum(acc, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = acc;
}

__global__ void __launch_bounds__(kOptThreads)
muon_apply_kernel(float* __restrict__ master, const __nv_bfloat16* __restrict__ update, __nv_bfloat16* __restrict__ w16, int64_t n,
                  const float* __restrict__ hyper, float lr_ratio, float weight_decay, float adjust) {
  const float lr = hyper[0] * lr_ratio;
  const float keep = 1.f - lr * weight_decay, step = lr * adjust;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float w = master[i] * keep - step * __bfloat162float(update[i]);
    master[i] = w;
    if (w16) w16[i] = __float2bfloat16(w);
  }
}

// partial: [sumsq_num_partials()] scratch; out_sumsq[0] = sum of squares of the bf16 update
void launch_muon_momentum(const void* grad, int grad_is_bf16, float* buf, void* out, int64_t n, const float* hyper,
                          const float* norm_sq, float momentum, int nesterov, float* partial, float* out_sumsq,
                          cudaStream_t stream) {
  if (n <= 0) return;
  const int P = 4 * kNumSM;
  count_launch(2);
  if (grad_is_bf16)
    muon_momentum_kernel<__nv_bfloat16><<<P, kOptThreads, 0, stream>>>((const __nv_bfloat16*)grad, buf, (__nv_bfloat16*)out, n, hyper,
                                                                       norm_sq, momentum, nesterov, partial);
  else
    muon_momentum_kernel<float><<<P, kOptThreads, 0, stream>>>((const float*)grad, buf, (__nv_bfloat16*)out, n, hyper, norm_sq,
                                                               momentum, nesterov, partial);
  sumsq_final_kernel<<<1, 256, 0, stream>>>(partial, P, out_sumsq, 0);
}

void launch_muon_apply(float* master, const void* update, void* w16, int64_t n, const float* hyper, float lr_ratio,
                       float weight_decay, float adjust, cudaStream_t stream) {
  if (n <= 0) return;
  int64_t blocks = (n + kOptThreads - 1) / kOptThreads;
  const int64_t cap = (int64_t)kNumSM * 16;
  count_launch(1);
  muon_apply_kernel<<<(int)(blocks < cap ? blocks : cap), kOptThreads, 0, stream>>>(
      master, (const __nv_bfloat16*)update, (__nv_bfloat16*)w16, n, hyper, lr_ratio, weight_decay, adjust);
}

// Hyper-parameters travel as kernel arguments (copied at launch), so the host can
// prepare step k+1 while step k is still queued: no staging buffer to overwrite.
struct HyperVals {
  float v[16];
};
__global__ void set_hyper_kernel(float* __restrict__ hyper, const HyperVals vals) {
  if (threadIdx.x < 16) hyper[threadIdx.x] = vals.v[threadIdx.x];
}

void launch_set_hyper(float* hyper, const float* host_vals16, cudaStream_t stream) {
  HyperVals vals;
  for (int i = 0; i < 16; ++i) vals.v[i] = host_vals16[i];
  count_launch(1);
  set_hyper_kernel<<<1, 32, 0, stream>>>(hyper, vals);
}

int sumsq_num_partials() { return 4 * kNumSM; }

void launch_sumsq(const void* g, int is_bf16, int64_t n, float* partial, float* out, int accumulate,
                  cudaStream_t stream) {
  const int P = sumsq_num_partials();
  count_launch(2);
  if (is_bf16)
    sumsq_partial_kernel<__nv_bfloat16><<<P, kOptThreads, 0, stream>>>((const __nv_bfloat16*)g, n,
                                                                        partial);
  else
    sumsq_partial_kernel<float><<<P, kOptThreads, 0, stream>>>((const float*)g, n, partial);
  sumsq_final_kernel<<<1, 256, 0, stream>>>(partial, P, out, accumulate);
}

void launch_adamw(float* master, float* m, float* v, const void* grad, int grad_is_bf16, void* w16,
                  int64_t n, const float* hyper, const float* norm_sq, cudaStream_t stream) {
  if (n <= 0) return;
  int64_t blocks = (n + kOptThreads - 1) / kOptThreads;
  const int64_t cap = (int64_t)kNumSM * 16;
  const int grid = (int)(blocks < cap ? blocks : cap);
  count_launch(1);
  if (grad_is_bf16)
    adamw_kernel<__nv_bfloat16><<<grid, kOptThreads, 0, stream>>>(
        master, m, v, (const __nv_bfloat16*)grad, (__nv_bfloat16*)w16, n, hyper, norm_sq);
  else
    adamw_kernel<float><<<grid, kOptThreads, 0, stream>>>(master, m, v, (const float*)grad,
                                                          (__nv_bfloat16*)w16, n, hyper, norm_sq);
}

}  // namespace sb200
