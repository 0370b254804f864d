// Allocation-free sum of squares (see no_alloc.h for the contract).
#include "no_alloc.h"

#include <stdio.h>

#include "common.cuh"

namespace {

// Scratch: one fp32 partial per 65,536-element chunk.  Lives in the library image on
// every device that loads it.  In host code the name below is only a stand-in for
// the symbol; kernels must be given the address from cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_partials[SB200_NOALLOC_MAX_PARTIALS];

constexpr int kThreads = 256;
constexpr int kMaxDevices = 64;

// partial[c] = sum of squares of chunk c  (chunk = 65,536 consecutive elements)
__global__ void __launch_bounds__(kThreads)
noalloc_partial_kernel(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ partial,
                       int n_chunks) {
  __shared__ float scratch[33];
  for (int c = blockIdx.x; c < n_chunks; c += gridDim.x) {
    const long long begin = (long long)c * SB200_NOALLOC_CHUNK;
    long long end = begin + SB200_NOALLOC_CHUNK;
    if (end > n) end = n;
    float acc = 0.f;
    for (long long i = begin + threadIdx.x; i < end; i += kThreads) {
      const float v = __bfloat162float(x[i]);
      acc += v * v;
    }
    acc = sb200::block_sum(acc, scratch);
    if (threadIdx.x == 0) partial[c] = acc;
  }
}

// out[0] (+)= partial[0] + partial[1] + ...  in a fixed order
__global__ void noalloc_final_kernel(const float* __restrict__ partial, int n_chunks,
                                     float* __restrict__ out, int accumulate) {
  __shared__ float scratch[33];
  float acc = 0.f;
  for (int i = threadIdx.x; i < n_chunks; i += blockDim.x) acc += partial[i];
  acc = sb200::block_sum(acc, scratch);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + acc : acc;
}

thread_local char t_error[256] = "";
float* g_scratch_addr[kMaxDevices] = {nullptr};

int fail(int code, const char* what, cudaError_t err = cudaSuccess) {
  if (err != cudaSuccess)
    snprintf(t_error, sizeof(t_error), "%s: %s", what, cudaGetErrorString(err));
  else
    snprintf(t_error, sizeof(t_error), "%s", what);
  return code;
}

}  // namespace

extern "C" const char* sb200_noalloc_last_error(void) { return t_error; }

extern "C" int sb200_sumsq_bf16_noalloc(const void* x, long long n, float* out, int accumulate,
                                        void* stream) {
  if (out == nullptr || n < 0 || (n > 0 && x == nullptr))
    return fail(SB200_NOALLOC_ERR_BAD_ARGUMENT, "sb200_sumsq_bf16_noalloc: null pointer or negative size");
  if (n > SB200_NOALLOC_MAX_ELEMENTS) {
    snprintf(t_error, sizeof(t_error),
             "sb200_sumsq_bf16_noalloc: n = %lld exceeds the fixed scratch capacity of %lld elements", n,
             (long long)SB200_NOALLOC_MAX_ELEMENTS);
    return SB200_NOALLOC_ERR_TOO_LARGE;
  }
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return fail(SB200_NOALLOC_ERR_CUDA, "cudaGetDevice", err);
  if (dev < 0 || dev >= kMaxDevices) return fail(SB200_NOALLOC_ERR_BAD_ARGUMENT, "device ordinal out of range");
  // one-time set-up per device (with that device current): device address of the scratch array
  float* scratch = g_scratch_addr[dev];
  if (scratch == nullptr) {
    void* ptr = nullptr;
    err = cudaGetSymbolAddress(&ptr, g_noalloc_partials);
    if (err != cudaSuccess || ptr == nullptr) return fail(SB200_NOALLOC_ERR_CUDA, "cudaGetSymbolAddress(scratch)", err);
    scratch = static_cast<float*>(ptr);
    g_scratch_addr[dev] = scratch;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int n_chunks = (int)((n + SB200_NOALLOC_CHUNK - 1) / SB200_NOALLOC_CHUNK);
  if (n_chunks > 0) {
    const int grid = n_chunks < 8 * sb200::kNumSM ? n_chunks : 8 * sb200::kNumSM;
    sb200::count_launch(1);
    noalloc_partial_kernel<<<grid, kThreads, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, scratch, n_chunks);
    err = cudaGetLastError();  // a refused first launch leaves the partials unwritten: do not reduce them
    if (err != cudaSuccess) return fail(SB200_NOALLOC_ERR_CUDA, "kernel launch (partials)", err);
  }
  sb200::count_launch(1);
  noalloc_final_kernel<<<1, 256, 0, s>>>(scratch, n_chunks, out, accumulate);
  err = cudaGetLastError();
  if (err != cudaSuccess) return fail(SB200_NOALLOC_ERR_CUDA, "kernel launch", err);
  t_error[0] = '\0';
  return SB200_NOALLOC_OK;
}
