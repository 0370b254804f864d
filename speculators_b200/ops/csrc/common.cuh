// Shared device helpers for the sm_100a kernels of this package.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb200 {

void count_launch(int n);

// Debug build (-DSB200_CHECK_BOUNDS): kernels validate data-dependent row indices before
// using them.  The first violation is recorded (site, index, limit) in a per-module device
// record that the host reads back; the access is skipped, so a bad index never becomes a
// fault.  In the normal build the check compiles to `true`.
//   sites: 1 rmsnorm gather row, 2 exchange push source row, 3 exchange push destination
//          row, 4 exchange pull source row
struct BoundsRecord {
  int site;
  long long index;
  long long limit;
};
#ifdef SB200_CHECK_BOUNDS
__device__ __forceinline__ bool bounds_ok(BoundsRecord* rec, long long idx, long long n, int site) {
  if (idx >= 0 && idx < n) return true;
  if (atomicCAS(&rec->site, 0, site) == 0) {
    rec->index = idx;
    rec->limit = n;
  }
  return false;
}
#define SB200_BOUNDS_RECORD static __device__ sb200::BoundsRecord g_bounds = {0, 0, 0};
#define SB200_IN_RANGE(idx, n, site) sb200::bounds_ok(&g_bounds, (long long)(idx), (long long)(n), site)
// host side: copy the module's record out and clear it
#define SB200_BOUNDS_READER(name)                                                       \
  int name(BoundsRecord* out) {                                                         \
    if (cudaMemcpyFromSymbol(out, g_bounds, sizeof(BoundsRecord)) != cudaSuccess) return -1; \
    const BoundsRecord zero = {0, 0, 0};                                                \
    return cudaMemcpyToSymbol(g_bounds, &zero, sizeof(BoundsRecord)) == cudaSuccess ? 0 : -1; \
  }
#else
#define SB200_BOUNDS_RECORD
#define SB200_IN_RANGE(idx, n, site) true
#define SB200_BOUNDS_READER(name)  \
  int name(BoundsRecord* out) {    \
    *out = BoundsRecord{0, 0, 0};  \
    return 0;                      \
  }
#endif

constexpr int kWarp = 32;
// B200: 148 SMs.  Persistent / grid-stride kernels size their grids from this.
constexpr int kNumSM = 148;

// Kernel attributes (the dynamic shared memory limit) belong to a device: a launcher sets them the first time it
// runs on each device of the process, not once per process.
struct PerDeviceOnce {
  bool done[64] = {};
  static int device() {
    int d = 0;
    return cudaGetDevice(&d) == cudaSuccess && d >= 0 && d < 64 ? d : -1;
  }
  bool needed() const { const int d = device(); return d < 0 || !done[d]; }
  void mark() { const int d = device(); if (d >= 0) done[d] = true; }
};

struct alignas(16) bf16x8 {
  __nv_bfloat162 v[4];
};

__device__ __forceinline__ void unpack8(const bf16x8& p, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p.v[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

__device__ __forceinline__ bf16x8 pack8(const float (&f)[8]) {
  bf16x8 p;
#pragma unroll
  for (int i = 0; i < 4; ++i) p.v[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return p;
}

__device__ __forceinline__ bf16x8 ld8(const __nv_bfloat16* ptr) {
  return *reinterpret_cast<const bf16x8*>(ptr);
}
__device__ __forceinline__ void st8(__nv_bfloat16* ptr, const bf16x8& v) {
  *reinterpret_cast<bf16x8*>(ptr) = v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; every thread gets the result.  `scratch` holds >= 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // protect scratch reuse across consecutive calls
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

}  // namespace sb200
