// Allocation-free entry point of the library (C ABI).
//
// This entry point has no counterpart in the reference implementation; it exists
// for callers of this library that are not allowed to allocate device memory.
//
// Who that is: code that runs where the CUDA allocator must not be touched, for
// instance a watchdog-driven health probe that computes a gradient norm while
// another thread of the training process may be stuck holding the caching
// allocator's lock, an out-of-memory handler that wants one last diagnostic when
// no device memory is left to allocate, or an embedding application that hands this
// library a fixed memory budget and forbids cudaMalloc / cudaFree after start-up.  The regular operator (`torch.ops.sb200.sumsq`) takes its
// scratch buffer from PyTorch's caching allocator on every call; this variant keeps
// its scratch in a fixed array that is part of the loaded library image.
//
//   int sb200_sumsq_bf16_noalloc(const void* x, long long n, float* out,
//                                int accumulate, void* stream);
//
// Computes out[0] = sum_i x[i]^2 (or out[0] += ... when `accumulate` != 0) over `n`
// bf16 values at device address `x`, in fp32, on CUDA stream `stream`
// (a cudaStream_t; nullptr = the legacy default stream).  `x` must be 2-byte
// aligned device memory, `out` a device float; both are supplied by the caller.
// The reduction order is fixed (one partial per 65,536-element chunk, partials
// summed by one block in index order), so equal inputs give bit-equal results.
//
// Limits and rules
//   * n must satisfy 0 <= n <= SB200_NOALLOC_MAX_ELEMENTS (2^30).  Larger sizes are
//     rejected with SB200_NOALLOC_ERR_TOO_LARGE; nothing is launched.
//   * The scratch array holds SB200_NOALLOC_MAX_PARTIALS floats (64 KiB).  Every GPU
//     that loads the library carries it until the process exits.
//   * The first call on a device resolves the device address of the scratch array
//     (cudaGetSymbolAddress, with that device current) and caches it; make that first
//     call before starting any stream capture on the device.
//   * The call itself never calls cudaMalloc, cudaFree or any allocating library
//     routine.
//   * All calls on one device share the scratch array, and it keeps the previous
//     call's partials.  Each call overwrites exactly the entries it reads, so nothing
//     has to be cleared between calls, but two calls whose kernels overlap on the GPU
//     (different streams without ordering, or different host threads) race on it.
//     Serialise calls per device.
//
// Return value: 0 on success, a negative SB200_NOALLOC_ERR_* code otherwise;
// sb200_noalloc_last_error() returns a static description of the last failure on
// the calling thread.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define SB200_NOALLOC_CHUNK 65536LL
#define SB200_NOALLOC_MAX_PARTIALS 16384
#define SB200_NOALLOC_MAX_ELEMENTS (SB200_NOALLOC_CHUNK * SB200_NOALLOC_MAX_PARTIALS)

#define SB200_NOALLOC_OK 0
#define SB200_NOALLOC_ERR_BAD_ARGUMENT (-1)
#define SB200_NOALLOC_ERR_TOO_LARGE (-2)
#define SB200_NOALLOC_ERR_CUDA (-3)

int sb200_sumsq_bf16_noalloc(const void* x, long long n, float* out, int accumulate, void* stream);
const char* sb200_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
