// Peer-visible device memory: allocation, CUDA IPC export / import.
//
// Buffers that other ranks of the same node read or write from their own kernels
// (gradient / weight buffers of the fused optimizer, control blocks) are allocated
// with cudaMalloc directly -- not from PyTorch's caching allocator, whose blocks are
// sub-allocated and may move -- exported as IPC handles, exchanged through
// torch.distributed, and opened by every peer.  NVSwitch gives every GPU a direct
// load/store path to the mapped memory.
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

namespace sb200 {

int peer_malloc(int64_t nbytes, void** out) {
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)nbytes) != cudaSuccess) return -1;
  if (cudaMemset(p, 0, (size_t)nbytes) != cudaSuccess) return -2;
  *out = p;
  return 0;
}
int peer_free(void* p) { return cudaFree(p) == cudaSuccess ? 0 : -1; }

int peer_export(void* p, unsigned char* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, p) != cudaSuccess) return -1;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
int peer_import(const unsigned char* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) return -1;
  *out = p;
  return 0;
}
int peer_close(void* p) { return cudaIpcCloseMemHandle(p) == cudaSuccess ? 0 : -1; }

}  // namespace sb200
