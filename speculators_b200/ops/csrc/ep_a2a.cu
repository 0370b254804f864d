// Expert-parallel token exchange over NVLink peer memory: the dispatch / combine
// all-to-all of a sparse MoE layer as row kernels that read and write the other ranks'
// buffers directly, fused with the permutation, the routing-weight scaling and the
// weighted sum that otherwise surround a library all-to-all.
//
//   push    every send slot (a token routed to an expert) is one warp: it copies the source
//           row, optionally scaled, straight into row dst_pos of rank dst_rank's receive
//           buffer (16-byte stores over NVLink).  The last CTA to finish publishes the
//           sender's sequence number in every rank's flag array (st.release.sys after a
//           system-scope fence).
//   wait    bounded poll (ld.acquire.sys) of the local flag array until every rank has
//           published the sequence number; gives up with a status code, never hangs.
//   pull    one warp per token sums its k rows, weighted, out of the ranks' buffers
//           (16-byte loads over NVLink) into the local output row, and can keep a local
//           copy of the gathered rows (the backward of the weighted sum needs them).
//   signal  publishes a sequence number without moving data ("my buffer is ready to be
//           pulled from").
//
// No kernel waits for a later launch of the same process: push / signal only publish,
// wait only polls, so a single process may drive several virtual ranks one phase at a time.
#include "common.cuh"
#include "ep_a2a.h"

namespace sb200 {

namespace {

__device__ __forceinline__ void ep_st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ep_ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

constexpr int kWarpsPerBlock = 8;

SB200_BOUNDS_RECORD

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
ep_push_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ src_row, const int* __restrict__ dst_rank,
               const int* __restrict__ dst_pos, const float* __restrict__ scale, int n_slots, int H, int src_rows, int capacity, EpPeers dst, unsigned int* done_counter, EpPeers flags, int my_rank, int world, uint32_t seq) {
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int s = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); s < n_slots; s += gridDim.x * kWarpsPerBlock) {
    const int r = dst_rank[s];
    if (r < 0 || r >= world) continue;
    const int64_t pos = dst_pos[s];
    if (!SB200_IN_RANGE(src_row[s], src_rows, 2) || !SB200_IN_RANGE(pos, capacity, 3)) continue;  // debug build only
    const __nv_bfloat16* in = src + (int64_t)src_row[s] * H;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(dst.ptr[r]) + pos * H;
    const float w = scale != nullptr ? scale[s] : 1.f;
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      unpack8(ld8(in + v * 8), f);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] *= w;
      st8(out + v * 8, pack8(f));  // w = 1: bf16 -> fp32 -> bf16 is exact
    }
  }
  // publish once every CTA's rows are on their way: each thread fences its own remote
  // stores, the last CTA to arrive writes the flags
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned int prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0;  // ready for the next launch
      __threadfence_system();
      for (int r = 0; r < world; ++r) ep_st_release_sys(reinterpret_cast<uint32_t*>(flags.ptr[r]) + my_rank, seq);
    }
  }
}

__global__ void ep_signal_kernel(EpPeers flags, int my_rank, int world, uint32_t seq) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    __threadfence_system();
    for (int r = 0; r < world; ++r) ep_st_release_sys(reinterpret_cast<uint32_t*>(flags.ptr[r]) + my_rank, seq);
  }
}

// status codes: 51 = a rank did not publish `seq` within the spin budget
__global__ void ep_wait_kernel(const uint32_t* __restrict__ flags_local, int world, uint32_t seq, uint32_t spin_limit, int* status) {
  const int r = threadIdx.x;
  if (r >= world) return;
  for (uint32_t i = 0; i < spin_limit; ++i) {
    const uint32_t v = ep_ld_acquire_sys(flags_local + r);
    if ((int32_t)(v - seq) >= 0) return;
    __nanosleep(64);
  }
  atomicCAS(status, 0, 51);
}

__global__ void __launch_bounds__(kWarpsPerBlock * 32)
ep_pull_kernel(EpPeers src, const int* __restrict__ src_rank, const int* __restrict__ src_pos, const float* __restrict__ weight,
               int T, int k, int H, int world, int capacity, __nv_bfloat16* __restrict__ out, __nv_bfloat16* __restrict__ rows_out) {
  const int lane = threadIdx.x & 31;
  const int nvec = H >> 3;
  for (int t = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5); t < T; t += gridDim.x * kWarpsPerBlock) {
    for (int v = lane; v < nvec; v += 32) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.f;
      for (int j = 0; j < k; ++j) {
        const int s = t * k + j;
        const int r = src_rank[s];
        if (r < 0 || r >= world) continue;
        if (!SB200_IN_RANGE(src_pos[s], capacity, 4)) continue;  // debug build only
        const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(src.ptr[r]) + (int64_t)src_pos[s] * H;
        const float w = weight != nullptr ? weight[s] : 1.f;
        const bf16x8 raw = ld8(row + v * 8);
        if (rows_out != nullptr) st8(rows_out + (int64_t)s * H + v * 8, raw);
        float f[8];
        unpack8(raw, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w, f[i], acc[i]);
      }
      st8(out + (int64_t)t * H + v * 8, pack8(acc));
    }
  }
}

int grid_for(int64_t units) {
  const int64_t blocks = (units + kWarpsPerBlock - 1) / kWarpsPerBlock;
  return (int)(blocks < 1 ? 1 : (blocks > 4 * kNumSM ? 4 * kNumSM : blocks));
}

}  // namespace

SB200_BOUNDS_READER(read_bounds_ep)

int launch_ep_push(const __nv_bfloat16* src, const int* src_row, const int* dst_rank, const int* dst_pos, const float* scale,
                   int n_slots, int H, int src_rows, int capacity, const EpPeers& dst, unsigned int* done_counter,
                   const EpPeers& flags, int my_rank, int world, uint32_t seq, cudaStream_t stream) {
  if (H % 8 != 0 || world < 1 || world > 16) return -1;
  count_launch(1);
  ep_push_kernel<<<grid_for(n_slots), kWarpsPerBlock * 32, 0, stream>>>(src, src_row, dst_rank, dst_pos, scale, n_slots, H, src_rows, capacity, dst, done_counter, flags,
                                                                       my_rank, world, seq);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int launch_ep_signal(const EpPeers& flags, int my_rank, int world, uint32_t seq, cudaStream_t stream) {
  if (world < 1 || world > 16) return -1;
  count_launch(1);
  ep_signal_kernel<<<1, 32, 0, stream>>>(flags, my_rank, world, seq);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int launch_ep_wait(const uint32_t* flags_local, int world, uint32_t seq, uint32_t spin_limit, int* status, cudaStream_t stream) {
  if (world < 1 || world > 16) return -1;
  count_launch(1);
  ep_wait_kernel<<<1, 32, 0, stream>>>(flags_local, world, seq, spin_limit, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int launch_ep_pull(const EpPeers& src, const int* src_rank, const int* src_pos, const float* weight, int T, int k, int H, int world,
                   int capacity, __nv_bfloat16* out, __nv_bfloat16* rows_out, cudaStream_t stream) {
  if (H % 8 != 0 || world < 1 || world > 16) return -1;
  count_launch(1);
  ep_pull_kernel<<<grid_for(T), kWarpsPerBlock * 32, 0, stream>>>(src, src_rank, src_pos, weight, T, k, H, world, capacity, out, rows_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace sb200
