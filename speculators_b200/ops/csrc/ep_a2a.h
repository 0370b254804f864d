// Launchers of the expert-parallel token exchange kernels (ep_a2a.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sb200 {

// Base address of one buffer on every rank, as mapped into this process (index = rank).
struct EpPeers {
  unsigned long long ptr[16];
};

// Slot s: row src_row[s] of `src` (scaled by scale[s] if given) -> row dst_pos[s] of rank
// dst_rank[s]'s buffer `dst`.  Afterwards `seq` is published at index my_rank of every
// rank's flag array.  src_rows / capacity: rows of `src` / of every rank's buffer (checked in the debug build).
int launch_ep_push(const __nv_bfloat16* src, const int* src_row, const int* dst_rank, const int* dst_pos, const float* scale,
                   int n_slots, int H, int src_rows, int capacity, const EpPeers& dst, unsigned int* done_counter, const EpPeers& flags,
                   int my_rank, int world,
                   uint32_t seq, cudaStream_t stream);
int launch_ep_signal(const EpPeers& flags, int my_rank, int world, uint32_t seq, cudaStream_t stream);
// Bounded wait until all `world` entries of the local flag array have reached `seq`; status 51 on expiry.
int launch_ep_wait(const uint32_t* flags_local, int world, uint32_t seq, uint32_t spin_limit, int* status, cudaStream_t stream);
// out[t] = sum_j weight[t*k+j] * row src_pos[t*k+j] of rank src_rank[t*k+j]'s buffer (rank < 0: skipped);
// rows_out (optional, [T*k, H]): the gathered rows themselves.
int launch_ep_pull(const EpPeers& src, const int* src_rank, const int* src_pos, const float* weight, int T, int k, int H, int world,
                   int capacity, __nv_bfloat16* out, __nv_bfloat16* rows_out, cudaStream_t stream);

}  // namespace sb200
