// Device-to-device hand-off of verifier hidden states over NVLink peer memory.
//
// The consumer (a trainer rank) owns a ring of fixed-size slots plus one control record
// per slot in peer-visible memory; the producer (the GPU that ran the verifier forward)
// maps both through CUDA IPC.  Per slot the control record holds
//
//   word 0  seq    written by the producer after the payload: "sample number seq is here"
//   word 1  ack    written by the consumer after it copied the payload out: "slot is free
//                  for the sample after seq"
//   word 2  rows   word 3  width      payload shape, written before seq
//
// push:  (bounded) wait until ack == seq - n_slots (the previous occupant was consumed),
//        copy the payload into the peer slot with 16-byte stores, fence, release-store seq.
// pop:   (bounded) wait until seq shows the wanted sample, copy the payload and its shape
//        out of the own slot, release-store ack (from then on the producer may overwrite
//        payload and shape).
//
// Both waits are bounded; when one runs out the kernel writes a code to the caller's
// status word and the copy part is skipped, so the context stays usable and the host
// decides what to do (retry, skip the sample, fail the step).
#include "common.cuh"

namespace sb200 {
namespace hs {

constexpr int kCtlWordsPerSlot = 4;
enum Status : int { kOk = 0, kTimeoutSlotBusy = 21, kTimeoutNoSample = 22 };

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// One thread polls `word` until it equals `want`; *go = 1 on success, 0 (and status) on expiry.
__global__ void wait_word_kernel(const uint32_t* word, uint32_t want, uint32_t spin_limit, int code, int* status, uint32_t* go) {
  for (uint32_t i = 0; i < spin_limit; ++i) {
    if (ld_acquire_sys(word) == want) {
      *go = 1;
      return;
    }
    __nanosleep(256);
  }
  *go = 0;
  atomicCAS(status, kOk, code);
}

// Copy nvec 16-byte vectors if *go; the last block to finish publishes `flag_value` at
// `flag` (release, system scope) after optionally recording the payload shape.
__global__ void __launch_bounds__(256)
copy_publish_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int64_t nvec, const uint32_t* go, uint32_t* ticket,
                    uint32_t* flag, uint32_t flag_value, uint32_t* shape_words, uint32_t rows, uint32_t width,
                    const uint32_t* shape_src, uint32_t* shape_dst) {
  if (*reinterpret_cast<const volatile uint32_t*>(go) == 0) return;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (int64_t)gridDim.x * blockDim.x) dst[i] = src[i];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t t = atomicAdd(ticket, 1u);
    if (t == gridDim.x - 1) {
      *ticket = 0;
      if (shape_words != nullptr) {  // push: record the payload shape before the sample becomes visible
        reinterpret_cast<volatile uint32_t*>(shape_words)[0] = rows;
        reinterpret_cast<volatile uint32_t*>(shape_words)[1] = width;
      }
      if (shape_dst != nullptr) {  // pop: take the shape out before the slot is handed back
        shape_dst[0] = reinterpret_cast<const volatile uint32_t*>(shape_src)[0];
        shape_dst[1] = reinterpret_cast<const volatile uint32_t*>(shape_src)[1];
      }
      __threadfence_system();
      st_release_sys(flag, flag_value);
    }
  }
}

}  // namespace hs

int hs_ring_ctl_words_per_slot() { return hs::kCtlWordsPerSlot; }

static int copy_grid(int64_t nvec) {
  int64_t g = (nvec + 255) / 256;
  const int64_t cap = 4 * kNumSM;
  return (int)(g < 1 ? 1 : (g < cap ? g : cap));
}

// Producer side.  slot_data / slot_ctl: this slot's payload area and control record in the
// consumer's memory (peer mapping).  scratch: two zero-initialised uint32 in local memory.
int launch_hs_push(const void* src, int64_t nbytes, void* slot_data, uint32_t* slot_ctl, uint32_t seq, uint32_t n_slots, uint32_t rows,
                   uint32_t width, uint32_t spin_limit, uint32_t* scratch, int* status, cudaStream_t stream) {
  if (nbytes <= 0 || (nbytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(slot_data) & 15)) return -1;
  const uint32_t free_when = seq >= n_slots ? seq - n_slots : 0u;  // ack of the previous occupant (0 = never used)
  count_launch(2);
  hs::wait_word_kernel<<<1, 1, 0, stream>>>(slot_ctl + 1, free_when, spin_limit, hs::kTimeoutSlotBusy, status, scratch);
  const int64_t nvec = nbytes >> 4;
  hs::copy_publish_kernel<<<copy_grid(nvec), 256, 0, stream>>>(static_cast<const uint4*>(src), static_cast<uint4*>(slot_data), nvec, scratch,
                                                              scratch + 1, slot_ctl + 0, seq, slot_ctl + 2, rows, width, nullptr, nullptr);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// Consumer side.  dst receives the payload and scratch[2..3] its shape (rows, width);
// afterwards ack := seq frees the slot.  scratch: four uint32 in local memory.
int launch_hs_pop(void* dst, int64_t nbytes, const void* slot_data, uint32_t* slot_ctl, uint32_t seq, uint32_t spin_limit, uint32_t* scratch,
                  int* status, cudaStream_t stream) {
  if (nbytes <= 0 || (nbytes & 15) || (reinterpret_cast<uintptr_t>(dst) & 15) || (reinterpret_cast<uintptr_t>(slot_data) & 15)) return -1;
  count_launch(2);
  hs::wait_word_kernel<<<1, 1, 0, stream>>>(slot_ctl + 0, seq, spin_limit, hs::kTimeoutNoSample, status, scratch);
  const int64_t nvec = nbytes >> 4;
  hs::copy_publish_kernel<<<copy_grid(nvec), 256, 0, stream>>>(static_cast<const uint4*>(slot_data), static_cast<uint4*>(dst), nvec, scratch,
                                                              scratch + 1, slot_ctl + 1, seq, nullptr, 0, 0, slot_ctl + 2, scratch + 2);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace sb200
