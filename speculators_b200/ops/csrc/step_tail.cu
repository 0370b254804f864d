// Tail of one training-time-test pass in one launch: masked-mean reduction of the per-row
// loss with a constant decay factor, full / conditional accuracy counters, and the in-place
// update of the "all previous passes were right" flags.
//
//   loss        = decay * sum_r(row_loss[r] * mask[r]) / (sum_r mask[r] + eps)
//   cond_total  = sum_r prev[r]                     (before the update)
//   prev[r]    &= (pred[r] == target[r])
//   correct     = sum_r (prev[r] & mask[r])         (after the update)
//   total       = sum_r mask[r]
//   weight[r]   = decay * mask[r] / (sum mask + eps)     (d loss / d row_loss[r], for backward)
//
// One CTA (rows are a few thousand): two passes over the rows, block-wide sums in between.
#include "common.cuh"

namespace sb200 {
namespace {

constexpr int kTailThreads = 1024;

__global__ void __launch_bounds__(kTailThreads)
step_tail_kernel(const float* __restrict__ row_loss, const int* __restrict__ pred, const int* __restrict__ target,
                 const uint8_t* __restrict__ mask, uint8_t* __restrict__ prev, int rows, float decay, float eps,
                 float* __restrict__ out, float* __restrict__ weight) {
  __shared__ float scratch[33];
  float s_loss = 0.f, s_mask = 0.f, s_prev = 0.f, s_correct = 0.f;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) {
    const bool m = mask[r] != 0;
    const bool was = prev[r] != 0;
    const bool now = was && (pred[r] == target[r]);
    prev[r] = now ? 1 : 0;
    s_prev += was ? 1.f : 0.f;
    s_mask += m ? 1.f : 0.f;
    s_correct += (now && m) ? 1.f : 0.f;
    s_loss += m ? row_loss[r] : 0.f;
  }
  s_loss = block_sum(s_loss, scratch);
  __syncthreads();
  s_mask = block_sum(s_mask, scratch);
  __syncthreads();
  s_prev = block_sum(s_prev, scratch);
  __syncthreads();
  s_correct = block_sum(s_correct, scratch);
  __shared__ float scale_s;
  if (threadIdx.x == 0) {
    const float scale = decay / (s_mask + eps);
    scale_s = scale;
    out[0] = s_loss * scale;
    out[1] = s_correct;
    out[2] = s_mask;
    out[3] = s_prev;
  }
  __syncthreads();
  const float scale = scale_s;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) weight[r] = mask[r] != 0 ? scale : 0.f;
}

}  // namespace

// out: float[4] = loss, correct, total, cond_total.  weight: float[rows].
void launch_step_tail(const float* row_loss, const int* pred, const int* target, const uint8_t* mask, uint8_t* prev, int rows,
                      float decay, float eps, float* out, float* weight, cudaStream_t stream) {
  count_launch(1);
  step_tail_kernel<<<1, kTailThreads, 0, stream>>>(row_loss, pred, target, mask, prev, rows, decay, eps, out, weight);
}

}  // namespace sb200
