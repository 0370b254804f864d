// Row-wise distillation losses between draft logits and verifier logits.
//
// One CTA per row.  Forward makes two streaming passes over the row pair: pass 1
// collects the online-softmax statistics (max, sum-exp) and the argmax of both
// rows, pass 2 reduces the selected divergence.  Nothing of size [rows, V] is
// written.  Backward recomputes both softmaxes from the saved statistics and
// writes d(logits) in bf16 with the closed forms
//     kl   : dp - tp
//     rkl  : dp * (log dp - log tp - L)
//     jsd  : 0.5 * dp * (log(dp / mix) - KL(dp || mix)),  mix = (dp + tp) / 2
//     ce   : dp - onehot(argmax tp)
//     tv   : -dp * (1[dp <= tp] - s),  s = sum of dp over {dp <= tp}
// (dp = softmax(logits), tp = softmax(targets), L the row loss).  The same five
// reductions exist as Triton programs in the reference
// (src/speculators/losses/fused.py:91-235); this file is an independent CUDA
// implementation with two additions: the row pairing takes a `shift`
// (logits row r is compared with targets row r + shift, which is how the TTT
// steps of EAGLE-3 align their targets) and both argmaxes are by-products, so the
// accuracy metrics need no extra pass over the vocabulary.
#include "common.cuh"
#include "loss_stats.cuh"

namespace sb200 {

enum LossOp : int { kOpKL = 0, kOpRKL = 1, kOpJSD = 2, kOpCE = 3, kOpTV = 4 };
constexpr int kLossThreads = 512;
constexpr int kNumStats = 5;  // m_d, z_d, m_t, z_t, per-op extra

// Combine per-thread stats across the block.  Result valid in every thread.
__device__ __forceinline__ void block_combine(RowStats& s, float* scratch, int* iscratch) {
  const float M = block_max(s.m, scratch);
  const float z = (s.m == -INFINITY) ? 0.f : s.z * __expf(s.m - M);
  const float Z = block_sum(z, scratch);
  // argmax with lowest-index tie break
  float bv = s.best;
  int bi = s.best_idx;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
      bv = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) {
    scratch[warp] = bv;
    iscratch[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    bv = lane < nwarp ? scratch[lane] : -INFINITY;
    bi = lane < nwarp ? iscratch[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) {
      scratch[32] = bv;
      iscratch[32] = bi;
    }
  }
  __syncthreads();
  s.m = M;
  s.z = Z;
  s.best = scratch[32];
  s.best_idx = iscratch[32];
  __syncthreads();
}

template <int OP>
__global__ void __launch_bounds__(kLossThreads)
loss_fwd_kernel(const __nv_bfloat16* __restrict__ logits, const __nv_bfloat16* __restrict__ targets,
                const uint8_t* __restrict__ active, const int64_t* __restrict__ labels,
                float* __restrict__ loss, float* __restrict__ stats, int* __restrict__ argmax_d,
                int* __restrict__ argmax_t, int rows, int V, int64_t ld_logits, int64_t ld_targets,
                int shift) {
  __shared__ float scratch[33];
  __shared__ int iscratch[33];
  const int r = blockIdx.x;
  if (r >= rows) return;
  float* st = stats + r;
  if (active && !active[r]) {
    if (threadIdx.x == 0) {
      loss[r] = 0.f;
#pragma unroll
      for (int k = 0; k < kNumStats; ++k) st[(int64_t)k * rows] = 0.f;
      if (argmax_d) argmax_d[r] = -1;
      if (argmax_t) argmax_t[r] = -2;
    }
    return;
  }
  const __nv_bfloat16* x = logits + (int64_t)r * ld_logits;
  // with integer labels (token cross-entropy) there is no target row to read
  const bool has_t = targets != nullptr;
  const __nv_bfloat16* t = has_t ? targets + (int64_t)(r + shift) * ld_targets : x;
  const bool vec_ok = ((V & 7) == 0) && ((ld_logits & 7) == 0) && ((ld_targets & 7) == 0);
  const int nvec = vec_ok ? (V >> 3) : 0;

  RowStats sd{-INFINITY, 0.f, -INFINITY, 0x7fffffff}, stt{-INFINITY, 0.f, -INFINITY, 0x7fffffff};
  float kl_a = 0.f;  // OP == kOpKL: the cross term, accumulated in the same pass
  for (int v = threadIdx.x; v < nvec; v += kLossThreads) {
    float a[8], b[8];
    unpack8(ld8(x + (v << 3)), a);
    online_update(sd, a, v << 3);
    if (has_t) {
      unpack8(ld8(t + (v << 3)), b);
      if (OP == kOpKL) online_update_kl(stt, kl_a, b, a, v << 3);
      else online_update(stt, b, v << 3);
    }
  }
  for (int c = (nvec << 3) + threadIdx.x; c < V; c += kLossThreads) {
    const float xc = __bfloat162float(x[c]);
    online_update_scalar(sd, xc, c);
    if (has_t) {
      if (OP == kOpKL) online_update_kl_scalar(stt, kl_a, __bfloat162float(t[c]), xc, c);
      else online_update_scalar(stt, __bfloat162float(t[c]), c);
    }
  }
  const float my_mt = stt.m;  // this thread's running max of the target row, before the block-wide combine
  block_combine(sd, scratch, iscratch);
  if (has_t) {
    block_combine(stt, scratch, iscratch);
  } else {
    stt.m = 0.f;
    stt.z = 1.f;
    int lab = labels ? (int)labels[r + shift] : 0;
    stt.best_idx = lab < 0 ? 0 : (lab >= V ? V - 1 : lab);
  }
  const float lse_d = sd.m + __logf(sd.z);
  const float lse_t = stt.m + __logf(stt.z);

  float acc0 = 0.f, acc1 = 0.f;
  if (OP == kOpCE) {
    if (threadIdx.x == 0) acc0 = lse_d - __bfloat162float(x[stt.best_idx]);
  } else if (OP == kOpKL) {
    // sum_v p_v (t_v - x_v) = (sum over threads of A rescaled to the row max) / Z_t; thread 0 adds
    // the normaliser terms once so that the block sum below yields the row's KL directly
    acc0 = (my_mt == -INFINITY) ? 0.f : kl_a * __expf(my_mt - stt.m) / stt.z;
    if (threadIdx.x == 0) acc0 += lse_d - lse_t;
  } else {
    auto body = [&](float xv, float tv) {
      const float ldp = xv - lse_d, ltp = tv - lse_t;
      const float dp = __expf(ldp), tp = __expf(ltp);
      if (OP == kOpKL) {
        if (tp > 0.f) acc0 += tp * (ltp - ldp);
      } else if (OP == kOpRKL) {
        if (dp > 0.f) acc0 += dp * (ldp - ltp);
      } else if (OP == kOpJSD) {
        const float mx = fmaxf(ldp, ltp);
        const float lm = mx + __logf(__expf(ldp - mx) + __expf(ltp - mx)) - 0.6931471805599453f;
        if (tp > 0.f) acc0 += tp * (ltp - lm);
        if (dp > 0.f) acc1 += dp * (ldp - lm);
      } else {  // TV
        acc0 += fminf(dp, tp);
        if (dp <= tp) acc1 += dp;
      }
    };
    for (int v = threadIdx.x; v < nvec; v += kLossThreads) {
      float a[8], b[8];
      unpack8(ld8(x + (v << 3)), a);
      unpack8(ld8(t + (v << 3)), b);
#pragma unroll
      for (int j = 0; j < 8; ++j) body(a[j], b[j]);
    }
    for (int c = (nvec << 3) + threadIdx.x; c < V; c += kLossThreads)
      body(__bfloat162float(x[c]), __bfloat162float(t[c]));
  }
  acc0 = block_sum(acc0, scratch);
  if (OP == kOpJSD || OP == kOpTV) acc1 = block_sum(acc1, scratch);
  if (threadIdx.x == 0) {
    float L, extra;
    if (OP == kOpKL || OP == kOpRKL) {
      L = acc0;
      extra = acc0;
    } else if (OP == kOpJSD) {
      L = 0.5f * (acc0 + acc1);
      extra = acc1;
    } else if (OP == kOpCE) {
      L = acc0;
      extra = (float)stt.best_idx;
    } else {
      L = 1.f - acc0;
      extra = acc1;
    }
    loss[r] = L;
    st[0] = sd.m;
    st[(int64_t)rows] = sd.z;
    st[(int64_t)2 * rows] = stt.m;
    st[(int64_t)3 * rows] = stt.z;
    st[(int64_t)4 * rows] = extra;
    if (argmax_d) argmax_d[r] = sd.best_idx;
    if (argmax_t) argmax_t[r] = stt.best_idx;
  }
}

// grid.x = total_rows (rows of the d(logits) buffer); rows >= `rows` or with a zero
// upstream gradient are zero-filled.
template <int OP>
__global__ void __launch_bounds__(kLossThreads)
loss_bwd_kernel(const __nv_bfloat16* __restrict__ logits, const __nv_bfloat16* __restrict__ targets,
                const float* __restrict__ grad_out, const float* __restrict__ stats,
                __nv_bfloat16* __restrict__ dlogits, int rows, int total_rows, int V,
                int64_t ld_logits, int64_t ld_targets, int64_t ld_dlogits, int shift) {
  const int r = blockIdx.x;
  if (r >= total_rows) return;
  __nv_bfloat16* d = dlogits + (int64_t)r * ld_dlogits;
  const bool vec_ok =
      ((V & 7) == 0) && ((ld_logits & 7) == 0) && ((ld_targets & 7) == 0) && ((ld_dlogits & 7) == 0);
  const int nvec = vec_ok ? (V >> 3) : 0;
  const float go = r < rows ? grad_out[r] : 0.f;
  // a row the forward skipped (inactive) has all-zero statistics; its sum-exp would be >= 1
  // otherwise.  Such a row gets no gradient whatever the upstream value is.
  const bool skipped = r < rows && stats[(int64_t)rows + r] == 0.f;
  if (go == 0.f || skipped) {
    bf16x8 z;
#pragma unroll
    for (int i = 0; i < 4; ++i) z.v[i] = __floats2bfloat162_rn(0.f, 0.f);
    for (int v = threadIdx.x; v < nvec; v += kLossThreads) st8(d + (v << 3), z);
    for (int c = (nvec << 3) + threadIdx.x; c < V; c += kLossThreads) d[c] = __float2bfloat16(0.f);
    return;
  }
  const __nv_bfloat16* x = logits + (int64_t)r * ld_logits;
  const __nv_bfloat16* t = targets + (int64_t)(r + shift) * ld_targets;
  const float* st = stats + r;
  const float lse_d = st[0] + __logf(st[(int64_t)rows]);
  const float lse_t = (OP == kOpCE) ? 0.f : st[(int64_t)2 * rows] + __logf(st[(int64_t)3 * rows]);
  const float extra = st[(int64_t)4 * rows];
  const int label = (OP == kOpCE) ? (int)extra : -1;

  auto grad = [&](float xv, float tv, int col) -> float {
    const float ldp = xv - lse_d;
    const float dp = __expf(ldp);
    if (OP == kOpCE) return go * (dp - (col == label ? 1.f : 0.f));
    const float ltp = tv - lse_t;
    const float tp = __expf(ltp);
    if (OP == kOpKL) return go * (dp - tp);
    if (OP == kOpRKL) return dp > 0.f ? go * dp * (ldp - ltp - extra) : 0.f;
    if (OP == kOpJSD) {
      const float mx = fmaxf(ldp, ltp);
      const float lm = mx + __logf(__expf(ldp - mx) + __expf(ltp - mx)) - 0.6931471805599453f;
      return dp > 0.f ? go * 0.5f * dp * ((ldp - lm) - extra) : 0.f;
    }
    return -go * dp * ((dp <= tp ? 1.f : 0.f) - extra);  // TV
  };
  for (int v = threadIdx.x; v < nvec; v += kLossThreads) {
    float a[8], b[8], o[8];
    unpack8(ld8(x + (v << 3)), a);
    if (OP != kOpCE) unpack8(ld8(t + (v << 3)), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = grad(a[j], OP != kOpCE ? b[j] : 0.f, (v << 3) + j);
    st8(d + (v << 3), pack8(o));
  }
  for (int c = (nvec << 3) + threadIdx.x; c < V; c += kLossThreads)
    d[c] = __float2bfloat16(
        grad(__bfloat162float(x[c]), OP != kOpCE ? __bfloat162float(t[c]) : 0.f, c));
}

int launch_loss_fwd(int op, const void* logits, const void* targets, const uint8_t* active,
                    const int64_t* labels, float* loss, float* stats, int* argmax_d, int* argmax_t, int rows, int V,
                    int64_t ld_logits, int64_t ld_targets, int shift, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (targets == nullptr && (labels == nullptr || op != kOpCE)) return -3;
  count_launch(1);
#define SB200_LF(OPV)                                                                            \
  loss_fwd_kernel<OPV><<<rows, kLossThreads, 0, stream>>>(                                        \
      (const __nv_bfloat16*)logits, (const __nv_bfloat16*)targets, active, labels, loss, stats,   \
      argmax_d, argmax_t, rows, V, ld_logits, ld_targets, shift)
  switch (op) {
    case kOpKL: SB200_LF(kOpKL); break;
    case kOpRKL: SB200_LF(kOpRKL); break;
    case kOpJSD: SB200_LF(kOpJSD); break;
    case kOpCE: SB200_LF(kOpCE); break;
    case kOpTV: SB200_LF(kOpTV); break;
    default: return -1;
  }
#undef SB200_LF
  return 0;
}

int launch_loss_bwd(int op, const void* logits, const void* targets, const float* grad_out,
                    const float* stats, void* dlogits, int rows, int total_rows, int V,
                    int64_t ld_logits, int64_t ld_targets, int64_t ld_dlogits, int shift,
                    cudaStream_t stream) {
  if (total_rows <= 0) return 0;
  count_launch(1);
#define SB200_LB(OPV)                                                                         \
  loss_bwd_kernel<OPV><<<total_rows, kLossThreads, 0, stream>>>(                               \
      (const __nv_bfloat16*)logits, (const __nv_bfloat16*)targets, grad_out, stats,            \
      (__nv_bfloat16*)dlogits, rows, total_rows, V, ld_logits, ld_targets, ld_dlogits, shift)
  switch (op) {
    case kOpKL: SB200_LB(kOpKL); break;
    case kOpRKL: SB200_LB(kOpRKL); break;
    case kOpJSD: SB200_LB(kOpJSD); break;
    case kOpCE: SB200_LB(kOpCE); break;
    case kOpTV: SB200_LB(kOpTV); break;
    default: return -1;
  }
#undef SB200_LB
  return 0;
}

}  // namespace sb200
