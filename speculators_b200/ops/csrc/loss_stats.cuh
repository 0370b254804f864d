// Online-softmax statistics of a logits row (and, for the KL divergence, of the target row with
// the cross term carried along), shared by the row-loss kernels and by the GEMM epilogue that
// computes the same statistics tile by tile.
#pragma once
#include "common.cuh"

namespace sb200 {

struct RowStats {
  float m, z;
  float best;
  int best_idx;
};

__device__ __forceinline__ void online_update(RowStats& s, const float (&x)[8], int col0) {
  float vmax = x[0];
#pragma unroll
  for (int j = 1; j < 8; ++j) vmax = fmaxf(vmax, x[j]);
  const float m_new = fmaxf(s.m, vmax);
  float add = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) add += __expf(x[j] - m_new);
  s.z = s.z * __expf(s.m - m_new) + add;
  s.m = m_new;
  if (vmax > s.best) {
    s.best = vmax;
#pragma unroll
    for (int j = 7; j >= 0; --j)
      if (x[j] == vmax) s.best_idx = col0 + j;  // lowest index wins inside the vector
  }
}

// KL(target || draft) in one pass: next to the target row's online softmax statistics keep
// A = sum_v e^{t_v - m}(t_v - x_v) relative to the same running max m, so that
// sum_v p_v (t_v - x_v) = A / Z needs no second read of the rows.
__device__ __forceinline__ void online_update_kl(RowStats& s, float& A, const float (&t)[8], const float (&x)[8], int col0) {
  float vmax = t[0];
#pragma unroll
  for (int j = 1; j < 8; ++j) vmax = fmaxf(vmax, t[j]);
  const float m_new = fmaxf(s.m, vmax);
  float add = 0.f, add_a = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float e = __expf(t[j] - m_new);
    add += e;
    if (e > 0.f) add_a += e * (t[j] - x[j]);  // zero-probability targets contribute nothing
  }
  const float resc = __expf(s.m - m_new);
  s.z = s.z * resc + add;
  A = A * resc + add_a;
  s.m = m_new;
  if (vmax > s.best) {
    s.best = vmax;
#pragma unroll
    for (int j = 7; j >= 0; --j)
      if (t[j] == vmax) s.best_idx = col0 + j;
  }
}

__device__ __forceinline__ void online_update_kl_scalar(RowStats& s, float& A, float t, float x, int col) {
  const float m_new = fmaxf(s.m, t);
  const float e = __expf(t - m_new), resc = __expf(s.m - m_new);
  s.z = s.z * resc + e;
  A = A * resc + (e > 0.f ? e * (t - x) : 0.f);
  s.m = m_new;
  if (t > s.best) {
    s.best = t;
    s.best_idx = col;
  }
}

__device__ __forceinline__ void online_update_scalar(RowStats& s, float x, int col) {
  const float m_new = fmaxf(s.m, x);
  s.z = s.z * __expf(s.m - m_new) + __expf(x - m_new);
  s.m = m_new;
  if (x > s.best) {
    s.best = x;
    s.best_idx = col;
  }
}

// Merge of two partial statistics of the same row (disjoint column sets): running max, rescaled
// sum-exp, larger best value with the lower column index on ties.
__device__ __forceinline__ void merge_stats(RowStats& a, const RowStats& b) {
  const float m = fmaxf(a.m, b.m);
  const float za = (a.m == -INFINITY) ? 0.f : a.z * __expf(a.m - m);
  const float zb = (b.m == -INFINITY) ? 0.f : b.z * __expf(b.m - m);
  a.m = m;
  a.z = za + zb;
  if (b.best > a.best || (b.best == a.best && b.best_idx < a.best_idx)) {
    a.best = b.best;
    a.best_idx = b.best_idx;
  }
}
// The same for the target row of the KL divergence: A is relative to the running max.
__device__ __forceinline__ void merge_stats_kl(RowStats& a, float& A_a, const RowStats& b, float A_b) {
  const float m = fmaxf(a.m, b.m);
  const float ra = (a.m == -INFINITY) ? 0.f : __expf(a.m - m), rb = (b.m == -INFINITY) ? 0.f : __expf(b.m - m);
  A_a = A_a * ra + A_b * rb;
  a.z = a.z * ra + b.z * rb;
  a.m = m;
  if (b.best > a.best || (b.best == a.best && b.best_idx < a.best_idx)) {
    a.best = b.best;
    a.best_idx = b.best_idx;
  }
}

}  // namespace sb200
