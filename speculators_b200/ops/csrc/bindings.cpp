// Torch operator registration for the sm_100a kernels of this package.
// Every op validates device / dtype / layout, then launches on the current stream.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "attention_params.h"
#include "ep_a2a.h"
#include <ATen/ATen.h>

namespace sb200 {
int rmsnorm_bwd_partial_rows(int rows, int H);
void launch_rmsnorm_fwd(const void*, const void*, const int64_t*, void*, float*, int, int, int64_t,
                        int64_t, float, int64_t, cudaStream_t);
struct BoundsRecord {
  int site;
  long long index;
  long long limit;
};
int read_bounds_norm(BoundsRecord*);
int read_bounds_ep(BoundsRecord*);
void launch_rmsnorm_bwd(const void*, const void*, const void*, const float*, void*, float*, float*,
                        int, int, int64_t, int64_t, int64_t, int, int, cudaStream_t);
void launch_swiglu_fwd(const void*, void*, int64_t, int, cudaStream_t);
void launch_swiglu_bwd(const void*, const void*, void*, int64_t, int, cudaStream_t);
void launch_rope(void*, const int64_t*, const float*, const float*, int64_t, int, int, int, int64_t,
                 int64_t, float, cudaStream_t);
int launch_loss_fwd(int, const void*, const void*, const uint8_t*, const int64_t*, float*, float*, int*,
                    int*, int, int, int64_t, int64_t, int, cudaStream_t);
int launch_loss_bwd(int, const void*, const void*, const float*, const float*, void*, int, int, int,
                    int64_t, int64_t, int64_t, int, cudaStream_t);
int64_t launch_count();
int launch_gemm_tn_tcgen05(const void*, const void*, void*, const void*, int, int, int, int64_t, int64_t, int64_t, int64_t, int,
                           int*, int, cudaStream_t);
int launch_gemm_tcgen05(const void*, const void*, void*, const void*, int, int, int, int64_t, int64_t, int64_t, int64_t, int, int, int,
                        int*, int, cudaStream_t);
void launch_moe_group_plan(const int*, int, int*, int*, cudaStream_t);
int launch_gemm_grouped(const void*, const void*, void*, int, int, int, int64_t, int64_t, int64_t, int, int, int, const int*, const int*, int, int*,
                        cudaStream_t);
int lmhead_stat_words();
int lmhead_tiles_n(int);
int launch_lmhead_logits_stats(const void*, const void*, void*, const void*, int, int, int, int64_t, int64_t, int64_t, int64_t, int, int, float*,
                               int*, cudaStream_t);
int launch_lmhead_combine(const float*, const void*, const uint8_t*, float*, float*, int*, int*, int, int, int64_t, int, cudaStream_t);
int sumsq_num_partials();
int peer_malloc(int64_t, void**);
int peer_free(void*);
int peer_export(void*, unsigned char*);
int peer_import(const unsigned char*, void**);
int peer_close(void*);
int fused_optim_ctl_words();
int fused_optim_num_partials();
int launch_fused_sharded_adamw(int, int, int64_t, const void* const*, void* const*, void* const*, const void*, void*, float*, float*,
                               float*, float*, float*, const float*, int*, uint32_t, cudaStream_t);
int launch_gemm_swiglu(const void*, const void*, void*, void*, int, int, int, int64_t, int64_t, int64_t, int64_t, int*, cudaStream_t);
int launch_gemm_scatter(const void*, const void*, void* const*, int, int, int, int, int, int64_t, int64_t, int*, cudaStream_t);
int tp_allreduce_ctl_words();
int launch_tp_reduce_broadcast(int, int, int, int, const void*, void* const*, void*, const void*, void* const*, int, int*, uint32_t, cudaStream_t);
int hs_ring_ctl_words_per_slot();
int launch_hs_push(const void*, int64_t, void*, uint32_t*, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t, uint32_t*, int*, cudaStream_t);
int launch_hs_pop(void*, int64_t, const void*, uint32_t*, uint32_t, uint32_t, uint32_t*, int*, cudaStream_t);
void launch_step_tail(const float*, const int*, const int*, const uint8_t*, uint8_t*, int, float, float, float*, float*, cudaStream_t);
void launch_sumsq(const void*, int, int64_t, float*, float*, int, cudaStream_t);
void launch_set_hyper(float*, const float*, cudaStream_t);
void launch_adamw(float*, float*, float*, const void*, int, void*, int64_t, const float*,
                  const float*, cudaStream_t);
void launch_muon_momentum(const void*, int, float*, void*, int64_t, const float*, const float*, float, int, float*, float*, cudaStream_t);
void launch_muon_apply(float*, const void*, void*, int64_t, const float*, float, float, float, cudaStream_t);
}  // namespace sb200

namespace {

using at::Tensor;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_rows(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, " must be bfloat16");
  TORCH_CHECK(t.dim() == 2 && t.stride(1) == 1, name, " must be 2-D with unit inner stride");
  TORCH_CHECK(t.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name,
              " rows must be 16-byte aligned");
}

void rmsnorm_fwd(const Tensor& x, const Tensor& w, const c10::optional<Tensor>& row_index, Tensor y,
                 c10::optional<Tensor> rstd, double eps) {
  check_rows(x, "x");
  check_rows(y, "y");
  const int H = (int)y.size(1);
  const int rows = (int)y.size(0);
  TORCH_CHECK(x.size(1) == H && w.numel() == H && w.is_contiguous() &&
                  w.scalar_type() == at::kBFloat16,
              "rmsnorm: shape/dtype mismatch");
  TORCH_CHECK(H % 8 == 0 && H <= 16384, "rmsnorm: H must be a multiple of 8 and <= 16384");
  const int64_t* idx = nullptr;
  if (row_index.has_value()) {
    TORCH_CHECK(row_index->scalar_type() == at::kLong && row_index->is_contiguous() &&
                    row_index->numel() == rows,
                "rmsnorm: row_index must be int64[rows]");
    idx = row_index->data_ptr<int64_t>();
  } else {
    TORCH_CHECK(x.size(0) == rows, "rmsnorm: row count mismatch");
  }
  float* rs = nullptr;
  if (rstd.has_value()) {
    TORCH_CHECK(rstd->scalar_type() == at::kFloat && rstd->numel() == rows && rstd->is_contiguous());
    rs = rstd->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(x.device());
  sb200::launch_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), idx, y.data_ptr(), rs, rows, H, x.stride(0),
                            y.stride(0), (float)eps, x.size(0), cur_stream());
}

void rmsnorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w, const Tensor& rstd, Tensor dx,
                 c10::optional<Tensor> dw, bool accumulate_dx, bool accumulate_dw) {
  check_rows(dy, "dy");
  check_rows(x, "x");
  check_rows(dx, "dx");
  const int rows = (int)x.size(0), H = (int)x.size(1);
  TORCH_CHECK(dy.size(0) == rows && dy.size(1) == H && dx.size(0) == rows && dx.size(1) == H);
  TORCH_CHECK(H % 8 == 0 && H <= 16384);
  c10::cuda::CUDAGuard guard(x.device());
  float* dwp = nullptr;
  float* dwo = nullptr;
  Tensor partial;
  if (dw.has_value()) {
    TORCH_CHECK(dw->scalar_type() == at::kFloat && dw->numel() == H && dw->is_contiguous());
    partial = at::empty({sb200::rmsnorm_bwd_partial_rows(rows, H), H}, dw->options());
    dwp = partial.data_ptr<float>();
    dwo = dw->data_ptr<float>();
  }
  sb200::launch_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr<float>(),
                            dx.data_ptr(), dwp, dwo, rows, H, dy.stride(0), x.stride(0),
                            dx.stride(0), accumulate_dx, accumulate_dw, cur_stream());
}

Tensor swiglu_fwd(const Tensor& gate_up) {
  check_rows(gate_up, "gate_up");
  TORCH_CHECK(gate_up.is_contiguous() && gate_up.size(1) % 16 == 0);
  const int64_t rows = gate_up.size(0);
  const int I = (int)(gate_up.size(1) / 2);
  c10::cuda::CUDAGuard guard(gate_up.device());
  Tensor h = at::empty({rows, I}, gate_up.options());
  sb200::launch_swiglu_fwd(gate_up.data_ptr(), h.data_ptr(), rows, I, cur_stream());
  return h;
}

Tensor swiglu_bwd(const Tensor& dh, const Tensor& gate_up) {
  check_rows(gate_up, "gate_up");
  check_rows(dh, "dh");
  TORCH_CHECK(gate_up.is_contiguous() && dh.is_contiguous() && dh.size(1) * 2 == gate_up.size(1));
  c10::cuda::CUDAGuard guard(gate_up.device());
  Tensor out = at::empty_like(gate_up);
  sb200::launch_swiglu_bwd(dh.data_ptr(), gate_up.data_ptr(), out.data_ptr(), gate_up.size(0),
                           (int)dh.size(1), cur_stream());
  return out;
}

// x: [tokens, >= heads*hd] view (row stride arbitrary); rotates the first `heads` heads in place.
void rope_(Tensor x, const Tensor& positions, const Tensor& cos_t, const Tensor& sin_t, int64_t heads,
           int64_t hd, int64_t rot, double sign) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.dim() == 2 && x.stride(1) == 1);
  TORCH_CHECK(x.size(1) >= heads * hd && rot % 2 == 0 && rot <= hd);
  TORCH_CHECK(positions.scalar_type() == at::kLong && positions.is_contiguous() &&
              positions.numel() == x.size(0));
  TORCH_CHECK(cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat &&
              cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.dim() == 2 &&
              cos_t.size(1) == rot / 2 && sin_t.sizes() == cos_t.sizes());
  c10::cuda::CUDAGuard guard(x.device());
  sb200::launch_rope(x.data_ptr(), positions.data_ptr<int64_t>(), cos_t.data_ptr<float>(),
                     sin_t.data_ptr<float>(), x.size(0), (int)heads, (int)hd, (int)rot, x.stride(0),
                     cos_t.size(0), (float)sign, cur_stream());
}

std::tuple<Tensor, Tensor, Tensor, Tensor> loss_fwd(int64_t op, const Tensor& logits,
                                                    const Tensor& targets,
                                                    const c10::optional<Tensor>& active,
                                                    int64_t shift, int64_t rows) {
  TORCH_CHECK(logits.is_cuda() && targets.is_cuda());
  TORCH_CHECK(logits.scalar_type() == at::kBFloat16 && targets.scalar_type() == at::kBFloat16);
  TORCH_CHECK(logits.dim() == 2 && targets.dim() == 2 && logits.stride(1) == 1 &&
              targets.stride(1) == 1 && logits.size(1) == targets.size(1));
  TORCH_CHECK(rows >= 0 && rows <= logits.size(0) && rows + shift <= targets.size(0) && shift >= 0);
  c10::cuda::CUDAGuard guard(logits.device());
  auto fopt = logits.options().dtype(at::kFloat);
  Tensor loss = at::empty({rows}, fopt);
  Tensor stats = at::empty({5, rows}, fopt);
  Tensor am_d = at::empty({rows}, logits.options().dtype(at::kInt));
  Tensor am_t = at::empty({rows}, logits.options().dtype(at::kInt));
  const uint8_t* act = nullptr;
  if (active.has_value()) {
    TORCH_CHECK((active->scalar_type() == at::kBool || active->scalar_type() == at::kByte) &&
                active->is_contiguous() && active->numel() == rows);
    act = reinterpret_cast<const uint8_t*>(active->data_ptr());
  }
  const int rc = sb200::launch_loss_fwd((int)op, logits.data_ptr(), targets.data_ptr(), act, nullptr,
                                        loss.data_ptr<float>(), stats.data_ptr<float>(),
                                        am_d.data_ptr<int>(), am_t.data_ptr<int>(), (int)rows,
                                        (int)logits.size(1), logits.stride(0), targets.stride(0),
                                        (int)shift, cur_stream());
  TORCH_CHECK(rc == 0, "loss_fwd: unknown op ", op);
  return {loss, stats, am_d, am_t};
}

// ---- grouped (mixture-of-experts) products ----------------------------------------------------
// counts int32[E] (device) -> (seg int32[E + 1], mtile_start int32[E + 1]): 128-row aligned segment offsets of the
// padded row order and the prefix sum of 256-row tiles per expert.  Nothing is read back to the host.
std::tuple<Tensor, Tensor> moe_group_plan(const Tensor& counts) {
  TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == at::kInt && counts.is_contiguous() && counts.dim() == 1);
  c10::cuda::CUDAGuard guard(counts.device());
  const int64_t E = counts.numel();
  Tensor seg = at::empty({E + 1}, counts.options());
  Tensor mts = at::empty({E + 1}, counts.options());
  sb200::launch_moe_group_plan(counts.data_ptr<int>(), (int)E, seg.data_ptr<int>(), mts.data_ptr<int>(), cur_stream());
  return {seg, mts};
}

// out[R, N] = x[R, K] . w_e^T for the rows of expert e (w: [E, N, K]); with `transposed` the weight is
// [E, K, N] read in place (input gradient: out[R, N] = x[R, K] . w_e).  Rows follow the padded order of moe_group_plan.
void gemm_grouped_rows(const Tensor& x, const Tensor& w, Tensor out, bool transposed, const Tensor& seg, const Tensor& mts, Tensor status) {
  check_rows(x, "x");
  check_rows(out, "out");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kBFloat16 && w.dim() == 3 && w.is_contiguous(), "w must be a contiguous bf16 [E, ., .] stack");
  const int64_t E = w.size(0), R = x.size(0), K = x.size(1);
  const int64_t N = transposed ? w.size(2) : w.size(1);
  TORCH_CHECK((transposed ? w.size(1) : w.size(2)) == K && out.size(0) == R && out.size(1) == N, "gemm_grouped_rows: shape mismatch");
  TORCH_CHECK(K % 128 == 0 && N % 256 == 0 && R % 128 == 0, "gemm_grouped_rows: K % 128, N % 256 and rows % 128 must be 0");
  TORCH_CHECK(seg.is_cuda() && seg.scalar_type() == at::kInt && seg.numel() == E + 1 && mts.scalar_type() == at::kInt && mts.numel() == E + 1);
  c10::cuda::CUDAGuard guard(x.device());
  const int rc = sb200::launch_gemm_grouped(x.data_ptr(), w.data_ptr(), out.data_ptr(), (int)R, (int)N, (int)K, x.stride(0), w.stride(1),
                                            out.stride(0), 0, 1, transposed ? 1 : 0, seg.data_ptr<int>(), mts.data_ptr<int>(), (int)E,
                                            status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "gemm_grouped_rows launch failed (", rc, ")");
}

// dw[e] (=, +=) dy[seg_e, :]^T . x[seg_e, :]  (dw: [E, M, N], dy: [R, M], x: [R, N]); an expert without rows gets zeros (store) / is left alone (accumulate).
void gemm_grouped_wgrad(const Tensor& dy, const Tensor& x, Tensor dw, bool accumulate, const Tensor& seg, const Tensor& mts, Tensor status) {
  check_rows(dy, "dy");
  check_rows(x, "x");
  TORCH_CHECK(dw.is_cuda() && dw.scalar_type() == at::kBFloat16 && dw.dim() == 3 && dw.is_contiguous());
  const int64_t E = dw.size(0), M = dw.size(1), N = dw.size(2), R = dy.size(0);
  TORCH_CHECK(dy.size(1) == M && x.size(1) == N && x.size(0) == R && R % 128 == 0, "gemm_grouped_wgrad: shape mismatch");
  TORCH_CHECK(seg.is_cuda() && seg.scalar_type() == at::kInt && seg.numel() == E + 1);
  c10::cuda::CUDAGuard guard(x.device());
  const int rc = sb200::launch_gemm_grouped(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), (int)M, (int)N, (int)R, dy.stride(0), x.stride(0), N,
                                            accumulate ? 1 : 0, 2, 1, seg.data_ptr<int>(), mts.data_ptr<int>(), (int)E, status.data_ptr<int>(),
                                            cur_stream());
  TORCH_CHECK(rc == 0, "gemm_grouped_wgrad launch failed (", rc, ")");
}

// lm_head product fused with the row loss: logits = x @ w^T on the tcgen05 kernel whose epilogue also
// reduces every (row, 256-column tile) of the logits and of targets[row + shift] to online-softmax
// records; a second kernel merges them into the outputs of loss_fwd.  op 0 (KL) or 3 (CE on the argmax).
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> lmhead_loss_fwd(int64_t op, const Tensor& x, const Tensor& w, const Tensor& targets,
                                                                   const c10::optional<Tensor>& active, int64_t shift, int64_t rows,
                                                                   Tensor status) {
  check_rows(x, "x");
  check_rows(w, "w");
  check_rows(targets, "targets");
  TORCH_CHECK(op == 0 || op == 3, "lmhead_loss_fwd: op 0 (kl) or 3 (ce)");
  const int64_t M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(w.size(1) == K && targets.size(1) == N && N % 8 == 0, "lmhead_loss_fwd: shape mismatch");
  TORCH_CHECK(rows >= 0 && rows <= M && shift >= 0 && rows + shift <= targets.size(0));
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  c10::cuda::CUDAGuard guard(x.device());
  auto fopt = x.options().dtype(at::kFloat);
  const int tiles_n = sb200::lmhead_tiles_n((int)N);
  Tensor logits = at::empty({M, N}, x.options());
  Tensor partial = at::empty({M, tiles_n, sb200::lmhead_stat_words()}, fopt);
  Tensor loss = at::empty({rows}, fopt);
  Tensor stats = at::empty({5, rows}, fopt);
  Tensor am_d = at::empty({rows}, x.options().dtype(at::kInt));
  Tensor am_t = at::empty({rows}, x.options().dtype(at::kInt));
  const uint8_t* act = nullptr;
  if (active.has_value()) {
    TORCH_CHECK((active->scalar_type() == at::kBool || active->scalar_type() == at::kByte) && active->is_contiguous() &&
                active->numel() == rows);
    act = reinterpret_cast<const uint8_t*>(active->data_ptr());
  }
  int rc = sb200::launch_lmhead_logits_stats(x.data_ptr(), w.data_ptr(), logits.data_ptr(), targets.data_ptr(), (int)M, (int)N, (int)K,
                                             x.stride(0), w.stride(0), logits.stride(0), targets.stride(0), (int)targets.size(0),
                                             (int)shift, partial.data_ptr<float>(), status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "lmhead_loss_fwd: GEMM launch failed (", rc, ")");
  rc = sb200::launch_lmhead_combine(partial.data_ptr<float>(), logits.data_ptr(), act, loss.data_ptr<float>(), stats.data_ptr<float>(),
                                    am_d.data_ptr<int>(), am_t.data_ptr<int>(), (int)rows, tiles_n, logits.stride(0), (int)op, cur_stream());
  TORCH_CHECK(rc == 0, "lmhead_loss_fwd: combine launch failed (", rc, ")");
  return {logits, loss, stats, am_d, am_t};
}

// Token cross-entropy: labels int64[rows]; rows with keep == 0 cost nothing and get loss 0.
std::tuple<Tensor, Tensor> ce_label_fwd(const Tensor& logits, const Tensor& labels, const c10::optional<Tensor>& keep) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == at::kBFloat16 && logits.dim() == 2 && logits.stride(1) == 1);
  const int64_t rows = logits.size(0);
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == rows);
  c10::cuda::CUDAGuard guard(logits.device());
  auto fopt = logits.options().dtype(at::kFloat);
  Tensor loss = at::empty({rows}, fopt);
  Tensor stats = at::empty({5, rows}, fopt);
  const uint8_t* act = nullptr;
  if (keep.has_value()) {
    TORCH_CHECK((keep->scalar_type() == at::kBool || keep->scalar_type() == at::kByte) && keep->is_contiguous() && keep->numel() == rows);
    act = reinterpret_cast<const uint8_t*>(keep->data_ptr());
  }
  const int rc = sb200::launch_loss_fwd(3, logits.data_ptr(), nullptr, act, labels.data_ptr<int64_t>(), loss.data_ptr<float>(),
                                        stats.data_ptr<float>(), nullptr, nullptr, (int)rows, (int)logits.size(1),
                                        logits.stride(0), logits.stride(0), 0, cur_stream());
  TORCH_CHECK(rc == 0, "ce_label_fwd failed (", rc, ")");
  return {loss, stats};
}

Tensor loss_bwd(int64_t op, const Tensor& logits, const Tensor& targets, const Tensor& grad_out,
                const Tensor& stats, int64_t shift, int64_t rows) {
  TORCH_CHECK(grad_out.scalar_type() == at::kFloat && grad_out.is_contiguous() &&
              grad_out.numel() == rows);
  TORCH_CHECK(stats.scalar_type() == at::kFloat && stats.is_contiguous() && stats.size(0) == 5 &&
              stats.size(1) == rows);
  c10::cuda::CUDAGuard guard(logits.device());
  Tensor d = at::empty({logits.size(0), logits.size(1)}, logits.options());
  const int rc = sb200::launch_loss_bwd(
      (int)op, logits.data_ptr(), targets.data_ptr(), grad_out.data_ptr<float>(),
      stats.data_ptr<float>(), d.data_ptr(), (int)rows, (int)logits.size(0), (int)logits.size(1),
      logits.stride(0), targets.stride(0), d.stride(0), (int)shift, cur_stream());
  TORCH_CHECK(rc == 0, "loss_bwd: unknown op ", op);
  return d;
}

void sumsq(const Tensor& g, Tensor out, bool accumulate) {
  TORCH_CHECK(g.is_cuda() && g.is_contiguous() && out.scalar_type() == at::kFloat && out.numel() >= 1);
  TORCH_CHECK(g.scalar_type() == at::kBFloat16 || g.scalar_type() == at::kFloat);
  c10::cuda::CUDAGuard guard(g.device());
  Tensor partial = at::empty({sb200::sumsq_num_partials()}, out.options());
  sb200::launch_sumsq(g.data_ptr(), g.scalar_type() == at::kBFloat16, g.numel(),
                      partial.data_ptr<float>(), out.data_ptr<float>(), accumulate, cur_stream());
}

// Muon, first half: buf <- momentum update of the clipped gradient, out <- bf16 (nesterov) update,
// out_sumsq[0] <- squared Frobenius norm of out.  partial: fp32[sumsq_num_partials()] scratch.
void muon_momentum(const Tensor& grad, Tensor buf, Tensor out, const Tensor& hyper, const Tensor& norm_sq, double momentum, bool nesterov,
                   Tensor partial, Tensor out_sumsq) {
  const int64_t n = buf.numel();
  TORCH_CHECK(grad.is_cuda() && grad.is_contiguous() && grad.numel() == n &&
              (grad.scalar_type() == at::kBFloat16 || grad.scalar_type() == at::kFloat));
  TORCH_CHECK(buf.is_cuda() && buf.scalar_type() == at::kFloat && buf.is_contiguous());
  TORCH_CHECK(out.is_cuda() && out.scalar_type() == at::kBFloat16 && out.is_contiguous() && out.numel() == n);
  TORCH_CHECK(hyper.is_cuda() && hyper.scalar_type() == at::kFloat && hyper.numel() >= 9);
  TORCH_CHECK(norm_sq.is_cuda() && norm_sq.scalar_type() == at::kFloat && norm_sq.numel() >= 1);
  TORCH_CHECK(partial.is_cuda() && partial.scalar_type() == at::kFloat && partial.numel() >= sb200::sumsq_num_partials());
  TORCH_CHECK(out_sumsq.is_cuda() && out_sumsq.scalar_type() == at::kFloat && out_sumsq.numel() >= 1);
  c10::cuda::CUDAGuard guard(buf.device());
  sb200::launch_muon_momentum(grad.data_ptr(), grad.scalar_type() == at::kBFloat16, buf.data_ptr<float>(), out.data_ptr(), n,
                              hyper.data_ptr<float>(), norm_sq.data_ptr<float>(), (float)momentum, nesterov ? 1 : 0,
                              partial.data_ptr<float>(), out_sumsq.data_ptr<float>(), cur_stream());
}

// Muon, second half: master <- master * (1 - lr * wd) - lr * adjust * update, w16 <- bf16(master); lr = hyper[0] * lr_ratio.
void muon_apply(Tensor master, const Tensor& update, c10::optional<Tensor> w16, const Tensor& hyper, double lr_ratio, double weight_decay,
                double adjust) {
  const int64_t n = master.numel();
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous());
  TORCH_CHECK(update.is_cuda() && update.scalar_type() == at::kBFloat16 && update.is_contiguous() && update.numel() == n);
  TORCH_CHECK(hyper.is_cuda() && hyper.scalar_type() == at::kFloat && hyper.numel() >= 9);
  void* w = nullptr;
  if (w16.has_value()) {
    TORCH_CHECK(w16->is_cuda() && w16->scalar_type() == at::kBFloat16 && w16->numel() == n && w16->is_contiguous());
    w = w16->data_ptr();
  }
  c10::cuda::CUDAGuard guard(master.device());
  sb200::launch_muon_apply(master.data_ptr<float>(), update.data_ptr(), w, n, hyper.data_ptr<float>(), (float)lr_ratio,
                           (float)weight_decay, (float)adjust, cur_stream());
}

int64_t sumsq_num_partials_binding() { return sb200::sumsq_num_partials(); }

// hyper (fp32[16], CUDA) <- vals (<= 16 host doubles), passed as kernel arguments.
void set_hyper(Tensor hyper, std::vector<double> vals) {
  TORCH_CHECK(hyper.is_cuda() && hyper.scalar_type() == at::kFloat && hyper.numel() >= 16 && hyper.is_contiguous());
  TORCH_CHECK(vals.size() <= 16);
  float host[16] = {0};
  for (size_t i = 0; i < vals.size(); ++i) host[i] = (float)vals[i];
  c10::cuda::CUDAGuard guard(hyper.device());
  sb200::launch_set_hyper(hyper.data_ptr<float>(), host, at::cuda::getCurrentCUDAStream());
}

void adamw(Tensor master, Tensor m, Tensor v, const Tensor& grad, c10::optional<Tensor> w16,
           const Tensor& hyper, const c10::optional<Tensor>& norm_sq) {
  const int64_t n = master.numel();
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous());
  TORCH_CHECK(m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat && m.numel() == n &&
              v.numel() == n && m.is_contiguous() && v.is_contiguous());
  TORCH_CHECK(grad.numel() == n && grad.is_contiguous() &&
              (grad.scalar_type() == at::kBFloat16 || grad.scalar_type() == at::kFloat));
  TORCH_CHECK(hyper.scalar_type() == at::kFloat && hyper.numel() >= 9 && hyper.is_cuda());
  void* w = nullptr;
  if (w16.has_value()) {
    TORCH_CHECK(w16->scalar_type() == at::kBFloat16 && w16->numel() == n && w16->is_contiguous());
    w = w16->data_ptr();
  }
  const float* ns = nullptr;
  if (norm_sq.has_value()) {
    TORCH_CHECK(norm_sq->scalar_type() == at::kFloat && norm_sq->is_cuda());
    ns = norm_sq->data_ptr<float>();
  }
  c10::cuda::CUDAGuard guard(master.device());
  sb200::launch_adamw(master.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
                      grad.data_ptr(), grad.scalar_type() == at::kBFloat16, w, n,
                      hyper.data_ptr<float>(), ns, cur_stream());
}

int64_t launch_count() { return sb200::launch_count(); }

// ---- peer memory + fused sharded optimizer -------------------------------------------------
int64_t peer_alloc(int64_t nbytes) {
  void* p = nullptr;
  TORCH_CHECK(sb200::peer_malloc(nbytes, &p) == 0, "peer_alloc: cudaMalloc of ", nbytes, " bytes failed");
  return reinterpret_cast<int64_t>(p);
}
void peer_release(int64_t ptr) { sb200::peer_free(reinterpret_cast<void*>(ptr)); }
Tensor peer_handle(int64_t ptr) {
  Tensor h = at::empty({64}, at::TensorOptions().dtype(at::kByte));
  TORCH_CHECK(sb200::peer_export(reinterpret_cast<void*>(ptr), h.data_ptr<uint8_t>()) == 0, "peer_handle: cudaIpcGetMemHandle failed");
  return h;
}
int64_t peer_open(const Tensor& handle) {
  TORCH_CHECK(handle.device().is_cpu() && handle.scalar_type() == at::kByte && handle.numel() == 64 && handle.is_contiguous());
  void* p = nullptr;
  TORCH_CHECK(sb200::peer_import(handle.data_ptr<uint8_t>(), &p) == 0, "peer_open: cudaIpcOpenMemHandle failed");
  return reinterpret_cast<int64_t>(p);
}
void peer_close(int64_t ptr) { sb200::peer_close(reinterpret_cast<void*>(ptr)); }
// Non-owning tensor over raw device memory (the caller keeps the allocation alive).
Tensor peer_tensor(int64_t ptr, int64_t numel, at::ScalarType dtype, int64_t device) {
  auto opts = at::TensorOptions().dtype(dtype).device(at::kCUDA, (c10::DeviceIndex)device);
  return at::from_blob(reinterpret_cast<void*>(ptr), {numel}, opts);
}
int64_t fused_optim_ctl_words() { return sb200::fused_optim_ctl_words(); }

// ---- tail of a training-time-test pass --------------------------------------------------------
// row_loss fp32[rows], pred / target int32[rows], mask uint8[rows] (0 / non-0), prev uint8 or bool [rows] (updated in place).
// Returns (out fp32[4] = loss, correct, total, cond_total; weight fp32[rows] = d loss / d row_loss).
std::tuple<Tensor, Tensor> step_tail(const Tensor& row_loss, const Tensor& pred, const Tensor& target, const Tensor& mask, Tensor prev,
                                     double decay, double eps) {
  const int64_t rows = row_loss.numel();
  TORCH_CHECK(row_loss.is_cuda() && row_loss.scalar_type() == at::kFloat && row_loss.is_contiguous());
  TORCH_CHECK(pred.scalar_type() == at::kInt && target.scalar_type() == at::kInt && pred.is_contiguous() && target.is_contiguous());
  TORCH_CHECK(pred.numel() >= rows && target.numel() >= rows && mask.numel() >= rows && prev.numel() >= rows);
  TORCH_CHECK((mask.scalar_type() == at::kByte || mask.scalar_type() == at::kBool) && mask.is_contiguous());
  TORCH_CHECK((prev.scalar_type() == at::kByte || prev.scalar_type() == at::kBool) && prev.is_contiguous());
  c10::cuda::CUDAGuard guard(row_loss.device());
  Tensor out = at::empty({4}, row_loss.options());
  Tensor weight = at::empty({rows}, row_loss.options());
  sb200::launch_step_tail(row_loss.data_ptr<float>(), pred.data_ptr<int>(), target.data_ptr<int>(),
                          static_cast<const uint8_t*>(mask.data_ptr()), static_cast<uint8_t*>(prev.data_ptr()), (int)rows, (float)decay,
                          (float)eps, out.data_ptr<float>(), weight.data_ptr<float>(), cur_stream());
  return {out, weight};
}

// ---- hidden-state ring (device-to-device hand-off) -----------------------------------------
int64_t hs_ring_ctl_words() { return sb200::hs_ring_ctl_words_per_slot(); }

// src: contiguous CUDA tensor (payload, size a multiple of 16 bytes); slot_data / slot_ctl: device addresses
// of the slot in the consumer's memory as mapped into this process; scratch: int32[2] zeros on this device.
void hs_push(const Tensor& src, int64_t slot_data, int64_t slot_ctl, int64_t seq, int64_t n_slots, int64_t rows, int64_t width,
             int64_t spin_limit, Tensor scratch, Tensor status) {
  TORCH_CHECK(src.is_cuda() && src.is_contiguous() && scratch.is_cuda() && status.is_cuda());
  TORCH_CHECK(scratch.scalar_type() == at::kInt && scratch.numel() >= 2 && status.scalar_type() == at::kInt && status.numel() >= 1);
  c10::cuda::CUDAGuard guard(src.device());
  const int rc = sb200::launch_hs_push(src.data_ptr(), (int64_t)src.nbytes(), reinterpret_cast<void*>(slot_data),
                                       reinterpret_cast<uint32_t*>(slot_ctl), (uint32_t)seq, (uint32_t)n_slots, (uint32_t)rows, (uint32_t)width,
                                       (uint32_t)spin_limit, reinterpret_cast<uint32_t*>(scratch.data_ptr<int>()), status.data_ptr<int>(),
                                       cur_stream());
  TORCH_CHECK(rc == 0, "hs_push: bad arguments or launch failure (", rc, ")");
}

void hs_pop(Tensor dst, int64_t slot_data, int64_t slot_ctl, int64_t seq, int64_t spin_limit, Tensor scratch, Tensor status) {
  TORCH_CHECK(dst.is_cuda() && dst.is_contiguous() && scratch.is_cuda() && status.is_cuda());
  TORCH_CHECK(scratch.scalar_type() == at::kInt && scratch.numel() >= 4 && status.scalar_type() == at::kInt && status.numel() >= 1);
  c10::cuda::CUDAGuard guard(dst.device());
  const int rc = sb200::launch_hs_pop(dst.data_ptr(), (int64_t)dst.nbytes(), reinterpret_cast<const void*>(slot_data),
                                      reinterpret_cast<uint32_t*>(slot_ctl), (uint32_t)seq, (uint32_t)spin_limit,
                                      reinterpret_cast<uint32_t*>(scratch.data_ptr<int>()), status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "hs_pop: bad arguments or launch failure (", rc, ")");
}

// g_ptrs / w_ptrs / ctl_ptrs: int64 CPU tensors [world] of device addresses valid on this rank.
// g_mc / w_mc: multicast (NVSwitch) addresses of the gradient / weight buffers, 0 = use the per-peer addresses.
void fused_sharded_adamw(int64_t world, int64_t rank, int64_t shard, const Tensor& g_ptrs, const Tensor& w_ptrs, const Tensor& ctl_ptrs,
                         int64_t g_mc, int64_t w_mc, Tensor master, Tensor m, Tensor v, Tensor gred, const Tensor& hyper, Tensor status, int64_t spin_limit) {
  // validated before the fixed-size pointer arrays below are filled
  TORCH_CHECK(world >= 1 && world <= 8 && rank >= 0 && rank < world && shard > 0 && shard % 8 == 0,
              "fused_sharded_adamw: need 1 <= world <= 8, 0 <= rank < world and a positive shard that is a multiple of 8");
  TORCH_CHECK(spin_limit > 0 && spin_limit <= 0xFFFFFFF0LL, "fused_sharded_adamw: spin_limit out of range");
  TORCH_CHECK(g_ptrs.device().is_cpu() && g_ptrs.scalar_type() == at::kLong && g_ptrs.numel() == world);
  TORCH_CHECK(w_ptrs.device().is_cpu() && w_ptrs.scalar_type() == at::kLong && w_ptrs.numel() == world);
  TORCH_CHECK(ctl_ptrs.device().is_cpu() && ctl_ptrs.scalar_type() == at::kLong && ctl_ptrs.numel() == world);
  for (const Tensor* t : {&master, &m, &v, &gred})
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == shard, "shard buffers must be fp32[shard]");
  TORCH_CHECK(hyper.is_cuda() && hyper.scalar_type() == at::kFloat && hyper.numel() >= 9);
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt);
  c10::cuda::CUDAGuard guard(master.device());
  const void* g[8];
  void* w[8];
  void* c[8];
  for (int q = 0; q < world; ++q) {
    g[q] = reinterpret_cast<const void*>(g_ptrs.data_ptr<int64_t>()[q]);
    w[q] = reinterpret_cast<void*>(w_ptrs.data_ptr<int64_t>()[q]);
    c[q] = reinterpret_cast<void*>(ctl_ptrs.data_ptr<int64_t>()[q]);
  }
  Tensor partial = at::empty({sb200::fused_optim_num_partials()}, master.options());
  const int rc = sb200::launch_fused_sharded_adamw((int)world, (int)rank, shard, g, w, c, reinterpret_cast<const void*>(g_mc),
                                                   reinterpret_cast<void*>(w_mc), master.data_ptr<float>(), m.data_ptr<float>(),
                                                   v.data_ptr<float>(), gred.data_ptr<float>(), partial.data_ptr<float>(),
                                                   hyper.data_ptr<float>(), status.data_ptr<int>(), (uint32_t)spin_limit, cur_stream());
  TORCH_CHECK(rc == 0, "fused_sharded_adamw launch failed (", rc, ")");
}

// ---- gated MLP: gate | up product with the activation in the GEMM epilogue ------------------------
// w: [2 I, K], gate rows first.  Returns (gate_up [M, 2 I], h [M, I] = silu(gate) * up).
std::tuple<Tensor, Tensor> gemm_swiglu(const Tensor& x, const Tensor& w, Tensor status) {
  check_rows(x, "x");
  check_rows(w, "w");
  const int64_t M = x.size(0), K = x.size(1), I = w.size(0) / 2;
  TORCH_CHECK(w.size(1) == K && w.size(0) == 2 * I && I % 128 == 0, "gemm_swiglu: w must be [2 I, K] with I a multiple of 128");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  c10::cuda::CUDAGuard guard(x.device());
  Tensor gate_up = at::empty({M, 2 * I}, x.options());
  Tensor h = at::empty({M, I}, x.options());
  const int rc = sb200::launch_gemm_swiglu(x.data_ptr(), w.data_ptr(), gate_up.data_ptr(), h.data_ptr(), (int)M, (int)I, (int)K, x.stride(0), w.stride(0),
                                           2 * I, I, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "gemm_swiglu launch failed (", rc, ")");
  return {gate_up, h};
}

// ---- row-parallel product of a tensor-parallel layer ------------------------------------------
// partial = x[M, K] . w[N, K]^T; the tile columns owned by rank o (N / world columns each, a multiple of 256) are stored
// into slot `rank` of stage_ptrs[o] ([world][M][N / world] on rank o; int64 CPU tensor of addresses valid on this device).
void gemm_scatter(const Tensor& x, const Tensor& w, const Tensor& stage_ptrs, int64_t rank, Tensor status) {
  check_rows(x, "x");
  check_rows(w, "w");
  const int64_t world = stage_ptrs.numel(), M = x.size(0), K = x.size(1), N = w.size(0);
  TORCH_CHECK(world >= 1 && world <= 8 && rank >= 0 && rank < world, "gemm_scatter: need 1 <= world <= 8 and 0 <= rank < world");
  TORCH_CHECK(stage_ptrs.device().is_cpu() && stage_ptrs.scalar_type() == at::kLong);
  TORCH_CHECK(w.size(1) == K && N % world == 0 && (N / world) % 256 == 0, "gemm_scatter: N / world must be a multiple of 256");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  c10::cuda::CUDAGuard guard(x.device());
  void* stage[8];
  for (int q = 0; q < world; ++q) stage[q] = reinterpret_cast<void*>(stage_ptrs.data_ptr<int64_t>()[q]);
  const int rc = sb200::launch_gemm_scatter(x.data_ptr(), w.data_ptr(), stage, (int)world, (int)rank, (int)M, (int)N, (int)K, x.stride(0),
                                            w.stride(0), status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "gemm_scatter launch failed (", rc, ")");
}

int64_t tp_allreduce_ctl_words() { return sb200::tp_allreduce_ctl_words(); }

// Reduces this rank's column slice of the staged partial products (stage: local [world, rows, cols]), adds the residual's
// slice (local [rows, world * cols], optional) and writes the slice into every rank's output (out_ptrs / out_mc).
void tp_reduce_broadcast(const Tensor& stage, const Tensor& out_ptrs, int64_t out_mc, const c10::optional<Tensor>& residual,
                         const Tensor& ctl_ptrs, int64_t rank, bool barrier, Tensor status, int64_t spin_limit) {
  TORCH_CHECK(stage.is_cuda() && stage.scalar_type() == at::kBFloat16 && stage.dim() == 3 && stage.is_contiguous(), "stage must be bf16 [world, rows, cols]");
  const int64_t world = stage.size(0), rows = stage.size(1), cols = stage.size(2);
  TORCH_CHECK(world >= 1 && world <= 8 && rank >= 0 && rank < world && cols % 8 == 0, "tp_reduce_broadcast: need 1 <= world <= 8 and cols % 8 == 0");
  TORCH_CHECK(spin_limit > 0 && spin_limit <= 0xFFFFFFF0LL, "tp_reduce_broadcast: spin_limit out of range");
  TORCH_CHECK(out_ptrs.device().is_cpu() && out_ptrs.scalar_type() == at::kLong && out_ptrs.numel() == world);
  TORCH_CHECK(ctl_ptrs.device().is_cpu() && ctl_ptrs.scalar_type() == at::kLong && ctl_ptrs.numel() == world);
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  const void* res = nullptr;
  if (residual.has_value()) {
    TORCH_CHECK(residual->is_cuda() && residual->scalar_type() == at::kBFloat16 && residual->is_contiguous() && residual->numel() == rows * world * cols &&
                (reinterpret_cast<uintptr_t>(residual->data_ptr()) & 15) == 0, "residual must be contiguous bf16 [rows, world * cols]");
    res = residual->data_ptr();
  }
  c10::cuda::CUDAGuard guard(stage.device());
  void* out[8];
  void* ctl[8];
  for (int q = 0; q < world; ++q) {
    out[q] = reinterpret_cast<void*>(out_ptrs.data_ptr<int64_t>()[q]);
    ctl[q] = reinterpret_cast<void*>(ctl_ptrs.data_ptr<int64_t>()[q]);
    TORCH_CHECK((reinterpret_cast<uintptr_t>(out[q]) & 15) == 0 && ctl[q] != nullptr, "tp_reduce_broadcast: misaligned output / missing control block");
  }
  const int rc = sb200::launch_tp_reduce_broadcast((int)world, (int)rank, (int)rows, (int)cols, stage.data_ptr(), out, reinterpret_cast<void*>(out_mc), res,
                                                   ctl, barrier ? 1 : 0, status.data_ptr<int>(), (uint32_t)spin_limit, cur_stream());
  TORCH_CHECK(rc == 0, "tp_reduce_broadcast launch failed (", rc, ")");
}

// ---- debug build: index checks -------------------------------------------------------------
bool checked_build() {
#ifdef SB200_CHECK_BOUNDS
  return true;
#else
  return false;
#endif
}
// One row (site, index, limit) per module with index checks; site 0 = nothing recorded since
// the last call.  Reading clears the records.  Always zeros in the normal build.
Tensor bounds_report() {
  Tensor out = at::zeros({2, 3}, at::TensorOptions().dtype(at::kLong));
  sb200::BoundsRecord rec[2];
  TORCH_CHECK(sb200::read_bounds_norm(&rec[0]) == 0 && sb200::read_bounds_ep(&rec[1]) == 0, "bounds_report: reading the device records failed");
  for (int i = 0; i < 2; ++i) {
    out[i][0] = (int64_t)rec[i].site;
    out[i][1] = (int64_t)rec[i].index;
    out[i][2] = (int64_t)rec[i].limit;
  }
  return out;
}

// ---- expert-parallel token exchange --------------------------------------------------------
// *_ptrs: int64 CPU tensors [world] with the address of one buffer on every rank as mapped here.
sb200::EpPeers ep_peers(const Tensor& ptrs, int64_t world) {
  TORCH_CHECK(ptrs.device().is_cpu() && ptrs.scalar_type() == at::kLong && ptrs.numel() == world && world >= 1 && world <= 16);
  sb200::EpPeers out{};
  for (int q = 0; q < world; ++q) out.ptr[q] = (unsigned long long)ptrs.data_ptr<int64_t>()[q];
  return out;
}
void check_slots(const Tensor& t, int64_t n, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous() && t.numel() == n, name, ": int32 CUDA [", n, "] expected");
}

void ep_push(const Tensor& src, const Tensor& src_row, const Tensor& dst_rank, const Tensor& dst_pos, const c10::optional<Tensor>& scale,
             const Tensor& dst_ptrs, int64_t capacity, Tensor counter, const Tensor& flag_ptrs, int64_t rank, int64_t world,
             int64_t seq) {
  check_rows(src, "src");
  TORCH_CHECK(src.is_contiguous() && src.size(1) % 8 == 0, "src rows must be contiguous with a multiple of 8 columns");
  const int64_t n = src_row.numel();
  check_slots(src_row, n, "src_row");
  check_slots(dst_rank, n, "dst_rank");
  check_slots(dst_pos, n, "dst_pos");
  if (scale.has_value()) TORCH_CHECK(scale->is_cuda() && scale->scalar_type() == at::kFloat && scale->is_contiguous() && scale->numel() == n);
  TORCH_CHECK(counter.is_cuda() && counter.scalar_type() == at::kInt && counter.numel() >= 1);
  c10::cuda::CUDAGuard guard(src.device());
  const sb200::EpPeers dstp = ep_peers(dst_ptrs, world), flg = ep_peers(flag_ptrs, world);
  const int rc = sb200::launch_ep_push((const __nv_bfloat16*)src.data_ptr(), src_row.data_ptr<int>(), dst_rank.data_ptr<int>(),
                                       dst_pos.data_ptr<int>(), scale.has_value() ? scale->data_ptr<float>() : nullptr, (int)n,
                                       (int)src.size(1), (int)src.size(0), (int)capacity, dstp,
                                       reinterpret_cast<unsigned int*>(counter.data_ptr<int>()), flg, (int)rank, (int)world, (uint32_t)seq,
                                       cur_stream());
  TORCH_CHECK(rc == 0, "ep_push launch failed (", rc, ")");
}

void ep_signal(const Tensor& flag_ptrs, int64_t rank, int64_t world, int64_t seq, const Tensor& on_device_of) {
  c10::cuda::CUDAGuard guard(on_device_of.device());
  const int rc = sb200::launch_ep_signal(ep_peers(flag_ptrs, world), (int)rank, (int)world, (uint32_t)seq, cur_stream());
  TORCH_CHECK(rc == 0, "ep_signal launch failed (", rc, ")");
}

void ep_wait(const Tensor& flags_local, int64_t world, int64_t seq, int64_t spin_limit, Tensor status) {
  TORCH_CHECK(flags_local.is_cuda() && flags_local.scalar_type() == at::kInt && flags_local.is_contiguous() && flags_local.numel() >= world);
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  c10::cuda::CUDAGuard guard(flags_local.device());
  const int rc = sb200::launch_ep_wait(reinterpret_cast<const uint32_t*>(flags_local.data_ptr<int>()), (int)world, (uint32_t)seq,
                                       (uint32_t)spin_limit, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "ep_wait launch failed (", rc, ")");
}

void ep_pull(const Tensor& src_ptrs, int64_t capacity, const Tensor& src_rank, const Tensor& src_pos, const c10::optional<Tensor>& weight,
             int64_t world, Tensor out, int64_t k, c10::optional<Tensor> rows_out) {
  check_rows(out, "out");
  TORCH_CHECK(out.is_contiguous() && out.size(1) % 8 == 0);
  const int64_t n = out.size(0) * k;
  check_slots(src_rank, n, "src_rank");
  check_slots(src_pos, n, "src_pos");
  if (weight.has_value()) TORCH_CHECK(weight->is_cuda() && weight->scalar_type() == at::kFloat && weight->is_contiguous() && weight->numel() == n);
  if (rows_out.has_value())
    TORCH_CHECK(rows_out->is_cuda() && rows_out->scalar_type() == at::kBFloat16 && rows_out->is_contiguous() &&
                rows_out->numel() == n * out.size(1), "rows_out: bf16 [T*k, H] expected");
  c10::cuda::CUDAGuard guard(out.device());
  const int rc = sb200::launch_ep_pull(ep_peers(src_ptrs, world), src_rank.data_ptr<int>(), src_pos.data_ptr<int>(),
                                       weight.has_value() ? weight->data_ptr<float>() : nullptr, (int)out.size(0), (int)k, (int)out.size(1),
                                       (int)world, (int)capacity, (__nv_bfloat16*)out.data_ptr(),
                                       rows_out.has_value() ? (__nv_bfloat16*)rows_out->data_ptr() : nullptr, cur_stream());
  TORCH_CHECK(rc == 0, "ep_pull launch failed (", rc, ")");
}

// ---- tcgen05 GEMM ------------------------------------------------------------------------
// out[M,N] = a[M,K] @ b[N,K]^T; epilogue 0 = store, 1 = out += result, 2 = result + residual.
// `status` (int32[1], device) receives a non-zero code if a bounded wait in the kernel ran out.
// variant: 0 = choose, 1 = one CTA per 128x256 tile, 2 = CTA pairs on 256x256 tiles.
void gemm_tn_variant(const Tensor& a, const Tensor& b, Tensor out, const c10::optional<Tensor>& residual, int64_t epilogue, Tensor status,
                     int64_t variant) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda() && status.is_cuda());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1);
  TORCH_CHECK(a.size(1) == b.size(1) && out.size(0) == a.size(0) && out.size(1) == b.size(0), "gemm_tn: shape mismatch");
  TORCH_CHECK(status.scalar_type() == at::kInt && status.numel() >= 1);
  const void* res = nullptr;
  int64_t ldr = 0;
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->dim() == 2 && residual->stride(1) == 1 &&
                residual->size(0) == out.size(0) && residual->size(1) == out.size(1));
    res = residual->data_ptr();
    ldr = residual->stride(0);
  }
  TORCH_CHECK(epilogue != 2 || res != nullptr, "gemm_tn: epilogue 2 needs a residual");
  c10::cuda::CUDAGuard guard(a.device());
  const int rc = sb200::launch_gemm_tn_tcgen05(a.data_ptr(), b.data_ptr(), out.data_ptr(), res, (int)a.size(0), (int)b.size(0),
                                               (int)a.size(1), a.stride(0), b.stride(0), out.stride(0), ldr, (int)epilogue,
                                               status.data_ptr<int>(), (int)variant, cur_stream());
  TORCH_CHECK(rc == 0, "gemm_tn launch failed (", rc, ")");
}

void gemm_tn(const Tensor& a, const Tensor& b, Tensor out, const c10::optional<Tensor>& residual, int64_t epilogue, Tensor status) {
  gemm_tn_variant(a, b, out, residual, epilogue, status, 0);
}

// out[M,N] (=, +=) op(a) @ op(b)^T with either operand stored transposed:
//   a_mn false: a is [M, K];  true: a is [K, M] (the product uses a^T, read in place)
//   b_mn false: b is [N, K];  true: b is [K, N]
// dgrad of a linear layer: gemm(dy[T,out], w[out,in], dx, b_mn = true);
// wgrad: gemm(dy[T,out], x[T,in], dw[out,in], a_mn = b_mn = true, epilogue 1 to accumulate).
void gemm(const Tensor& a, const Tensor& b, Tensor out, int64_t epilogue, bool a_mn, bool b_mn, Tensor status) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda() && status.is_cuda());
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16);
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1);
  TORCH_CHECK(epilogue == 0 || epilogue == 1, "gemm: epilogue 0 (store) or 1 (accumulate)");
  const int64_t M = a_mn ? a.size(1) : a.size(0), K = a_mn ? a.size(0) : a.size(1);
  const int64_t N = b_mn ? b.size(1) : b.size(0), Kb = b_mn ? b.size(0) : b.size(1);
  TORCH_CHECK(K == Kb && out.size(0) == M && out.size(1) == N, "gemm: shape mismatch");
  TORCH_CHECK(status.scalar_type() == at::kInt && status.numel() >= 1);
  c10::cuda::CUDAGuard guard(a.device());
  const int rc = sb200::launch_gemm_tcgen05(a.data_ptr(), b.data_ptr(), out.data_ptr(), nullptr, (int)M, (int)N, (int)K, a.stride(0),
                                            b.stride(0), out.stride(0), 0, (int)epilogue, a_mn ? 1 : 0, b_mn ? 1 : 0,
                                            status.data_ptr<int>(), 0, cur_stream());
  TORCH_CHECK(rc == 0, "gemm launch failed (", rc, ")");
}

// ---- masked attention ------------------------------------------------------------------
void check_heads(const Tensor& t, const char* name, int64_t hd) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 3, name, ": bf16 CUDA [T, heads, hd] expected");
  TORCH_CHECK(t.size(2) == hd && t.stride(2) == 1 && t.stride(1) == hd, name, ": heads must be contiguous");
  TORCH_CHECK(t.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name, ": rows must be 16-byte aligned");
}

sb200::AttnParams make_params(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& lo, const Tensor& hi,
                              const c10::optional<Tensor>& ke, const c10::optional<Tensor>& ve,
                              const c10::optional<Tensor>& ext_idx, double scale) {
  const int64_t hd = q.size(2);
  check_heads(q, "q", hd);
  check_heads(k, "k", hd);
  check_heads(v, "v", hd);
  TORCH_CHECK(hd == 64 || hd == 128 || hd == 256, "attention: head_dim must be 64, 128 or 256");
  TORCH_CHECK(k.size(0) == v.size(0) && k.size(1) == v.size(1) && q.size(1) % k.size(1) == 0);
  TORCH_CHECK(lo.scalar_type() == at::kInt && hi.scalar_type() == at::kInt && lo.is_contiguous() && hi.is_contiguous() &&
              lo.numel() == q.size(0) && hi.numel() == q.size(0), "lo/hi must be int32[Tq]");
  sb200::AttnParams p{};
  p.q = (const __nv_bfloat16*)q.data_ptr();
  p.k = (const __nv_bfloat16*)k.data_ptr();
  p.v = (const __nv_bfloat16*)v.data_ptr();
  p.lo = lo.data_ptr<int>();
  p.hi = hi.data_ptr<int>();
  p.Tq = (int)q.size(0);
  p.Tc = (int)k.size(0);
  p.nh = (int)q.size(1);
  p.nkv = (int)k.size(1);
  p.q_rs = q.stride(0);
  p.k_rs = k.stride(0);
  p.v_rs = v.stride(0);
  p.scale = (float)scale;
  if (ext_idx.has_value() && ext_idx->numel() > 0) {
    TORCH_CHECK(ke.has_value() && ve.has_value(), "extra keys need k_ext and v_ext");
    check_heads(*ke, "k_ext", hd);
    check_heads(*ve, "v_ext", hd);
    TORCH_CHECK(ke->size(0) == ve->size(0) && ke->size(1) == p.nkv && ve->size(1) == p.nkv);
    TORCH_CHECK(ext_idx->scalar_type() == at::kInt && ext_idx->is_contiguous() && ext_idx->dim() == 2 && ext_idx->size(0) == p.Tq);
    p.ke = (const __nv_bfloat16*)ke->data_ptr();
    p.ve = (const __nv_bfloat16*)ve->data_ptr();
    p.ext_idx = ext_idx->data_ptr<int>();
    p.Te = (int)ke->size(0);
    p.E = (int)ext_idx->size(1);
    p.ke_rs = ke->stride(0);
    p.ve_rs = ve->stride(0);
  }
  return p;
}

// Block-structured extras (tcgen05 kernels): the extra keys of row r are the rows of its block of `block` rows in
// k_ext / v_ext (only up to r with `causal`); the per-row index list is then not used.
void use_block_extras(sb200::AttnParams& p, const Tensor& q, int64_t block, bool causal) {
  if (block <= 0) return;
  TORCH_CHECK(p.ke != nullptr && p.ve != nullptr, "block-structured extras need k_ext and v_ext");
  TORCH_CHECK(128 % block == 0, "block-structured extras: the block size must divide 128");
  TORCH_CHECK(p.Te >= p.Tq, "block-structured extras: k_ext / v_ext hold one row per query row");
  p.E = 0;
  p.ext_idx = nullptr;
  p.ext_block = (int)block;
  p.ext_causal = causal ? 1 : 0;
  (void)q;
}

std::tuple<Tensor, Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& lo, const Tensor& hi,
                                    const c10::optional<Tensor>& ke, const c10::optional<Tensor>& ve,
                                    const c10::optional<Tensor>& ext_idx, double scale) {
  sb200::AttnParams p = make_params(q, k, v, lo, hi, ke, ve, ext_idx, scale);
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = at::empty({q.size(0), q.size(1), q.size(2)}, q.options());
  Tensor lse2 = at::empty({q.size(1), q.size(0)}, q.options().dtype(at::kFloat));
  p.out = (__nv_bfloat16*)out.data_ptr();
  p.o_rs = out.stride(0);
  p.lse2 = lse2.data_ptr<float>();
  const int rc = sb200::launch_attn_fwd(p, (int)q.size(2), cur_stream());
  TORCH_CHECK(rc == 0, "attn_fwd launch failed (", rc, ")");
  return {out, lse2};
}

// Forward on the tcgen05 tensor cores (head_dim 128).  `status` (int32[1], device) receives a
// non-zero code if a bounded wait in the kernel ran out.
std::tuple<Tensor, Tensor> attn_fwd_tc(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& lo, const Tensor& hi,
                                       const c10::optional<Tensor>& ke, const c10::optional<Tensor>& ve,
                                       const c10::optional<Tensor>& ext_idx, double scale, Tensor status, int64_t ext_block,
                                       bool ext_causal) {
  sb200::AttnParams p = make_params(q, k, v, lo, hi, ke, ve, ext_idx, scale);
  use_block_extras(p, q, ext_block, ext_causal);
  TORCH_CHECK(q.size(2) == 128, "attn_fwd_tc: head_dim must be 128");
  TORCH_CHECK(status.is_cuda() && status.scalar_type() == at::kInt && status.numel() >= 1);
  c10::cuda::CUDAGuard guard(q.device());
  Tensor out = at::empty({q.size(0), q.size(1), q.size(2)}, q.options());
  Tensor lse2 = at::empty({q.size(1), q.size(0)}, q.options().dtype(at::kFloat));
  p.out = (__nv_bfloat16*)out.data_ptr();
  p.o_rs = out.stride(0);
  p.lse2 = lse2.data_ptr<float>();
  const int rc = sb200::launch_attn_fwd_tc(p, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "attn_fwd_tc launch failed (", rc, ")");
  return {out, lse2};
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> attn_bwd(
    const Tensor& dout, const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& lse2,
    const Tensor& lo, const Tensor& hi, const c10::optional<Tensor>& ke, const c10::optional<Tensor>& ve,
    const c10::optional<Tensor>& ext_idx, double scale, int64_t impl, const c10::optional<Tensor>& status, int64_t ext_block,
    bool ext_causal) {
  // impl 0: mma.sync kernels; 1: tcgen05 kernels (head_dim 128; `status` receives a code if a bounded wait ran out)
  sb200::AttnParams p = make_params(q, k, v, lo, hi, ke, ve, ext_idx, scale);
  TORCH_CHECK(ext_block <= 0 || impl == 1, "block-structured extras run on the tcgen05 kernels only");
  use_block_extras(p, q, ext_block, ext_causal);
  const int64_t hd = q.size(2);
  if (impl == 1) {
    TORCH_CHECK(hd == 128, "attn_bwd: the tcgen05 kernels need head_dim 128");
    TORCH_CHECK(status.has_value() && status->is_cuda() && status->scalar_type() == at::kInt && status->numel() >= 1);
  }
  check_heads(dout, "dout", hd);
  check_heads(out, "out", hd);
  TORCH_CHECK(dout.size(0) == q.size(0) && dout.size(1) == q.size(1) && out.sizes() == dout.sizes());
  TORCH_CHECK(lse2.scalar_type() == at::kFloat && lse2.is_contiguous() && lse2.numel() == q.size(0) * q.size(1));
  c10::cuda::CUDAGuard guard(q.device());
  Tensor dq = at::empty({q.size(0), q.size(1), hd}, q.options());
  Tensor dk = at::empty({k.size(0), k.size(1), hd}, q.options());
  Tensor dv = at::empty({k.size(0), k.size(1), hd}, q.options());
  Tensor delta = at::empty({q.size(1), q.size(0)}, lse2.options());
  Tensor dke, dve;
  if (p.E > 0 || p.ext_block > 0) {
    dke = at::zeros({p.Te, p.nkv, hd}, lse2.options());
    dve = at::zeros({p.Te, p.nkv, hd}, lse2.options());
    p.dke = dke.data_ptr<float>();
    p.dve = dve.data_ptr<float>();
  } else {
    dke = at::empty({0}, lse2.options());
    dve = at::empty({0}, lse2.options());
  }
  Tensor dkv_part;
  if (p.nh > p.nkv) {  // grouped queries: per-head fp32 partials, summed in head order afterwards
    dkv_part = at::empty({p.nh / p.nkv, 2, k.size(0), k.size(1), hd}, lse2.options());
    p.dkv_part = dkv_part.data_ptr<float>();
  }
  const int n_tiles = (p.Tc + sb200::kAttnKeyTile - 1) / sb200::kAttnKeyTile;
  Tensor qmin = at::empty({n_tiles}, lo.options());
  Tensor qmax = at::empty({n_tiles}, lo.options());
  p.out = (__nv_bfloat16*)out.data_ptr();
  p.o_rs = out.stride(0);
  p.lse2 = lse2.data_ptr<float>();
  p.dout = (const __nv_bfloat16*)dout.data_ptr();
  p.do_rs = dout.stride(0);
  p.delta = delta.data_ptr<float>();
  p.dq = (__nv_bfloat16*)dq.data_ptr();
  p.dq_rs = dq.stride(0);
  p.dk = (__nv_bfloat16*)dk.data_ptr();
  p.dv = (__nv_bfloat16*)dv.data_ptr();
  p.tile_qmin = qmin.data_ptr<int>();
  p.tile_qmax = qmax.data_ptr<int>();
  const int rc = impl == 1 ? sb200::launch_attn_bwd_tc(p, qmin.data_ptr<int>(), qmax.data_ptr<int>(), status->data_ptr<int>(), cur_stream())
                           : sb200::launch_attn_bwd(p, (int)hd, qmin.data_ptr<int>(), qmax.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "attn_bwd launch failed (", rc, ")");
  return {dq, dk, dv, dke, dve};
}

}  // namespace

TORCH_LIBRARY(sb200, m) {
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("rope_", &rope_);
  m.def("loss_fwd", &loss_fwd);
  m.def("loss_bwd", &loss_bwd);
  m.def("ce_label_fwd", &ce_label_fwd);
  m.def("sumsq", &sumsq);
  m.def("adamw", &adamw);
  m.def("muon_momentum", &muon_momentum);
  m.def("muon_apply", &muon_apply);
  m.def("sumsq_num_partials", &sumsq_num_partials_binding);
  m.def("set_hyper", &set_hyper);
  m.def("launch_count", &launch_count);
  m.def("peer_alloc", &peer_alloc);
  m.def("peer_release", &peer_release);
  m.def("peer_handle", &peer_handle);
  m.def("peer_open", &peer_open);
  m.def("peer_close", &peer_close);
  m.def("peer_tensor", &peer_tensor);
  m.def("fused_optim_ctl_words", &fused_optim_ctl_words);
  m.def("fused_sharded_adamw", &fused_sharded_adamw);
  m.def("gemm_swiglu", &gemm_swiglu);
  m.def("gemm_scatter", &gemm_scatter);
  m.def("tp_allreduce_ctl_words", &tp_allreduce_ctl_words);
  m.def("tp_reduce_broadcast", &tp_reduce_broadcast);
  m.def("step_tail", &step_tail);
  m.def("checked_build", &checked_build);
  m.def("bounds_report", &bounds_report);
  m.def("ep_push", &ep_push);
  m.def("ep_signal", &ep_signal);
  m.def("ep_wait", &ep_wait);
  m.def("ep_pull", &ep_pull);
  m.def("hs_ring_ctl_words", &hs_ring_ctl_words);
  m.def("hs_push", &hs_push);
  m.def("hs_pop", &hs_pop);
  m.def("gemm_tn", &gemm_tn);
  m.def("gemm", &gemm);
  m.def("lmhead_loss_fwd", &lmhead_loss_fwd);
  m.def("moe_group_plan", &moe_group_plan);
  m.def("gemm_grouped_rows", &gemm_grouped_rows);
  m.def("gemm_grouped_wgrad", &gemm_grouped_wgrad);
  m.def("gemm_tn_variant", &gemm_tn_variant);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_fwd_tc", &attn_fwd_tc);
  m.def("attn_bwd", &attn_bwd);
}
