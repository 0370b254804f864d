"""Hot operators of the framework.

Every function here has two implementations behind one signature:

* CUDA tensors run the hand-written sm_100a kernels of ``csrc/`` through
  ``torch.ops.sb200`` (bf16 storage, fp32 math).  There is no fallback on a GPU:
  a missing extension is a hard error.
* CPU tensors (any float dtype) run a plain PyTorch formulation.  That path is the
  numerical oracle the kernel tests compare against, and it is what the gloo /
  world_size > 1 plumbing tests execute.

All functions are differentiable; the CUDA paths carry their own backward
kernels via ``torch.autograd.Function``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from speculators_b200.ops import _ext
from speculators_b200.ops.attention import AttnSpec, masked_attention, masked_attention_reference

__all__ = [
    "AttnSpec",
    "LOSS_OPS",
    "adamw_step_",
    "eagle3_input_concat",
    "fused_row_loss",
    "check_gemm_status",
    "gemm_status",
    "GroupPlan",
    "grouped_linear",
    "grouped_linear_ok",
    "linear",
    "linear_swiglu",
    "lm_head_loss_raw",
    "masked_attention",
    "matmul_nn",
    "matmul_nt",
    "matmul_tn",
    "masked_attention_reference",
    "native",
    "rms_norm",
    "rope_",
    "rope_split",
    "sum_of_squares",
    "swiglu",
    "token_cross_entropy",
    "ttt_step_tail",
]

LOSS_OPS = {"kl_div": 0, "rkl": 1, "jsd": 2, "ce": 3, "tv": 4}


def native():
    """``torch.ops.sb200`` (builds / loads the extension on first use)."""
    return _ext.lib()


def _use_native(t: torch.Tensor) -> bool:
    return t.is_cuda


# --------------------------------------------------------------------------- linear
_GEMM_STATUS: dict[int, torch.Tensor] = {}


def _own_gemm_enabled() -> bool:
    import os

    return os.environ.get("SB200_LINEAR_GEMM", "tcgen05") != "cublas"


def _gemm_operand_ok(t: torch.Tensor) -> bool:
    return (t.is_cuda and t.dtype == torch.bfloat16 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0
            and t.data_ptr() % 16 == 0)


def gemm_status(device: torch.device) -> torch.Tensor:
    """The device word the tcgen05 GEMM writes a non-zero code to if one of its bounded
    waits ever runs out (it should stay 0; read it where a host sync is acceptable)."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _GEMM_STATUS:
        _GEMM_STATUS[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _GEMM_STATUS[idx]


_WAIT_CODES = {
    1: "GEMM producer", 2: "GEMM MMA issuer", 3: "GEMM epilogue",
    31: "attention forward producer", 32: "attention forward MMA issuer", 33: "attention forward softmax",
    41: "attention dQ producer", 42: "attention dQ MMA issuer", 43: "attention dQ element-wise warps",
    44: "attention dK/dV producer", 45: "attention dK/dV MMA issuer", 46: "attention dK/dV element-wise warps",
}


def check_gemm_status() -> None:
    """Raise if a tcgen05 kernel (GEMM or attention) launched by this process reported a wait
    that ran out; the kernels share one status word per device."""
    for idx, word in _GEMM_STATUS.items():
        code = int(word.item())
        if code:
            word.zero_()
            raise RuntimeError(f"a tcgen05 kernel on cuda:{idx} gave up waiting (code {code}: {_WAIT_CODES.get(code, 'unknown wait')})")


def _forward_gemm(x2: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None) -> torch.Tensor:
    """``x2 @ w.T (+ residual)`` for 2-D operands.  bf16 CUDA operands with 16-byte aligned
    rows run on the package's tcgen05 kernel (the residual is read in its epilogue, no
    copy of it is made); everything else goes to the library."""
    if _gemm_operand_ok(x2) and _gemm_operand_ok(w) and _own_gemm_enabled() and (
        residual is None or (_gemm_operand_ok(residual) and residual.shape == (x2.shape[0], w.shape[0]))
    ):
        out = torch.empty((x2.shape[0], w.shape[0]), dtype=x2.dtype, device=x2.device)
        native().gemm_tn(x2, w, out, residual, 2 if residual is not None else 0, gemm_status(x2.device))
        return out
    if residual is not None:
        return torch.addmm(residual, x2, w.t())
    return x2 @ w.t()


def _dgrad_gemm(dy2: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """``dy2 @ w`` (input gradient of a linear layer) on the tcgen05 kernel: the weight is read
    as stored, ``[out, in]`` with ``in`` contiguous, as an MN-major B operand."""
    dx = out if out is not None else torch.empty((dy2.shape[0], w.shape[1]), dtype=dy2.dtype, device=dy2.device)
    native().gemm(dy2, w, dx, 1 if accumulate else 0, False, True, gemm_status(dy2.device))
    return dx


def _wgrad_gemm(dy2: torch.Tensor, x2: torch.Tensor, out: torch.Tensor | None, accumulate: bool) -> torch.Tensor:
    """``dy2.T @ x2`` (weight gradient) on the tcgen05 kernel, both operands read in place as
    MN-major tiles, stored into or added to ``out`` in the epilogue."""
    if out is None:
        out = torch.empty((dy2.shape[1], x2.shape[1]), dtype=dy2.dtype, device=dy2.device)
    native().gemm(dy2, x2, out, 1 if accumulate else 0, True, True, gemm_status(dy2.device))
    return out


def matmul_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b.T`` for 2-D tensors; bf16 CUDA operands with aligned rows use the tcgen05 kernel."""
    if _gemm_operand_ok(a) and _gemm_operand_ok(b) and _own_gemm_enabled():
        return _forward_gemm(a, b, None)
    return a @ b.t()


def matmul_nn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """``a @ b`` for 2-D tensors (``b`` read as stored, no transpose copy), optionally stored
    into / added to ``out``."""
    if _gemm_operand_ok(a) and _gemm_operand_ok(b) and _own_gemm_enabled() and (out is None or _gemm_operand_ok(out)):
        return _dgrad_gemm(a, b, out, accumulate)
    if out is None:
        return a @ b
    return out.addmm_(a, b) if accumulate else torch.mm(a, b, out=out)


def matmul_tn(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None, accumulate: bool = False) -> torch.Tensor:
    """``a.T @ b`` for 2-D tensors, optionally stored into / added to ``out``."""
    if _gemm_operand_ok(a) and _gemm_operand_ok(b) and _own_gemm_enabled() and (out is None or _gemm_operand_ok(out)):
        return _wgrad_gemm(a, b, out, accumulate)
    if out is None:
        return a.t() @ b
    return out.addmm_(a.t(), b) if accumulate else torch.mm(a.t(), b, out=out)


# --------------------------------------------------------------------------- grouped (expert) linears
class GroupPlan:
    """Padded row order of a grouped product, all on the device: expert ``e`` owns the rows
    ``seg[e] .. seg[e] + counts[e]`` of a ``[capacity, .]`` buffer, ``seg[e]`` a multiple of 128,
    the rows up to ``seg[e + 1]`` are zero.  ``dest[i]`` is the padded row of the ``i``-th row of
    the expert-sorted order.  Built without reading anything back to the host."""

    def __init__(self, counts: torch.Tensor, num_rows: int):
        counts32 = counts.to(torch.int32).contiguous()
        E = counts32.numel()
        self.seg, self.mtile_start = native().moe_group_plan(counts32)
        self.capacity = (num_rows + 127 * E + 127) // 128 * 128  # worst case: every expert's tail padded by 127 rows
        start = torch.cumsum(counts32, 0) - counts32  # unpadded offsets
        expert_of = torch.repeat_interleave(torch.arange(E, device=counts.device), counts32.long(), output_size=num_rows)
        self.dest = (torch.arange(num_rows, device=counts.device) - start[expert_of] + self.seg[expert_of]).long()

    def pad(self, x_sorted: torch.Tensor) -> torch.Tensor:
        out = x_sorted.new_zeros((self.capacity, x_sorted.shape[1]))
        return out.index_copy(0, self.dest, x_sorted)

    def unpad(self, y_padded: torch.Tensor) -> torch.Tensor:
        return _UnpadRowsFn.apply(y_padded, self.dest)


class _UnpadRowsFn(torch.autograd.Function):
    """``y_padded[dest]`` for distinct ``dest``: the gradient is a row copy into zeros, where autograd's
    ``index_select`` backward would add with atomics (0.67 ms against 0.23 ms for 40960 x 2048 rows)."""

    @staticmethod
    def forward(ctx, y_padded, dest):
        ctx.save_for_backward(dest)
        ctx.rows = y_padded.shape[0]
        return y_padded.index_select(0, dest)

    @staticmethod
    def backward(ctx, dy):
        (dest,) = ctx.saved_tensors
        return dy.new_zeros((ctx.rows, dy.shape[1])).index_copy_(0, dest, dy), None


class _GroupedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_pad, weight, seg, mts):
        out = torch.empty((x_pad.shape[0], weight.shape[1]), dtype=x_pad.dtype, device=x_pad.device)
        native().gemm_grouped_rows(x_pad, weight, out, False, seg, mts, gemm_status(x_pad.device))
        ctx.save_for_backward(x_pad, weight, seg, mts)
        return out

    @staticmethod
    def backward(ctx, dy):
        x_pad, weight, seg, mts = ctx.saved_tensors
        dy = dy if (dy.stride(-1) == 1 and dy.stride(0) % 8 == 0 and dy.data_ptr() % 16 == 0) else dy.contiguous()
        status = gemm_status(dy.device)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = torch.empty_like(x_pad)
            native().gemm_grouped_rows(dy, weight, dx, True, seg, mts, status)
        if ctx.needs_input_grad[1]:
            dw = torch.empty_like(weight)
            native().gemm_grouped_wgrad(dy, x_pad, dw, False, seg, mts, status)
        return dx, dw, None, None


def grouped_linear_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    """Whether ``grouped_linear`` can run on the tcgen05 kernel for these operands."""
    return (_own_gemm_enabled() and _gemm_operand_ok(x) and weight.is_cuda and weight.dtype == torch.bfloat16 and weight.dim() == 3
            and weight.is_contiguous() and weight.shape[1] % 256 == 0 and weight.shape[2] % 256 == 0 and x.shape[0] % 128 == 0)


def grouped_linear(x_pad: torch.Tensor, weight: torch.Tensor, plan: GroupPlan) -> torch.Tensor:
    """``y[r] = weight[e(r)] @ x_pad[r]`` for rows in the padded expert order of ``plan``
    (``weight``: ``[E, out, in]``).  Forward, input gradient and per-expert weight gradient are
    grouped launches of the tcgen05 GEMM whose tile schedule reads the experts' row counts from
    device memory, so the call has fixed shapes and no host synchronisation."""
    return _GroupedLinearFn.apply(x_pad, weight, plan.seg, plan.mtile_start)


class _LinearFn(torch.autograd.Function):
    """``y = x @ W[rows].T (+ residual)`` with the weight gradient accumulated in place.

    When the training engine has attached a flat gradient view to the weight
    (``weight._flat_grad``), backward runs ``grad[rows].addmm_(dy.T, x)``: one GEMM
    whose epilogue adds into the gradient buffer, instead of a GEMM into a temporary
    followed by autograd's separate accumulation pass over the whole weight.  The
    residual, when given, rides in the forward GEMM's epilogue (``beta = 1``).
    """

    @staticmethod
    def forward(ctx, x, weight, residual, r0, r1):
        # x is [rows, in]; the result is a fresh tensor (never a view), so callers may
        # rotate / normalise it in place
        w = weight if r0 is None else weight[r0:r1]
        y = _forward_gemm(x, w, residual)
        ctx.save_for_backward(x, weight)
        ctx.rows = (r0, r1)
        ctx.has_residual = residual is not None
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, weight = ctx.saved_tensors
        dx, dw = _linear_backward(x2, weight, ctx.rows, dy, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        dres = dy if ctx.has_residual and ctx.needs_input_grad[2] else None
        return dx, dw, dres, None, None


def _linear_backward(x2, weight, rows, dy, need_dx: bool, need_dw: bool):
    """``(dx, dw)`` of ``y = x2 @ weight[rows].T``; ``dw`` is ``None`` when the gradient went
    straight into the flat buffer the training engine attached to the weight."""
    r0, r1 = rows
    w = weight if r0 is None else weight[r0:r1]
    dy2 = dy if (dy.stride(-1) == 1 and dy.stride(0) % 8 == 0 and dy.data_ptr() % 16 == 0) else dy.contiguous()
    dx = dw = None
    own = _own_gemm_enabled() and _gemm_operand_ok(dy2) and _gemm_operand_ok(w) and _gemm_operand_ok(x2)
    if need_dx:
        dx = _dgrad_gemm(dy2, w) if own else dy2 @ w
    if need_dw:
        flat = getattr(weight, "_flat_grad", None)
        if flat is not None:
            target = flat if r0 is None else flat[r0:r1]
            fresh = getattr(weight, "_grad_fresh", False)
            if fresh:
                # first gradient of this weight since the engine's zero_grad, which left
                # the buffer uncleared: store instead of accumulate
                weight._grad_fresh = False
                if r0 is not None:
                    flat.zero_()
            if own and _gemm_operand_ok(target):
                _wgrad_gemm(dy2, x2, target, accumulate=not fresh or r0 is not None)
            elif fresh and r0 is None:
                torch.mm(dy2.t(), x2, out=flat)
            else:
                target.addmm_(dy2.t(), x2)
        elif r0 is None:
            dw = _wgrad_gemm(dy2, x2, None, accumulate=False) if own else dy2.t() @ x2
        else:
            dw = torch.zeros_like(weight)
            if own and _gemm_operand_ok(dw[r0:r1]):
                _wgrad_gemm(dy2, x2, dw[r0:r1], accumulate=False)
            else:
                dw[r0:r1] = dy2.t() @ x2
    return dx, dw


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, residual: torch.Tensor | None = None,
           rows: tuple[int, int] | None = None) -> torch.Tensor:
    """``x @ weight[rows].T (+ bias) (+ residual)``.  On CUDA in bf16 the forward product
    runs on the package's tcgen05 GEMM with the residual read in its epilogue
    (``SB200_LINEAR_GEMM=cublas`` sends it to the library instead); the two backward
    products run on the same kernel with the transposed operands read in place (MN-major
    tiles), the weight gradient accumulating in the epilogue into the engine's flat
    gradient buffer."""
    if x.is_cuda and (weight.requires_grad or x.requires_grad) and torch.is_grad_enabled():
        r0, r1 = rows if rows is not None else (None, None)
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        res2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
        y = _LinearFn.apply(x2, weight, res2, r0, r1)
        if len(lead) != 1:
            y = y.view(*lead, y.shape[-1])
        if bias is not None:
            y = y + (bias if rows is None else bias[rows[0] : rows[1]])
        return y
    w = weight if rows is None else weight[rows[0] : rows[1]]
    b = bias if (bias is None or rows is None) else bias[rows[0] : rows[1]]
    if x.is_cuda and x.dtype == torch.bfloat16 and b is None and not torch.is_grad_enabled() and _own_gemm_enabled():
        x2 = x.reshape(-1, x.shape[-1])
        res2 = residual.reshape(-1, residual.shape[-1]) if residual is not None else None
        return _forward_gemm(x2, w, res2).view(*x.shape[:-1], w.shape[0])
    y = F.linear(x, w, b)
    return y if residual is None else y + residual


# --------------------------------------------------------------------------- rmsnorm
_RMSNORM_MAX_WIDTH = 16384


def _rms_norm_ref(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    dt = x.dtype
    xf = x.float()
    xf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    return weight * xf.to(dt)


class _RMSNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        # allocated in the caller's shape and returned as it is: a view made in here could not be
        # modified in place afterwards (the rotary kernel does that to normalised q / k heads)
        y = torch.empty(x.shape, dtype=x.dtype, device=x.device)
        rstd = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
        native().rmsnorm_fwd(x2, weight, None, y.view(-1, H), rstd, eps)
        ctx.save_for_backward(x2, weight, rstd)
        ctx.shape = x.shape
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, weight, rstd = ctx.saved_tensors
        H = x2.shape[-1]
        dy2 = dy.reshape(-1, H)
        if dy2.stride(-1) != 1 or dy2.stride(0) % 8:
            dy2 = dy2.contiguous()
        dx = torch.empty_like(x2)
        dw = None
        if ctx.needs_input_grad[1]:
            dw = torch.empty(H, dtype=torch.float32, device=x2.device)
        native().rmsnorm_bwd(dy2, x2, weight, rstd, dx, dw, False, False)
        return dx.view(ctx.shape), (dw.to(weight.dtype) if dw is not None else None), None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm over the last dim: ``weight * (x / rms(x))`` with fp32 statistics.  Rows of up to
    16384 elements run on the package's kernels (one row per CTA with the row in registers; one row
    per warp for rows of up to 256); wider rows (the concatenated auxiliary states of a 70B-class
    verifier: 3 x 8192) use the element-wise formulation."""
    if _use_native(x) and x.shape[-1] <= _RMSNORM_MAX_WIDTH and x.shape[-1] % 8 == 0:
        return _RMSNormFn.apply(x, weight, eps)
    return _rms_norm_ref(x, weight, eps)


class _Eagle3InputFn(torch.autograd.Function):
    """``cat([rmsnorm(embeds; w_e), rmsnorm(hidden; w_h)], -1)`` written by two
    strided launches into one [T, 2H] buffer (no separate concat copy)."""

    @staticmethod
    def forward(ctx, embeds, hidden, w_e, w_h, eps):
        T, H = hidden.shape
        out = torch.empty((T, 2 * H), dtype=hidden.dtype, device=hidden.device)
        rs_e = torch.empty(T, dtype=torch.float32, device=hidden.device)
        rs_h = torch.empty(T, dtype=torch.float32, device=hidden.device)
        nat = native()
        nat.rmsnorm_fwd(embeds, w_e, None, out[:, :H], rs_e, eps)
        nat.rmsnorm_fwd(hidden, w_h, None, out[:, H:], rs_h, eps)
        ctx.save_for_backward(embeds, hidden, w_e, w_h, rs_e, rs_h)
        ctx.set_materialize_grads(False)
        # second result: the normalised-hidden half on its own, so that a consumer of just
        # that half (the residual branch) hands its gradient back as [T, H] instead of
        # autograd padding it to [T, 2H] (zero fill + copy + add)
        return out, out[:, H:]

    @staticmethod
    def backward(ctx, dout, dhalf):
        embeds, hidden, w_e, w_h, rs_e, rs_h = ctx.saved_tensors
        T, H = hidden.shape
        if dout is None:
            dout = torch.zeros((T, 2 * H), dtype=hidden.dtype, device=hidden.device)
        if dout.stride(1) != 1 or dout.stride(0) % 8:
            dout = dout.contiguous()
        nat = native()
        need_e, need_h, need_we, need_wh = ctx.needs_input_grad[:4]
        d_e = d_h = dw_e = dw_h = None
        if need_e or need_we:
            d_e = torch.empty_like(embeds)
            dw_e = torch.empty(H, dtype=torch.float32, device=hidden.device) if need_we else None
            nat.rmsnorm_bwd(dout[:, :H], embeds, w_e, rs_e, d_e, dw_e, False, False)
        if need_h or need_wh:
            d_h = torch.empty_like(hidden)
            dw_h = torch.empty(H, dtype=torch.float32, device=hidden.device) if need_wh else None
            dy_h = dout[:, H:] if dhalf is None else dout[:, H:] + dhalf
            nat.rmsnorm_bwd(dy_h, hidden, w_h, rs_h, d_h, dw_h, False, False)
        return (
            d_e if need_e else None,
            d_h if need_h else None,
            dw_e.to(w_e.dtype) if dw_e is not None else None,
            dw_h.to(w_h.dtype) if dw_h is not None else None,
            None,
        )


def eagle3_input_concat(embeds, hidden, w_embed_norm, w_hidden_norm, eps, return_hidden_half: bool = False):
    """First-layer input of an EAGLE-3 draft: both halves normalised, concatenated
    (``[T, 2H]``).  With ``return_hidden_half`` also returns the normalised-hidden half
    ``[T, H]`` as a result of its own (a view of the first on CUDA)."""
    if _use_native(hidden):
        out, half = _Eagle3InputFn.apply(embeds.contiguous(), hidden.contiguous(), w_embed_norm, w_hidden_norm, eps)
    else:
        out = torch.cat([_rms_norm_ref(embeds, w_embed_norm, eps), _rms_norm_ref(hidden, w_hidden_norm, eps)], dim=-1)
        half = out[:, hidden.shape[-1]:]
    return (out, half) if return_hidden_half else out


# --------------------------------------------------------------------------- swiglu
class _SwiGLUFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        ctx.save_for_backward(gate_up)
        return native().swiglu_fwd(gate_up)

    @staticmethod
    def backward(ctx, dh):
        (gate_up,) = ctx.saved_tensors
        return native().swiglu_bwd(dh.contiguous(), gate_up)


class _GateUpSwiGLUFn(torch.autograd.Function):
    """``h = silu(x @ Wg.T) * (x @ Wu.T)`` with ``W = [Wg; Wu]``: one GEMM whose epilogue stores the
    gate | up product (saved for the backward pass) and the activated product."""

    @staticmethod
    def forward(ctx, x2, weight):
        gate_up, h = native().gemm_swiglu(x2, weight, gemm_status(x2.device))
        ctx.save_for_backward(x2, weight, gate_up)
        return h

    @staticmethod
    def backward(ctx, dh):
        x2, weight, gate_up = ctx.saved_tensors
        dgu = native().swiglu_bwd(dh.contiguous(), gate_up)
        dx, dw = _linear_backward(x2, weight, (None, None), dgu, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return dx, dw


def linear_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor | None:
    """``swiglu(linear(x, weight))`` for a stacked ``[gate; up]`` weight in one launch: the
    activation is formed in the GEMM's epilogue from the accumulator (``SB200_FUSED_SWIGLU=0``
    switches it off).  ``None`` when the operands do not suit the kernel (other dtype or device,
    intermediate size not a multiple of 128) and the caller should run the two steps."""
    import os

    x2 = x.reshape(-1, x.shape[-1])
    if (not _own_gemm_enabled() or os.environ.get("SB200_FUSED_SWIGLU", "1") == "0" or not _gemm_operand_ok(x2) or not _gemm_operand_ok(weight)
            or weight.shape[0] % 256 or weight.shape[1] != x2.shape[1]):
        return None
    h = _GateUpSwiGLUFn.apply(x2, weight)
    return h.view(*x.shape[:-1], h.shape[-1])


def swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` where ``gate_up = [gate | up]`` along the last dim."""
    if _use_native(gate_up):
        shape = gate_up.shape
        out = _SwiGLUFn.apply(gate_up.reshape(-1, shape[-1]).contiguous())
        return out.view(*shape[:-1], shape[-1] // 2)
    gate, up = gate_up.chunk(2, dim=-1)
    return F.silu(gate) * up


# --------------------------------------------------------------------------- rope
def _rope_ref(x, positions, cos_t, sin_t, heads, hd, rot, sign):
    T = x.shape[0]
    xv = x[:, : heads * hd].reshape(T, heads, hd)
    pos = positions.clamp(0, cos_t.shape[0] - 1)
    c = cos_t[pos].unsqueeze(1).to(torch.float32)
    s = (sin_t[pos] * sign).unsqueeze(1).to(torch.float32)
    half = rot // 2
    x1 = xv[..., :half].float()
    x2 = xv[..., half:rot].float()
    y = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, xv[..., rot:].float()], dim=-1).to(x.dtype)
    return torch.cat([y.reshape(T, heads * hd), x[:, heads * hd :]], dim=-1)


class _RopeFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, positions, cos_t, sin_t, heads, hd, rot):
        ctx.save_for_backward(positions, cos_t, sin_t)
        ctx.cfg = (heads, hd, rot)
        native().rope_(x, positions, cos_t, sin_t, heads, hd, rot, 1.0)
        ctx.mark_dirty(x)
        return x

    @staticmethod
    def backward(ctx, dx):
        positions, cos_t, sin_t = ctx.saved_tensors
        heads, hd, rot = ctx.cfg
        dx = dx.clone()  # the incoming gradient may be shared with other consumers
        native().rope_(dx, positions, cos_t, sin_t, heads, hd, rot, -1.0)
        return dx, None, None, None, None, None, None


def rope_(x, positions, cos_t, sin_t, heads: int, hd: int, rot: int):
    """Neox rotary embedding of the first ``heads`` heads of every row of ``x``
    (``[T, >= heads*hd]``), rotating the first ``rot`` channels of each head.
    In place on CUDA; returns the rotated tensor."""
    if _use_native(x):
        if x._is_view() or x.stride(-1) != 1:  # noqa: SLF001
            # rotating a view in place would rewrite its base's history (and is refused outright for
            # views that custom functions hand out): work on a private copy instead
            x = x.clone(memory_format=torch.contiguous_format)
        return _RopeFn.apply(x, positions, cos_t, sin_t, heads, hd, rot)
    return _rope_ref(x, positions, cos_t, sin_t, heads, hd, rot, 1.0)


class _RopeSplitFn(torch.autograd.Function):
    """Rotate the q|k heads of a fused projection buffer in place and hand out the
    q / k / v column blocks as views.  Backward gathers the three gradients into one
    fresh buffer (a single concatenation instead of three zero-filled slice
    gradients and their sums) and un-rotates it in place."""

    @staticmethod
    def forward(ctx, qkv, positions, cos_t, sin_t, heads, hd, rot, nq, nk):
        ctx.save_for_backward(positions, cos_t, sin_t)
        ctx.cfg = (heads, hd, rot)
        qkv = qkv.detach()
        native().rope_(qkv, positions, cos_t, sin_t, heads, hd, rot, 1.0)
        q, k, v = qkv[:, :nq], qkv[:, nq : nq + nk], qkv[:, nq + nk :]
        return q, k, v

    @staticmethod
    def backward(ctx, dq, dk, dv):
        positions, cos_t, sin_t = ctx.saved_tensors
        heads, hd, rot = ctx.cfg
        d = torch.cat([dq, dk, dv], dim=-1)
        native().rope_(d, positions, cos_t, sin_t, heads, hd, rot, -1.0)
        return d, None, None, None, None, None, None, None, None


def rope_split(qkv, positions, cos_t, sin_t, heads: int, hd: int, rot: int, nq: int, nk: int):
    """``rope_`` on the first ``heads`` heads of ``qkv`` ([T, nq + nk + nv]) followed by
    the split into ``(q [T, nq], k [T, nk], v [T, rest])``.  On CUDA the buffer is
    rotated in place and the results are views of it: the caller must own ``qkv``
    (a fresh projection output) and must not modify the views in place."""
    if _use_native(qkv) and qkv.requires_grad and torch.is_grad_enabled():
        return _RopeSplitFn.apply(qkv, positions, cos_t, sin_t, heads, hd, rot, nq, nk)
    out = rope_(qkv, positions, cos_t, sin_t, heads, hd, rot)
    return out[:, :nq], out[:, nq : nq + nk], out[:, nq + nk :]


# --------------------------------------------------------------------------- losses
def _row_loss_ref(op: str, logits, targets):
    """fp32 per-row loss and both argmaxes (``logits``/``targets``: [rows, V])."""
    lq = torch.log_softmax(logits.float(), dim=-1)
    lp = torch.log_softmax(targets.float(), dim=-1)
    if op == "kl_div":
        p = lp.exp()
        loss = torch.where(p > 0, p * (lp - lq), torch.zeros_like(p)).sum(-1)
    elif op == "rkl":
        q = lq.exp()
        loss = torch.where(q > 0, q * (lq - lp), torch.zeros_like(q)).sum(-1)
    elif op == "jsd":
        lm = torch.logaddexp(lq, lp) - 0.6931471805599453
        p, q = lp.exp(), lq.exp()
        loss = 0.5 * ((p * (lp - lm)).sum(-1) + (q * (lq - lm)).sum(-1))
    elif op == "ce":
        loss = -lq.gather(-1, targets.argmax(-1, keepdim=True)).squeeze(-1)
    elif op == "tv":
        loss = 1.0 - torch.minimum(lq.exp(), lp.exp()).sum(-1)
    else:
        raise ValueError(f"unknown loss op {op!r}")
    return loss


class _RowLossFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, targets, op, shift, rows, active):
        loss, stats, am_d, am_t = native().loss_fwd(op, logits, targets, active, shift, rows)
        ctx.save_for_backward(logits, targets, stats)
        ctx.cfg = (op, shift, rows)
        ctx.mark_non_differentiable(am_d, am_t)
        return loss, am_d, am_t

    @staticmethod
    def backward(ctx, dloss, _a, _b):
        logits, targets, stats = ctx.saved_tensors
        op, shift, rows = ctx.cfg
        d = native().loss_bwd(op, logits, targets, dloss.contiguous().float(), stats, shift, rows)
        return d, None, None, None, None, None


class _LmHeadLossFn(torch.autograd.Function):
    """``fused_row_loss(op, hidden @ weight.T, targets, shift, rows, active)`` with the head's GEMM
    and the forward reduction of the loss in one kernel: the logits tile is reduced to
    online-softmax records while it is still in tensor memory, so the forward never re-reads
    ``[T, V]`` logits and targets.  The logits are stored (bf16) for the backward pass, which is
    the row-loss backward kernel followed by the input-gradient GEMM."""

    @staticmethod
    def forward(ctx, hidden, weight, targets, op, shift, rows, active):
        logits, loss, stats, am_d, am_t = native().lmhead_loss_fwd(op, hidden, weight, targets, active, shift, rows, gemm_status(hidden.device))
        ctx.save_for_backward(hidden, weight, targets, logits, stats)
        ctx.cfg = (op, shift, rows)
        ctx.mark_non_differentiable(am_d, am_t)
        return loss, am_d, am_t

    @staticmethod
    def backward(ctx, dloss, _a, _b):
        hidden, weight, targets, logits, stats = ctx.saved_tensors
        op, shift, rows = ctx.cfg
        d = native().loss_bwd(op, logits, targets, dloss.contiguous().float(), stats, shift, rows)
        dx, dw = _linear_backward(hidden, weight, (None, None), d, ctx.needs_input_grad[0], ctx.needs_input_grad[1])
        return dx, dw, None, None, None, None, None


FUSED_HEAD_OPS = ("kl_div", "ce")


def lm_head_loss_raw(op: str, hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor, shift: int, rows: int, active):
    """Per-row loss between ``(hidden @ weight.T)[r]`` and ``targets[r + shift]`` for ``r < rows``
    plus both argmaxes (int32), like ``fused_row_loss_raw`` on the product; ``None`` when the
    fused head does not apply (other loss, other dtype / layout, not switched on) and the caller
    should form the logits itself.  Opt-in (``SB200_FUSED_HEAD=1``): at 2048 x 32000 x 4096 the
    fused kernel measured 0.466 ms against 0.443 ms for the GEMM followed by the row-loss
    kernel (its statistics epilogue holds the tensor pipe at 70 % active against 88 % for the
    plain store epilogue), so the two-kernel form is the default."""
    import os

    if (op not in FUSED_HEAD_OPS or not _own_gemm_enabled() or os.environ.get("SB200_FUSED_HEAD", "0") != "1"
            or not (_gemm_operand_ok(hidden) and _gemm_operand_ok(weight) and _gemm_operand_ok(targets))
            or weight.shape[0] % 8 or hidden.shape[0] <= 128):
        return None
    return _LmHeadLossFn.apply(hidden, weight, targets, LOSS_OPS[op], shift, rows, active)


class _StepTailFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, row_loss, pred, target, mask, prev, decay, eps):
        out, weight = native().step_tail(row_loss, pred, target, mask, prev, decay, eps)
        ctx.save_for_backward(weight)
        ctx.mark_dirty(prev)
        ctx.mark_non_differentiable(prev)
        return out, prev

    @staticmethod
    def backward(ctx, dout, _dprev):
        (weight,) = ctx.saved_tensors
        return weight * dout[0], None, None, None, None, None, None


def ttt_step_tail(row_loss, pred_ids, target_ids, mask, prev_correct, decay: float, eps: float):
    """Masked-mean loss of one training-time-test pass and its accuracy counters.

    ``row_loss`` fp32 ``[rows]`` (differentiable), ``pred_ids`` / ``target_ids`` integer
    ``[rows]``, ``mask`` bool / uint8 ``[rows]``, ``prev_correct`` bool / uint8 ``[>= rows]``
    (AND-ed in place with this pass's hits).  Returns fp32 ``[4]``: ``loss =
    decay * sum(row_loss * mask) / (sum(mask) + eps)``, ``correct = sum(prev & hit & mask)``,
    ``total = sum(mask)``, ``cond_total = sum(prev before the update)``.  One launch on
    CUDA; the same arithmetic with torch ops elsewhere."""
    rows = row_loss.shape[0]
    if _use_native(row_loss) and pred_ids.dtype == torch.int32 and target_ids.dtype == torch.int32:
        out, _ = _StepTailFn.apply(row_loss.contiguous(), pred_ids, target_ids, mask, prev_correct, float(decay), float(eps))
        return out
    m = mask[:rows].bool()
    was = prev_correct[:rows].bool()
    cond_total = was.sum().float()
    now = was & (pred_ids[:rows] == target_ids[:rows])
    prev_correct[:rows] = now.to(prev_correct.dtype)
    mf = m.to(row_loss.dtype)
    loss = decay * (row_loss * mf).sum() / (mf.sum() + eps)
    return torch.stack([loss, (now & m).sum().float(), mf.sum().float(), cond_total])


def fused_row_loss_raw(op: str, logits, targets, shift: int, rows: int, active):
    """``fused_row_loss`` on CUDA without the widening of the argmax by-products (int32)."""
    if logits.stride(-1) != 1:
        logits = logits.contiguous()
    if targets.stride(-1) != 1:
        targets = targets.contiguous()
    return _RowLossFn.apply(logits, targets, LOSS_OPS[op], shift, rows, active)


def fused_row_loss(op: str, logits, targets, shift: int = 0, rows: int | None = None, active=None):
    """Per-row loss between ``logits[r]`` and ``targets[r + shift]`` for ``r < rows``.

    Returns ``(loss[rows] fp32, argmax_logits[rows], argmax_targets[rows])``.
    ``active`` (bool[rows], optional) marks rows worth computing; inactive rows get
    loss 0 and sentinel argmaxes (-1 / -2, never equal).  Gradients flow to
    ``logits`` only; the buffer that comes back has ``logits.shape`` with rows
    ``>= rows`` zeroed.
    """
    if logits.dim() != 2 or targets.dim() != 2:
        raise ValueError("fused_row_loss expects [rows, V] inputs")
    if rows is None:
        rows = min(logits.shape[0], targets.shape[0] - shift)
    if _use_native(logits):
        if logits.stride(-1) != 1:
            logits = logits.contiguous()
        if targets.stride(-1) != 1:
            targets = targets.contiguous()
        loss, am_d, am_t = _RowLossFn.apply(logits, targets, LOSS_OPS[op], shift, rows, active)
        return loss, am_d.long(), am_t.long()
    lg = logits[:rows]
    tg = targets[shift : shift + rows]
    loss = _row_loss_ref(op, lg, tg)
    am_d, am_t = lg.argmax(-1), tg.argmax(-1)
    if active is not None:
        act = active.bool()
        loss = torch.where(act, loss, torch.zeros_like(loss))
        am_d = torch.where(act, am_d, torch.full_like(am_d, -1))
        am_t = torch.where(act, am_t, torch.full_like(am_t, -2))
    return loss, am_d, am_t


class _TokenCEFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, keep):
        loss, stats = native().ce_label_fwd(logits, labels, keep)
        ctx.save_for_backward(logits, stats)
        return loss

    @staticmethod
    def backward(ctx, dloss):
        logits, stats = ctx.saved_tensors
        # the CE backward only needs the saved label (stats[4]) and the draft statistics
        d = native().loss_bwd(LOSS_OPS["ce"], logits, logits, dloss.contiguous().float(), stats, 0, logits.shape[0])
        return d, None, None


def token_cross_entropy(logits: torch.Tensor, labels: torch.Tensor, keep: torch.Tensor | None = None) -> torch.Tensor:
    """Per-row cross-entropy of ``logits [n, V]`` against integer ``labels [n]``;
    rows with ``keep == False`` contribute 0 (and no gradient)."""
    if _use_native(logits):
        if logits.stride(-1) != 1:
            logits = logits.contiguous()
        keep_b = keep.to(torch.bool).contiguous() if keep is not None else None
        return _TokenCEFn.apply(logits, labels.long().contiguous(), keep_b)
    loss = F.cross_entropy(logits.float(), labels.long(), reduction="none")
    return loss if keep is None else torch.where(keep.bool(), loss, torch.zeros_like(loss))


# --------------------------------------------------------------------------- optimizer
def sum_of_squares(flat: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> torch.Tensor:
    """``out[0] (+)= sum(flat**2)`` in fp32, deterministic two-stage reduction."""
    if _use_native(flat):
        native().sumsq(flat, out, accumulate)
    else:
        s = flat.float().pow(2).sum()
        out[0] = out[0] + s if accumulate else s
    return out


HYPER_LEN = 16


def adamw_step_(master, m, v, grad, w16, hyper, norm_sq=None) -> None:
    """One fused AdamW step over flat buffers.  ``hyper`` (fp32[16], same device):
    lr, beta1, beta2, eps, weight_decay, bias_correction1, bias_correction2,
    max_grad_norm (<= 0 disables clipping), grad_scale.  ``norm_sq`` holds the global
    sum of squared (unscaled) gradients.  ``w16`` (optional) receives the bf16 copy."""
    if _use_native(master):
        native().adamw(master, m, v, grad, w16, hyper, norm_sq)
        return
    lr, b1, b2, eps, wd, bc1, bc2, max_norm, gscale = (float(hyper[i]) for i in range(9))
    if max_norm > 0 and norm_sq is not None:
        coef = max_norm / (gscale * float(norm_sq[0]) ** 0.5 + 1e-6)
        if coef < 1.0:
            gscale *= coef
    g = grad.float() * gscale
    master.mul_(1 - lr * wd)
    m.mul_(b1).add_(g, alpha=1 - b1)
    v.mul_(b2).addcmul_(g, g, value=1 - b2)
    denom = v.sqrt() / (bc2**0.5) + eps
    master.addcdiv_(m, denom, value=-lr / bc1)
    if w16 is not None:
        w16.copy_(master)
