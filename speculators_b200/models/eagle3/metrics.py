"""Per-TTT-step loss and accuracy for EAGLE-3.

Step ``s`` compares ``logits[:T-s]`` with ``targets[s:]`` under ``loss_mask[s:]``
(src/speculators/models/eagle3/metrics.py:16-119).  The fused path passes the
shift to the row-loss kernel instead of slicing, so the gradient comes back for
the full ``[T, V]`` logits without a padded copy, and both argmaxes for the
accuracy counters are produced by the same kernel launch.
"""

from __future__ import annotations

from functools import partial

import torch

from speculators_b200.losses import LossConfig, exp_loss_decay, kl_div_loss, reduce_masked
from speculators_b200.losses.rowwise import rowwise_terms
from speculators_b200.models.metrics import compute_accuracy_single_step

__all__ = ["align_for_step", "compute_metrics", "compute_metrics_from_hidden"]


def align_for_step(logits, targets, loss_mask, prev_correct, ttt_step: int):
    """Slice views that line up draft step ``ttt_step`` with its targets."""
    if ttt_step > 0:
        logits = logits[:, :-ttt_step]
        prev_correct = prev_correct[:, :-ttt_step] if prev_correct is not None else None
    targets = targets[:, ttt_step:]
    loss_mask = loss_mask[:, ttt_step:] if loss_mask is not None else None
    return logits, targets, loss_mask, prev_correct


USE_FUSED_TAIL = True  # tests flip this to compare against the op-by-op formulation


def _single_fused_primitive(loss_config: LossConfig) -> tuple[str, float] | None:
    """``(kernel op, weight)`` when the configuration is one fused primitive term."""
    from speculators_b200.losses.rowwise import _PRIMITIVES, _is_fused
    from speculators_b200.losses.utils import loss_name_of

    if len(loss_config) != 1:
        return None
    (fn, weight), = loss_config.values()
    name = loss_name_of(fn)
    return (name, float(weight)) if name in _PRIMITIVES and _is_fused(fn) else None


def _compute_metrics_fused(logits, targets, loss_mask, prev_correct, ttt_step: int, decay: float, op: str, weight: float, head=None):
    """CUDA fast path for one fused loss term: row-loss kernel + one tail kernel (masked
    mean, decay, accuracy counters, ``prev_correct`` update) instead of ~30 small ops.  With
    ``head = (hidden [T, H], lm_head weight)`` instead of ``logits`` the head's GEMM and the
    forward reduction of the loss run as one kernel (``None`` is returned if that does not apply)."""
    from speculators_b200 import ops
    from speculators_b200.losses.utils import _REDUCTION_EPS

    T = logits.shape[1] if head is None else head[0].shape[0]
    rows = T - ttt_step
    mask_u8 = loss_mask.reshape(-1)[ttt_step:]
    if mask_u8.dtype not in (torch.bool, torch.uint8):
        mask_u8 = mask_u8 != 0
    prev_flat = prev_correct.reshape(-1)
    active = mask_u8.bool() | prev_flat[:rows]
    if head is None:
        row_loss, pred, tgt = ops.fused_row_loss_raw(op, logits.reshape(T, -1), targets.reshape(targets.shape[1], -1), ttt_step, rows, active)
    else:
        fused = ops.lm_head_loss_raw(op, head[0], head[1], targets.reshape(targets.shape[1], -1), ttt_step, rows, active)
        if fused is None:
            return None
        row_loss, pred, tgt = fused
    out = ops.ttt_step_tail(row_loss, pred, tgt, mask_u8.contiguous(), prev_flat, decay, _REDUCTION_EPS)
    loss = out[0] * weight if weight != 1.0 else out[0]
    stats = out.detach()
    one = torch.ones((), device=row_loss.device)
    metrics = {
        f"loss_{ttt_step}_sum": stats[0] * weight if weight != 1.0 else stats[0], f"loss_{ttt_step}_total": one,
        f"full_acc_{ttt_step}_sum": stats[1], f"full_acc_{ttt_step}_total": stats[2],
        f"cond_acc_{ttt_step}_sum": stats[1], f"cond_acc_{ttt_step}_total": stats[3],
    }
    return loss, metrics


def compute_metrics_from_hidden(hidden, head_weight, targets, loss_mask, prev_correct, ttt_step: int, ttt_step_loss_decay: float,
                                loss_config: LossConfig | None = None):
    """``compute_metrics`` of ``hidden @ head_weight.T`` without a separate pass over the
    logits: the lm_head GEMM's epilogue reduces each tile for the loss.  Returns ``None`` when
    that path does not apply (not CUDA bf16, a loss other than one fused KL / CE term, ...);
    the caller then forms the logits and calls ``compute_metrics``."""
    if loss_config is None:
        loss_config = {"kl_div": (kl_div_loss, 1.0)}
    if not (USE_FUSED_TAIL and hidden.is_cuda and hidden.dtype == torch.bfloat16 and hidden.dim() == 2 and loss_mask is not None
            and prev_correct is not None and prev_correct.dtype == torch.bool and prev_correct.is_contiguous()):
        return None
    single = _single_fused_primitive(loss_config)
    if single is None:
        return None
    return _compute_metrics_fused(None, targets, loss_mask, prev_correct, ttt_step, float(ttt_step_loss_decay) ** ttt_step, *single,
                                  head=(hidden, head_weight))


def compute_metrics(logits, targets, loss_mask, prev_correct, ttt_step: int, ttt_step_loss_decay: float, loss_config: LossConfig | None = None):
    """Returns ``(step_loss, metrics)``; updates ``prev_correct`` in place."""
    if loss_config is None:
        loss_config = {"kl_div": (kl_div_loss, 1.0)}
    if USE_FUSED_TAIL and logits.is_cuda and logits.dtype == torch.bfloat16 and loss_mask is not None and prev_correct is not None and prev_correct.dtype == torch.bool:
        single = _single_fused_primitive(loss_config)
        if single is not None and prev_correct.is_contiguous():
            return _compute_metrics_fused(logits, targets, loss_mask, prev_correct, ttt_step, float(ttt_step_loss_decay) ** ttt_step, *single)
    T = logits.shape[1]
    rows = T - ttt_step
    device = logits.device
    s_mask = loss_mask[:, ttt_step:] if loss_mask is not None else torch.ones(1, rows, dtype=torch.bool, device=device)
    s_prev = prev_correct[:, :rows] if prev_correct is not None else None
    active = s_mask.to(torch.bool).reshape(-1)
    if s_prev is not None:
        active = active | s_prev.reshape(-1)
    pos_idx = torch.full((1, rows), ttt_step, device=device, dtype=torch.long)
    decay = partial(exp_loss_decay, gamma=ttt_step_loss_decay)

    per_term, pred_ids, target_ids = rowwise_terms(
        loss_config, logits.reshape(T, -1), targets.reshape(targets.shape[1], -1), shift=ttt_step, rows=rows, active=active
    )
    total = torch.zeros((), device=device, dtype=torch.float32)
    term_scalars = {}
    for name, (_, weight) in loss_config.items():
        term = reduce_masked(per_term[name].unsqueeze(0), s_mask, pos_idx, decay)
        if len(loss_config) > 1:
            term_scalars[f"{name}_loss"] = term.detach()
        total = total + weight * term

    full_c, full_t, cond_c, cond_t = compute_accuracy_single_step(
        pred_ids.unsqueeze(0), target_ids.unsqueeze(0), s_mask, s_prev
    )
    one = torch.ones((), device=device)
    metrics = {f"loss_{ttt_step}_sum": total.detach().clone(), f"loss_{ttt_step}_total": one}
    for name, value in term_scalars.items():
        metrics[f"{name}_{ttt_step}_sum"] = value
        metrics[f"{name}_{ttt_step}_total"] = one.clone()
    metrics[f"full_acc_{ttt_step}_sum"] = full_c
    metrics[f"full_acc_{ttt_step}_total"] = full_t
    metrics[f"cond_acc_{ttt_step}_sum"] = cond_c
    metrics[f"cond_acc_{ttt_step}_total"] = cond_t
    return total, metrics
