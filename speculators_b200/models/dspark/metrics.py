"""DSpark loss and metrics (src/speculators/models/dspark/metrics.py:49-163):
``loss = compound(logits, targets) + alpha * BCE(confidence, accept_rate)`` where
``accept_rate = 1 - TV(logits, targets)`` is computed analytically and detached;
plus calibration counters and the expected accepted length per block."""

from __future__ import annotations

import torch
from torch.nn.functional import binary_cross_entropy_with_logits

from speculators_b200.losses import LossConfig, tv_loss
from speculators_b200.models.dflash.metrics import block_decay_fn, weighted_terms
from speculators_b200.models.metrics import compute_accuracy_multi_step

__all__ = ["compute_metrics"]

_EPS = 1e-8


def _masked_decayed_mean(elementwise, loss_mask, pos_idx, decay_fn):
    mask = loss_mask.to(elementwise.dtype)
    weighted = elementwise * mask
    if decay_fn is not None:
        weighted = weighted * decay_fn(pos_idx.to(weighted.dtype), elementwise_loss=elementwise)
    return (weighted.sum(dim=1) / (mask.sum(dim=1) + _EPS)).mean()


def compute_metrics(logits, targets, confidence_logits, loss_mask, block_size: int, loss_config: LossConfig, tv_loss_fn=tv_loss,
                    gamma: float = 4.0, confidence_head_alpha: float = 1.0, per_position_loss_weight: str = "fixed-exp-decay",
                    dpace_alpha: float = 0.5, sample_from_anchor: bool = True):
    device = logits.device
    n = logits.shape[1]
    pos_idx = (torch.arange(n, device=device) % block_size).unsqueeze(0)
    start = 0 if sample_from_anchor else 1
    decay = block_decay_fn(per_position_loss_weight, loss_mask, block_size, gamma, dpace_alpha, sample_from_anchor)
    loss, parts, pred_ids, target_ids = weighted_terms(loss_config, logits, targets, loss_mask, pos_idx, decay)

    with torch.no_grad():
        accept_rate = 1.0 - tv_loss_fn(logits.detach(), targets)  # [1, n]
        blocks = n // block_size
        draft_mask = loss_mask.to(accept_rate.dtype).view(blocks, block_size)[:, start:]
        accept_prefix = (accept_rate.view(blocks, block_size)[:, start:] * draft_mask).cumprod(dim=-1)

    metrics: dict[str, torch.Tensor] = {}
    if confidence_logits is not None:
        bce = binary_cross_entropy_with_logits(confidence_logits.float(), accept_rate.detach().float(), reduction="none")
        conf_loss = _masked_decayed_mean(bce, loss_mask, pos_idx, decay)
        loss = loss + confidence_head_alpha * conf_loss
        with torch.no_grad():
            mask_f = loss_mask.to(accept_rate.dtype)
            total = mask_f.sum().clamp_min(1.0)
            prob = confidence_logits.float().sigmoid()
            metrics["confidence_loss_sum"] = conf_loss.detach().clone()
            metrics["confidence_loss_total"] = torch.ones((), device=device)
            metrics["confidence_abs_error_sum"] = ((prob - accept_rate).abs() * mask_f).sum()
            metrics["confidence_abs_error_total"] = total
            metrics["confidence_pred_mean_sum"] = (prob * mask_f).sum()
            metrics["confidence_pred_mean_total"] = total.clone()
            conf_prefix = (prob.view(blocks, block_size)[:, start:] * draft_mask).cumprod(dim=-1)
            metrics["confidence_cumprod_bias_sum"] = ((conf_prefix - accept_prefix) * draft_mask).sum()
            metrics["confidence_cumprod_bias_total"] = draft_mask.sum().clamp_min(1.0)

    one = torch.ones((), device=device)
    metrics["loss_sum"] = loss.detach().clone()
    metrics["loss_total"] = one
    for name, value in parts.items():
        metrics[f"{name}_sum"] = value
        metrics[f"{name}_total"] = one.clone()
    with torch.no_grad():
        mask_f = loss_mask.to(accept_rate.dtype)
        metrics["accept_rate_sum"] = (accept_rate * mask_f).sum()
        metrics["accept_rate_total"] = mask_f.sum().clamp_min(1.0)
        block_len = accept_prefix.sum(dim=-1) + 1.0
        block_valid = (draft_mask.sum(dim=-1) > 0).to(accept_rate.dtype)
        metrics["accept_len_sum"] = (block_len * block_valid).sum()
        metrics["accept_len_total"] = block_valid.sum().clamp_min(1.0)
    correct, total_pos = compute_accuracy_multi_step(pred_ids.unsqueeze(0), target_ids.unsqueeze(0), loss_mask, pos_idx, block_size)
    metrics["full_acc_sum"] = correct[start:].sum()
    metrics["full_acc_total"] = total_pos[start:].sum()
    for pos in range(start, block_size):
        metrics[f"position_{pos}_acc_sum"] = correct[pos]
        metrics[f"position_{pos}_acc_total"] = total_pos[pos]
    return loss, metrics
