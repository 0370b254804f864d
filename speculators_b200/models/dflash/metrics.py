"""DFlash loss / accuracy / expected-accepted-length
(src/speculators/models/dflash/metrics.py:20-108)."""

from __future__ import annotations

from functools import partial

import torch

from speculators_b200.losses import LossConfig, dflash_loss_decay, dpace_loss_decay, kl_div_loss, reduce_masked
from speculators_b200.losses.rowwise import rowwise_terms
from speculators_b200.models.metrics import compute_accuracy_multi_step

__all__ = ["block_decay_fn", "compute_metrics", "weighted_terms"]


def block_decay_fn(per_position_loss_weight: str, loss_mask, block_size: int, gamma: float, dpace_alpha: float, sample_from_anchor: bool):
    if per_position_loss_weight == "dpace":
        return partial(dpace_loss_decay, loss_mask=loss_mask, block_size=block_size, dpace_alpha=dpace_alpha)
    return partial(dflash_loss_decay, gamma=gamma, sample_from_anchor=sample_from_anchor)


def weighted_terms(loss_config: LossConfig, logits, targets, loss_mask, pos_idx, decay_fn):
    """-> (loss, {term scalars}, pred_ids, target_ids)"""
    n = logits.shape[1]
    per_term, pred_ids, target_ids = rowwise_terms(
        loss_config, logits.reshape(n, -1), targets.reshape(n, -1), shift=0, rows=n, active=None
    )
    loss = torch.zeros((), device=logits.device, dtype=torch.float32)
    parts = {}
    for name, (_, weight) in loss_config.items():
        term = reduce_masked(per_term[name].unsqueeze(0), loss_mask, pos_idx, decay_fn)
        if len(loss_config) > 1:
            parts[f"{name}_loss"] = term.detach()
        loss = loss + weight * term
    return loss, parts, pred_ids, target_ids


def compute_metrics(logits, targets, loss_mask, block_size: int = 1, gamma: float = 4.0, loss_config: LossConfig | None = None,
                    per_position_loss_weight: str = "fixed-exp-decay", dpace_alpha: float = 0.5, sample_from_anchor: bool = False):
    if loss_config is None:
        loss_config = {"kl_div": (kl_div_loss, 1.0)}
    device = logits.device
    n = logits.shape[1]
    pos_idx = (torch.arange(n, device=device) % block_size).unsqueeze(0)
    decay = block_decay_fn(per_position_loss_weight, loss_mask, block_size, gamma, dpace_alpha, sample_from_anchor)
    loss, parts, pred_ids, target_ids = weighted_terms(loss_config, logits, targets, loss_mask, pos_idx, decay)
    correct, total = compute_accuracy_multi_step(pred_ids.unsqueeze(0), target_ids.unsqueeze(0), loss_mask, pos_idx, block_size)
    one = torch.ones((), device=device)
    metrics = {"loss_sum": loss.detach().clone(), "loss_total": one}
    for name, value in parts.items():
        metrics[f"{name}_sum"] = value
        metrics[f"{name}_total"] = one.clone()
    start = 0 if sample_from_anchor else 1
    metrics["full_acc_sum"] = correct[start:].sum()
    metrics["full_acc_total"] = total[start:].sum()
    eal = torch.zeros((), device=device)
    run = torch.ones((), device=device)
    for pos in range(start, block_size):
        metrics[f"position_{pos}_acc_sum"] = correct[pos]
        metrics[f"position_{pos}_acc_total"] = total[pos]
        run = run * (correct[pos] / total[pos].clamp(min=1.0))
        eal = eal + run
    metrics["eal_sum"] = eal
    metrics["eal_total"] = one.clone()
    return loss, metrics
