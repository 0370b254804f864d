"""P-EAGLE loss and per-depth accuracy (src/speculators/models/peagle/metrics.py:17-77):
compound loss over the sampled rows with no position decay, accuracy split by depth."""

from __future__ import annotations

import torch

from speculators_b200.losses import LossConfig, kl_div_loss, reduce_masked
from speculators_b200.losses.rowwise import rowwise_terms
from speculators_b200.models.metrics import compute_accuracy_multi_step

__all__ = ["compute_metrics"]


def compute_metrics(logits, targets, loss_mask, anchor_pos, depth, num_depths: int, loss_config: LossConfig | None = None,
                    row_valid: torch.Tensor | None = None):
    if loss_config is None:
        loss_config = {"kl_div": (kl_div_loss, 1.0)}
    device = logits.device
    n = logits.shape[1]
    sampled_mask = loss_mask.reshape(-1)[anchor_pos + depth].unsqueeze(0)
    if row_valid is not None:  # padding rows of the fixed-shape sampler take no part
        sampled_mask = sampled_mask * row_valid.to(sampled_mask.dtype).unsqueeze(0)
    pos = depth.unsqueeze(0)
    per_term, pred_ids, target_ids = rowwise_terms(
        loss_config, logits.reshape(n, -1), targets.reshape(n, -1), shift=0, rows=n, active=sampled_mask.reshape(-1).bool()
    )
    loss = torch.zeros((), device=device, dtype=torch.float32)
    parts = {}
    for name, (_, weight) in loss_config.items():
        term = reduce_masked(per_term[name].unsqueeze(0), sampled_mask, pos, None)
        if len(loss_config) > 1:
            parts[f"{name}_loss"] = term.detach()
        loss = loss + weight * term
    with torch.no_grad():
        correct, total = compute_accuracy_multi_step(pred_ids.unsqueeze(0), target_ids.unsqueeze(0), sampled_mask, pos, num_depths)
    one = torch.ones((), device=device)
    metrics = {"loss_sum": loss.detach(), "loss_total": one, "full_acc_sum": correct.sum(), "full_acc_total": total.sum()}
    for name, value in parts.items():
        metrics[f"{name}_sum"] = value
        metrics[f"{name}_total"] = one.clone()
    for d in range(num_depths):
        metrics[f"position_{d}_acc_sum"] = correct[d]
        metrics[f"position_{d}_acc_total"] = total[d]
    return loss, metrics
