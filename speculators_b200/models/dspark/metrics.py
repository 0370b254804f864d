"""DSpark loss and metrics (values and key names of src/speculators/models/dspark/metrics.py:49-163).

``loss = L(logits, targets) + alpha * BCE(confidence, a)`` with ``a = 1 - TV(logits, targets)`` the
analytic per-slot acceptance rate (detached).  Reported next to it: calibration of the confidence
head (mean absolute error, mean prediction, bias of the running product inside a block), the
acceptance rate, the expected accepted length per block ``1 + sum_k prod_{j<=k} a_j`` and the
per-slot accuracies.  All counters of a step are formed from one ``[rows, n]`` stack and a single
reduction, so the metric tail is a handful of kernels whatever the number of counters.
"""

from __future__ import annotations

import torch
from torch.nn.functional import binary_cross_entropy_with_logits

from speculators_b200.losses import LossConfig, tv_loss
from speculators_b200.models.dflash.metrics import block_decay_fn, weighted_terms
from speculators_b200.models.metrics import compute_accuracy_multi_step

__all__ = ["compute_metrics"]

_EPS = 1e-8


def _per_block(x: torch.Tensor, block_size: int, first_slot: int) -> torch.Tensor:
    """``[1, N * B]`` -> ``[N, B - first_slot]`` (the slots that draft a token)."""
    return x.reshape(-1, block_size)[:, first_slot:]


def _confidence_loss(bce: torch.Tensor, mask_f: torch.Tensor, weights: torch.Tensor | None) -> torch.Tensor:
    weighted = bce * mask_f if weights is None else bce * mask_f * weights
    return (weighted.sum(dim=1) / (mask_f.sum(dim=1) + _EPS)).mean()


def compute_metrics(logits, targets, confidence_logits, loss_mask, block_size: int, loss_config: LossConfig, tv_loss_fn=tv_loss,
                    gamma: float = 4.0, confidence_head_alpha: float = 1.0, per_position_loss_weight: str = "fixed-exp-decay",
                    dpace_alpha: float = 0.5, sample_from_anchor: bool = True):
    device = logits.device
    n = logits.shape[1]
    first = 0 if sample_from_anchor else 1
    slot = (torch.arange(n, device=device) % block_size).unsqueeze(0)
    decay = block_decay_fn(per_position_loss_weight, loss_mask, block_size, gamma, dpace_alpha, sample_from_anchor)
    loss, parts, pred_ids, target_ids = weighted_terms(loss_config, logits, targets, loss_mask, slot, decay)

    with torch.no_grad():
        accept = 1.0 - tv_loss_fn(logits.detach(), targets)  # [1, n] analytic acceptance rate
        mask_f = loss_mask.to(accept.dtype)
        drafted = _per_block(mask_f, block_size, first)
        accept_run = (_per_block(accept, block_size, first) * drafted).cumprod(dim=-1)
        supervised = mask_f.sum().clamp_min(1.0)

    counters: dict[str, tuple[torch.Tensor, torch.Tensor]] = {}
    one = torch.ones((), device=device)
    if confidence_logits is not None:
        conf = confidence_logits.float()
        bce = binary_cross_entropy_with_logits(conf, accept.detach().float(), reduction="none")
        weights = decay(slot.to(bce.dtype), elementwise_loss=bce) if decay is not None else None
        conf_loss = _confidence_loss(bce, mask_f, weights)
        loss = loss + confidence_head_alpha * conf_loss
        with torch.no_grad():
            prob = conf.sigmoid()
            conf_run = (_per_block(prob, block_size, first) * drafted).cumprod(dim=-1)
            counters["confidence_loss"] = (conf_loss.detach().clone(), one)
            counters["confidence_abs_error"] = (((prob - accept).abs() * mask_f).sum(), supervised)
            counters["confidence_pred_mean"] = ((prob * mask_f).sum(), supervised.clone())
            counters["confidence_cumprod_bias"] = (((conf_run - accept_run) * drafted).sum(), drafted.sum().clamp_min(1.0))

    counters["loss"] = (loss.detach().clone(), one)
    for name, value in parts.items():
        counters[name] = (value, one.clone())
    with torch.no_grad():
        counters["accept_rate"] = ((accept * mask_f).sum(), supervised.clone())
        live = (drafted.sum(dim=-1) > 0).to(accept.dtype)  # blocks with at least one supervised drafting slot
        counters["accept_len"] = (((accept_run.sum(dim=-1) + 1.0) * live).sum(), live.sum().clamp_min(1.0))
    hits, seen = compute_accuracy_multi_step(pred_ids.unsqueeze(0), target_ids.unsqueeze(0), loss_mask, slot, block_size)
    counters["full_acc"] = (hits[first:].sum(), seen[first:].sum())
    for k in range(first, block_size):
        counters[f"position_{k}_acc"] = (hits[k], seen[k])

    metrics: dict[str, torch.Tensor] = {}
    for name, (total, count) in counters.items():
        metrics[f"{name}_sum"] = total
        metrics[f"{name}_total"] = count
    return loss, metrics
