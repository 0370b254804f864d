"""Accuracy counters shared by the algorithms.  Everything is returned as raw
``(sum, total)`` counts so ranks can be summed before dividing, and nothing here
synchronises with the host (no ``masked_select`` / data-dependent shapes), which
keeps a training step capturable in a CUDA graph.  Semantics:
src/speculators/models/metrics.py:6-69."""

from __future__ import annotations

import torch

__all__ = ["compute_accuracy_multi_step", "compute_accuracy_single_step"]


def compute_accuracy_single_step(pred_ids, target_ids, loss_mask=None, prev_correct=None):
    """Returns ``(full_correct, full_total, cond_correct, cond_total)``.

    ``prev_correct`` (bool, same shape) is AND-ed in place with this step's hits;
    ``cond_total`` is how many positions were still all-correct before this step.
    Counts are restricted to ``loss_mask`` when it is given.
    """
    hit = pred_ids == target_ids
    if prev_correct is not None:
        cond_total = prev_correct.sum().float()
        prev_correct.logical_and_(hit)
        hit = prev_correct
    else:
        cond_total = torch.tensor(float(hit.numel()), device=hit.device)
    if loss_mask is not None:
        mask = loss_mask.to(torch.bool)
        correct = (hit & mask).sum().float()
        total = mask.sum().float()
    else:
        correct = hit.sum().float()
        total = torch.tensor(float(hit.numel()), device=hit.device)
    return correct, total, correct.clone(), cond_total


@torch.no_grad()
def compute_accuracy_multi_step(pred_ids, target_ids, loss_mask, pos_idx, num_pos: int):
    """Per-block-position ``(correct[num_pos], total[num_pos])`` over masked positions."""
    mask = loss_mask.to(torch.bool).reshape(-1)
    hit = ((pred_ids == target_ids).reshape(-1) & mask).float()
    pos = pos_idx.reshape(-1).long()
    correct = torch.zeros(num_pos, dtype=torch.float, device=hit.device).scatter_add_(0, pos, hit)
    total = torch.zeros(num_pos, dtype=torch.float, device=hit.device).scatter_add_(0, pos, mask.float())
    return correct, total
