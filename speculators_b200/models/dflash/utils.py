"""Anchor selection and block indexing for DFlash / DSpark.

``select_anchors`` draws up to ``num_anchors`` distinct positions uniformly from
the loss-masked positions (the last ``block_size`` positions are never anchors),
returns them sorted and padded with zeros, plus a validity flag per slot
(src/speculators/models/dflash/utils.py:21-67).  It is written with fixed output
shapes and without reading anything back to the host -- a random key per
position, ``topk`` of the keys -- so the training step stays capturable in a
CUDA graph; the reference uses ``nonzero`` + ``randperm``, which yields the same
distribution but synchronises.
"""

from __future__ import annotations

import torch

__all__ = ["get_base_indices_for_anchored_blocks", "select_anchors"]


def get_base_indices_for_anchored_blocks(anchor_positions: torch.Tensor, block_size: int) -> torch.Tensor:
    """``[num_anchors] -> [num_anchors * block_size]``: anchor, anchor+1, ..."""
    a = anchor_positions.to(torch.long).reshape(-1)
    return (a[:, None] + torch.arange(block_size, device=a.device, dtype=torch.long)[None, :]).reshape(-1)


def select_anchors(loss_mask: torch.Tensor, num_anchors: int, block_size: int):
    if loss_mask.ndim != 2:
        raise ValueError(f"Expected [B, T], got {loss_mask.shape}")
    if block_size <= 0:
        raise ValueError(f"Expected block size > 0, got {block_size}")
    valid = loss_mask[0].bool().clone()
    valid[-block_size:] = False
    T = valid.shape[0]
    device = valid.device
    keys = torch.where(valid, torch.rand(T, device=device), torch.full((T,), 2.0, device=device))
    k = min(num_anchors, T)
    picked_keys, picked = torch.topk(keys, k, largest=False)
    ok = picked_keys < 2.0
    # valid picks first in ascending position order, invalid slots behind them
    order = torch.sort(torch.where(ok, picked, torch.full_like(picked, T))).values
    ok_sorted = order < T
    anchors = torch.zeros(num_anchors, dtype=torch.long, device=device)
    anchor_valid = torch.zeros(num_anchors, dtype=torch.bool, device=device)
    anchors[:k] = torch.where(ok_sorted, order, torch.zeros_like(order))
    anchor_valid[:k] = ok_sorted
    return anchors, anchor_valid
