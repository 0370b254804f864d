"""COD (conditional-on-distribution) sampling for P-EAGLE.

Depth 0 keeps every position.  Depth ``d >= 1`` keeps
``int((n_valid - d) * max(r**d, r_min))`` positions drawn from the successors of
the previous depth's picks that are still inside the loss mask, so deeper
prediction groups get geometrically fewer rows.  Each kept row is identified by
the position its rollout started from (``anchor_pos``) and its ``depth``; the
token it stands for sits at ``anchor_pos + depth``.  Semantics:
src/speculators/models/peagle/data.py:6-86.
"""

from __future__ import annotations

import torch

__all__ = ["generate_cod_sample_indices"]


def generate_cod_sample_indices(
    seq_length: int, loss_mask: torch.Tensor, num_depths: int = 8, down_sample_ratio: float = 0.7,
    down_sample_ratio_min: float = 0.2, filter_position_zero: bool = True, max_anchors: int | None = None,
):
    """-> ``(anchor_pos, depth)``, both int64 ``[total_sampled]``, depth-major."""
    mask = loss_mask.reshape(-1)
    device = mask.device
    valid = torch.nonzero(mask == 1, as_tuple=False).squeeze(-1)
    seeds = valid
    if max_anchors is not None and valid.numel() > max_anchors:
        seeds = valid[torch.randperm(valid.numel(), device=device)[:max_anchors]].sort().values
    is_valid = torch.zeros(seq_length, dtype=torch.bool, device=device)
    is_valid[valid] = True
    anchors = [torch.arange(seq_length, device=device)]
    depths = [torch.zeros(seq_length, dtype=torch.long, device=device)]
    pool = seeds
    for d in range(1, num_depths):
        want = int(max(0, seeds.numel() - d) * max(down_sample_ratio**d, down_sample_ratio_min))
        if want <= 0:
            break
        if pool.numel() >= want:
            picked = pool[torch.randperm(pool.numel(), device=device)[:want]].sort().values
        else:
            picked = pool
        nxt = (picked + 1) % seq_length
        if filter_position_zero:
            nxt = nxt[nxt != 0]
        pool = nxt[is_valid[nxt]]
        anchors.append(picked - d)
        depths.append(torch.full((picked.numel(),), d, dtype=torch.long, device=device))
    return torch.cat(anchors), torch.cat(depths)
