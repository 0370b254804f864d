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

__all__ = ["cod_capacities", "generate_cod_sample_indices", "generate_cod_sample_indices_fixed"]


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


def cod_capacities(seq_length: int, num_depths: int, down_sample_ratio: float, down_sample_ratio_min: float,
                   max_anchors: int | None = None) -> list[int]:
    """Upper bound of the number of rows per depth (depth 0 first): what the sampler
    would keep if every position were inside the loss mask."""
    seeds = seq_length if max_anchors is None else min(seq_length, max_anchors)
    caps = [seq_length]
    for d in range(1, num_depths):
        want = int(max(0, seeds - d) * max(down_sample_ratio**d, down_sample_ratio_min))
        if want <= 0:
            break
        caps.append(want)
    return caps


def _random_subset(member: torch.Tensor, count: torch.Tensor, capacity: int, generator=None) -> tuple[torch.Tensor, torch.Tensor]:
    """``min(count, member.sum())`` positions drawn uniformly without replacement from the
    set ``member`` (bool ``[T]``), ascending, in a ``[capacity]`` array padded with ``T``;
    second result: which entries are real.  Fixed shapes, no host synchronisation."""
    T = member.shape[0]
    keys = torch.rand(T, device=member.device, generator=generator)
    keys = torch.where(member, keys, torch.full_like(keys, 2.0))
    order = torch.argsort(keys)[:capacity]  # members first, in random order
    take = torch.minimum(count, member.sum())
    real = torch.arange(capacity, device=member.device) < take
    picked = torch.where(real, order, torch.full_like(order, T)).sort().values
    return picked, picked < T


def generate_cod_sample_indices_fixed(
    seq_length: int, loss_mask: torch.Tensor, num_depths: int = 8, down_sample_ratio: float = 0.7,
    down_sample_ratio_min: float = 0.2, filter_position_zero: bool = True, max_anchors: int | None = None, generator=None,
):
    """Same sampling law as ``generate_cod_sample_indices`` with shapes that depend only
    on the arguments (``sum(cod_capacities(...))`` rows), so the step can be captured in a
    CUDA graph: -> ``(anchor_pos, depth, row_valid)``.  Rows that the variable-shape
    sampler would not have produced carry ``row_valid = False`` (``anchor_pos = 0``); every
    count that depends on the mask (valid positions, pool sizes, ``want``) stays on the
    device."""
    T = seq_length
    mask = loss_mask.reshape(-1)
    device = mask.device
    is_valid = mask == 1
    caps = cod_capacities(T, num_depths, down_sample_ratio, down_sample_ratio_min, max_anchors)
    n_valid = is_valid.sum()
    if max_anchors is not None and max_anchors < T:
        seed_pos, seed_real = _random_subset(is_valid, torch.full_like(n_valid, max_anchors), max_anchors, generator)
        pool = torch.zeros(T + 1, dtype=torch.bool, device=device)
        pool[seed_pos] = seed_real
        pool = pool[:T]
        n_seeds = torch.clamp(n_valid, max=max_anchors)
    else:
        pool, n_seeds = is_valid, n_valid
    anchors = [torch.arange(T, device=device)]
    depths = [torch.zeros(T, dtype=torch.long, device=device)]
    valids = [torch.ones(T, dtype=torch.bool, device=device)]
    for d, cap in enumerate(caps[1:], start=1):
        factor = max(down_sample_ratio**d, down_sample_ratio_min)
        want = (torch.clamp(n_seeds - d, min=0).double() * factor).floor().long()
        picked, real = _random_subset(pool, want, cap, generator)
        nxt = torch.where(real, (picked + 1) % T, torch.full_like(picked, T))
        ok = real & is_valid[nxt.clamp(max=T - 1)]
        if filter_position_zero:
            ok = ok & (nxt != 0)
        nxt_pool = torch.zeros(T + 1, dtype=torch.bool, device=device)
        # index_fill_ takes the value as a kernel argument; ``pool[idx] = True`` would copy a host scalar,
        # which a CUDA graph capture refuses
        nxt_pool.index_fill_(0, torch.where(ok, nxt, torch.full_like(nxt, T)), True)
        pool = nxt_pool[:T]
        anchors.append(torch.where(real, picked - d, torch.zeros_like(picked)))
        depths.append(torch.full((cap,), d, dtype=torch.long, device=device))
        valids.append(real)
    return torch.cat(anchors), torch.cat(depths), torch.cat(valids)
