"""P-EAGLE attention pattern as an ``AttnSpec``.

Rows are the COD samples, depth-major: the first ``T`` rows are depth 0 (one per
original position), later rows belong to rollouts ``(anchor, depth >= 1)``.  A
query ``(a, d)`` sees

* depth-0 keys at positions ``<= a`` of the same document (inside the sliding
  window ``> a + d - window`` when one is set) -- an interval over the first ``T``
  rows, and
* the earlier members ``(a, 1..d)`` of its own rollout -- explicit keys among the
  rows after ``T``.

Queries whose anchor is padding see nothing.  This is the reference's
``create_peagle_mask_mod`` (src/speculators/models/peagle/attention.py:46-72)
without the ``[Q, KV]`` mask evaluation.
"""

from __future__ import annotations

import torch

from speculators_b200.models.eagle3.attention import causal_document_interval
from speculators_b200.ops import AttnSpec

__all__ = ["dense_peagle_mask", "peagle_attn_spec"]


def peagle_attn_spec(anchor_pos, depth, document_ids, num_depths: int, sliding_window: int | None = None,
                     row_valid: torch.Tensor | None = None) -> AttnSpec:
    """``row_valid`` (bool ``[n]``, optional): rows marked False (padding of the
    fixed-shape sampler) see nothing and are nobody's key."""
    doc = document_ids.reshape(-1)
    T = doc.shape[0]
    n = anchor_pos.shape[0]
    device = doc.device
    doc_lo, _ = causal_document_interval(doc, None)
    lo = doc_lo[anchor_pos].to(torch.int64)
    if sliding_window is not None:
        lo = torch.maximum(lo, anchor_pos + depth - int(sliding_window) + 1)
    hi = anchor_pos + 1
    pad = doc[anchor_pos] == -1
    if row_valid is not None:
        pad = pad | ~row_valid
    hi = torch.where(pad, torch.zeros_like(hi), hi)
    lo = torch.where(pad, torch.zeros_like(lo), lo)
    extra = None
    if num_depths > 1 and n > T:
        # row index (relative to T) of every existing (anchor, depth >= 1) sample
        table = torch.full((num_depths, T), -1, dtype=torch.int32, device=device)
        rows = torch.arange(n, device=device)
        deep = depth >= 1
        if row_valid is None:
            table[depth[deep], anchor_pos[deep]] = (rows[deep] - T).to(torch.int32)
        else:  # fixed shapes: scatter every row, invalid ones into a spare column
            col = torch.where(deep & row_valid, anchor_pos, torch.full_like(anchor_pos, T))
            wide = torch.full((num_depths, T + 1), -1, dtype=torch.int32, device=device)
            wide[depth, col] = (rows - T).to(torch.int32)
            table = wide[:, :T]
        cols = []
        for d in range(1, num_depths):
            cand = table[d][anchor_pos]
            cols.append(torch.where((depth >= d) & ~pad, cand, torch.full_like(cand, -1)))
        extra = torch.stack(cols, dim=1).contiguous()
    return AttnSpec(lo=lo.to(torch.int32), hi=hi.to(torch.int32), extra_idx=extra)


def dense_peagle_mask(anchor_pos, depth, document_ids, sliding_window: int | None = None) -> torch.Tensor:
    """The mask written directly from its definition, ``[n, n]`` (tests)."""
    doc = document_ids.reshape(-1)
    qa, ka = anchor_pos[:, None], anchor_pos[None, :]
    qd, kd = depth[:, None], depth[None, :]
    ok = (doc[qa] == doc[ka]) & (doc[qa] != -1)
    window = (ka > qa + qd - sliding_window) if sliding_window is not None else torch.ones_like(ok)
    return ok & (((kd == 0) & (qa >= ka) & window) | ((qa == ka) & (qd >= kd)))
