"""DFlash anchored-block attention as an ``AttnSpec``.

Queries are ``N * B`` noise tokens (block ``j`` belongs to anchor ``a_j``); keys
are the ``T`` projected verifier states followed by the noise tokens.  A query of
block ``j`` sees base positions ``< a_j`` of the anchor's document (``>= a_j -
window`` on sliding layers) and the tokens of its own block -- all of them, or on
causal sliding layers only those at or before its own slot.  Reference:
``create_anchor_block_mask_mod`` (src/speculators/models/dflash/attention.py:7-100).
"""

from __future__ import annotations

import torch

from speculators_b200.models.eagle3.attention import causal_document_interval
from speculators_b200.ops import AttnSpec

__all__ = ["anchor_block_attn_spec", "dense_anchor_block_mask"]


def anchor_block_attn_spec(document_ids, anchor_positions, block_size: int, sliding_window: int | None = None,
                           sliding_window_non_causal: bool = False) -> AttnSpec:
    doc = document_ids.reshape(-1)
    device = doc.device
    a = anchor_positions.to(device=device, dtype=torch.long).reshape(-1)
    n = a.numel()
    qa = a.repeat_interleave(block_size)
    doc_lo, _ = causal_document_interval(doc, None)
    lo = doc_lo[qa].to(torch.int64)
    if sliding_window is not None:
        lo = torch.maximum(lo, qa - int(sliding_window))
    hi = qa.clone()
    pad = doc[qa] == -1
    hi = torch.where(pad, torch.zeros_like(hi), hi)
    lo = torch.where(pad, torch.zeros_like(lo), lo)
    slot = torch.arange(block_size, device=device)
    block = torch.arange(n, device=device).repeat_interleave(block_size)
    extra = (block[:, None] * block_size + slot[None, :]).to(torch.int32)
    causal_in_block = sliding_window is not None and not sliding_window_non_causal
    if causal_in_block:
        q_slot = slot.repeat(n)
        extra = torch.where(slot[None, :] <= q_slot[:, None], extra, torch.full_like(extra, -1))
    return AttnSpec(lo=lo.to(torch.int32), hi=hi.to(torch.int32), extra_idx=extra.contiguous())


def dense_anchor_block_mask(document_ids, total_seq_len: int, anchor_positions, block_size: int,
                            sliding_window: int | None = None, sliding_window_non_causal: bool = False) -> torch.Tensor:
    """Mask written from its definition, ``[N*B, T + N*B]`` (tests)."""
    doc = document_ids.reshape(-1)
    a = anchor_positions.reshape(-1).long()
    q_len = a.numel() * block_size
    q = torch.arange(q_len, device=doc.device)[:, None]
    kv = torch.arange(total_seq_len + q_len, device=doc.device)[None, :]
    q_anchor = a.repeat_interleave(block_size)[:, None]
    base = kv % total_seq_len
    is_base = kv < total_seq_len
    same_doc = (doc[q_anchor] == doc[base]) & (doc[q_anchor] != -1)
    window = (base >= q_anchor - sliding_window) if sliding_window is not None else torch.ones_like(same_doc)
    prefix = is_base & same_doc & (base < q_anchor) & window
    same_block = (~is_base) & (q // block_size == (kv - total_seq_len) // block_size)
    if sliding_window is not None and not sliding_window_non_causal:
        same_block = same_block & (kv <= q + total_seq_len)
    return prefix | same_block
