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

__all__ = ["anchor_block_attn_spec", "create_anchor_block_mask_mod", "dense_anchor_block_mask"]


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
    return AttnSpec(lo=lo.to(torch.int32), hi=hi.to(torch.int32), extra_idx=extra.contiguous(), extra_block=int(block_size),
                    extra_block_causal=bool(causal_in_block))


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


def create_anchor_block_mask_mod(document_ids: torch.Tensor, total_seq_len: int, anchor_positions: torch.Tensor, block_size: int,
                                 sliding_window: int | None = None, sliding_window_non_causal: bool = False):
    """Element-level form of the anchored-block mask in the ``mask_mod(b, h, q_idx, kv_idx)``
    convention of ``torch.nn.attention.flex_attention``; returns ``(mask_mod, q_len, kv_len)``
    with ``q_len = n_anchors * block_size`` and ``kv_len = total_seq_len + q_len`` (the packed
    sequence followed by the synthetic blocks).  Same rule as ``dense_anchor_block_mask`` /
    ``anchor_block_attn_spec``: block ``j`` sees the keys of its anchor's document before the
    anchor (inside the window, if any) and its own block - all of it, or only earlier slots
    when a window is set and ``sliding_window_non_causal`` is off
    (src/speculators/models/dflash/attention.py:7-107)."""
    if anchor_positions.ndim != 1:
        raise ValueError(f"anchor_positions must be 1D, got shape {tuple(anchor_positions.shape)}")
    anchors = anchor_positions.to(device=document_ids.device, dtype=torch.long)
    q_len = anchors.numel() * block_size
    anchor_of_query = anchors.repeat_interleave(block_size)
    causal_in_block = sliding_window is not None and not sliding_window_non_causal

    def mask_mod(_b, _h, q_idx, kv_idx):
        anchor = anchor_of_query[q_idx]
        position = kv_idx % total_seq_len
        in_sequence = kv_idx < total_seq_len
        same_doc = (document_ids[anchor] == document_ids[position]) & (document_ids[anchor] != -1)
        prefix = in_sequence & same_doc & (position < anchor)
        if sliding_window is not None:
            prefix = prefix & (position >= anchor - sliding_window)
        own_block = (~in_sequence if isinstance(in_sequence, torch.Tensor) else not in_sequence) & (
            q_idx // block_size == (kv_idx - total_seq_len) // block_size)
        if causal_in_block:
            own_block = own_block & (kv_idx <= q_idx + total_seq_len)
        return prefix | own_block

    return mask_mod, q_len, total_seq_len + q_len
