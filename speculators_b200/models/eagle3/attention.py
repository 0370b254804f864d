"""EAGLE-3 attention pattern as an ``AttnSpec``.

Training-time-test (TTT) runs the draft layer ``S`` times over the same ``T``
positions.  Pass ``s`` sees the keys of pass 0 under a causal, same-document
(optionally sliding-window) mask, and from every later pass ``1..s`` only the key
at its own position.  In the reference that is the ``mask_mod``
``(causal & window & same_doc & q_not_pad) | (kv % T == q)`` over a KV axis that
grows by ``T`` per pass (src/speculators/models/eagle3/attention.py:11-34, the
block-mask extension :37-112).  Here the first term is the interval
``[max(doc_start, q - window + 1), q]`` and the second a list of ``s`` explicit
keys; padded rows (document id -1) keep only their own position.

Document ids are expected as the collate function produces them: equal ids form
one contiguous run, padding is -1.
"""

from __future__ import annotations

import torch

from speculators_b200.ops import AttnSpec

__all__ = ["causal_document_interval", "dense_ttt_mask", "ttt_attn_spec"]


def causal_document_interval(document_ids: torch.Tensor, sliding_window: int | None = None):
    """``(lo, hi)`` int32 [T]: allowed context keys of each query under causal +
    same-document (+ window) masking."""
    doc = document_ids.reshape(-1)
    T = doc.shape[0]
    idx = torch.arange(T, device=doc.device)
    new_run = torch.ones(T, dtype=torch.bool, device=doc.device)
    new_run[1:] = doc[1:] != doc[:-1]
    start = torch.cummax(torch.where(new_run, idx, torch.zeros_like(idx)), dim=0).values
    lo = start
    if sliding_window is not None:
        lo = torch.maximum(lo, idx - int(sliding_window) + 1)
    lo = torch.where(doc == -1, idx, lo)
    return lo.to(torch.int32), (idx + 1).to(torch.int32)


def ttt_attn_spec(document_ids: torch.Tensor, ttt_step: int, sliding_window: int | None = None, interval=None) -> AttnSpec:
    lo, hi = interval if interval is not None else causal_document_interval(document_ids, sliding_window)
    T = lo.shape[0]
    extra = None
    if ttt_step > 0:
        idx = torch.arange(T, device=lo.device, dtype=torch.int32)
        extra = torch.stack([idx + j * T for j in range(ttt_step)], dim=1).contiguous()
    return AttnSpec(lo=lo, hi=hi, extra_idx=extra)


def dense_ttt_mask(document_ids: torch.Tensor, ttt_step: int, sliding_window: int | None = None) -> torch.Tensor:
    """The same pattern written directly from its definition as a boolean
    ``[T, (ttt_step + 1) * T]`` matrix (used by tests to pin ``ttt_attn_spec``)."""
    doc = document_ids.reshape(-1)
    T = doc.shape[0]
    q = torch.arange(T, device=doc.device)[:, None]
    kv = torch.arange((ttt_step + 1) * T, device=doc.device)[None, :]
    causal = q >= kv
    if sliding_window is not None:
        causal = causal & (kv > q - sliding_window)
    same_doc = (doc[q] != -1) & (doc[q] == doc[kv % T])
    return (causal & same_doc) | (kv % T == q)
