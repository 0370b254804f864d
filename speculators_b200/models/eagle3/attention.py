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

__all__ = [
    "block_mask_to_dense_attention_mask", "causal_document_interval", "create_combined_mask_mod", "dense_ttt_mask",
    "extend_dense_mask_for_draft_tokens", "extend_mask_for_draft_tokens", "ttt_attn_spec",
]


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


def create_combined_mask_mod(document_ids: torch.Tensor, total_seq_len: int, sliding_window: int | None = None):
    """Element-level form of the training-time-test mask, in the ``mask_mod(b, h, q_idx,
    kv_idx)`` convention of ``torch.nn.attention.flex_attention`` (usable with its
    ``create_mask`` / ``create_block_mask``, or as an oracle for ``ttt_attn_spec``).  Keys
    ``kv_idx >= total_seq_len`` are the appended draft passes: pass ``p`` holds position
    ``kv_idx - p * total_seq_len``.  A query sees the causal (optionally windowed) keys of
    its own document - padding rows (document -1) see none - plus, in every pass, the key
    at its own position (src/speculators/models/eagle3/attention.py:11-34)."""

    def mask_mod(_b, _h, q_idx, kv_idx):
        position = kv_idx % total_seq_len
        in_document = (document_ids[q_idx] != -1) & (document_ids[q_idx] == document_ids[position])
        causal = q_idx >= kv_idx
        if sliding_window is not None:
            causal = causal & (kv_idx > q_idx - sliding_window)
        return (causal & in_document) | (position == q_idx)

    return mask_mod


def extend_dense_mask_for_draft_tokens(mask: torch.Tensor, total_seq_len: int) -> torch.Tensor:
    """Append the key columns of one more training-time-test pass to a dense mask
    ``[..., total_seq_len, kv_len]``: query ``q`` sees exactly the new key ``q``.  Boolean
    masks get an identity block; additive float masks get 0 on the diagonal and ``-inf``
    elsewhere, so that the new block means the same in both conventions
    (src/speculators/models/eagle3/attention.py:115-132 appends the 0/1 identity in the
    mask's dtype, which for an additive mask admits every new key)."""
    eye = torch.eye(total_seq_len, dtype=torch.bool, device=mask.device)
    if mask.dtype == torch.bool:
        block = eye
    else:
        block = torch.zeros(total_seq_len, total_seq_len, dtype=mask.dtype, device=mask.device).masked_fill(~eye, float("-inf"))
    block = block.reshape((1,) * (mask.dim() - 2) + block.shape).expand(*mask.shape[:-2], total_seq_len, total_seq_len)
    return torch.cat([mask, block], dim=-1)


# ---- interoperability with torch's flex-attention block masks ---------------------------------
# The package's own attention does not use block masks; these two helpers exist for code that
# drives ``torch.nn.attention.flex_attention`` with the same training-time-test pattern
# (src/speculators/models/eagle3/attention.py:37-112, :135-148).
def extend_mask_for_draft_tokens(block_mask):
    """A ``BlockMask`` whose key axis is one training-time-test pass longer: query block ``i``
    additionally sees the new key block ``i`` (the ``mask_mod`` decides which elements inside;
    with ``create_combined_mask_mod`` only the diagonal).  Requires square blocks and a query
    axis of the original sequence length; the ``mask_mod`` is kept."""
    from torch.nn.attention.flex_attention import BlockMask

    q_block, kv_block = block_mask.BLOCK_SIZE
    if q_block != kv_block:
        raise ValueError(f"square blocks expected, got {block_mask.BLOCK_SIZE}")
    q_len, kv_len = block_mask.seq_lengths
    counts, indices = block_mask.kv_num_blocks, block_mask.kv_indices
    n_q_blocks = counts.shape[-1]
    n_kv_blocks = -(-kv_len // kv_block)
    width = n_kv_blocks + n_q_blocks

    def widen(table):
        grown = table.new_full((*table.shape[:-1], width), -1)
        grown[..., : table.shape[-1]] = table
        return grown

    new_indices = widen(indices)
    appended = torch.arange(n_kv_blocks, width, device=indices.device, dtype=indices.dtype).expand(counts.shape)
    new_indices.scatter_(-1, counts.long().unsqueeze(-1), appended.unsqueeze(-1))  # first free column of each row
    full_counts, full_indices = block_mask.full_kv_num_blocks, block_mask.full_kv_indices
    return BlockMask.from_kv_blocks(
        kv_num_blocks=counts + 1, kv_indices=new_indices,
        full_kv_num_blocks=full_counts, full_kv_indices=None if full_indices is None else widen(full_indices),
        BLOCK_SIZE=block_mask.BLOCK_SIZE, mask_mod=block_mask.mask_mod, seq_lengths=(q_len, kv_len + n_q_blocks * kv_block),
    )


def block_mask_to_dense_attention_mask(block_mask, device: torch.device, dtype: torch.dtype) -> torch.Tensor:
    """Element mask ``[B, H, q_len, kv_len]`` of a ``BlockMask`` (1 = attend) from its
    ``mask_mod``, evaluated for all pairs at once."""
    batch, heads, q_len, kv_len = block_mask.shape
    b = torch.arange(batch, device=device).view(-1, 1, 1, 1)
    h = torch.arange(heads, device=device).view(1, -1, 1, 1)
    q = torch.arange(q_len, device=device).view(1, 1, -1, 1)
    kv = torch.arange(kv_len, device=device).view(1, 1, 1, -1)
    allowed = block_mask.mask_mod(b, h, q, kv)
    return torch.as_tensor(allowed, device=device).expand(batch, heads, q_len, kv_len).to(dtype)
