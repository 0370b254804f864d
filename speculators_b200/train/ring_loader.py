"""Trainer-side loader over an NVLink hidden-state ring: batches built on the device.

The reference's online path goes verifier -> store -> ``ArrowDataset.__getitem__`` -> CPU
collate -> pinned memory -> device (src/speculators/train/data.py:220-255, 344-393).  When the
verifier's GPUs write hidden states straight into a ring in the trainer GPU's memory
(``hs_connectors/nvlink.py``) none of that is needed: the popped sample already sits on the
training device, and the post-collate batch (EAGLE-3 / P-EAGLE pairing shift, padding to the
packed length, positions, document ids, loss mask) is a handful of device ops on it.  No host
copy of a hidden state is made at any point.

Payload convention of a ring sample: ``hidden_states`` ``[rows, (A + 1) * H]`` = the ``A``
auxiliary layers concatenated, then the last layer's output; ``token_ids`` ``[rows]``.
"""

from __future__ import annotations

import torch

__all__ = ["RingBatchLoader", "batch_from_ring_sample"]


def batch_from_ring_sample(sample: dict, hidden_size: int, seq_len: int, loss_mask: torch.Tensor | None = None,
                           lengths: list[int] | None = None) -> dict:
    """One post-collate batch (``[1, seq_len, ...]``, fixed shapes) from one ring sample, on the
    sample's device.  Applies the EAGLE-3 pairing per document (hidden state of token ``t - 1`` with
    token ``t``: drop each document's last hidden state and first token, positions start at 1), keeps
    at most ``seq_len`` rows and pads the rest (document id -1, mask 0).

    ``lengths``: the token counts of the documents packed in the sample, in order (default: the whole
    sample is one document); ``loss_mask``: per-token mask of the sample, shifted like the ids.  The
    result equals what ``CollateFn`` with ``shift_batch`` builds from the documents' file samples."""
    hs, ids = sample["hidden_states"], sample["token_ids"].long()
    rows = hs.shape[0]
    width = hs.shape[1]
    aux_w = width - hidden_size
    dev = hs.device
    # row t of the batch reads hidden state src[t] and token / target / mask src[t] + 1 (indices built on the host: a few KB)
    src_parts, pos_parts, doc_parts, start, room = [], [], [], 0, seq_len
    for d, length in enumerate(lengths if lengths is not None else [rows]):
        keep = min(max(0, min(int(length), rows - start) - 1), room)
        if keep > 0:
            src_parts.append(torch.arange(start, start + keep))
            pos_parts.append(torch.arange(1, keep + 1))
            doc_parts.append(torch.full((keep,), d, dtype=torch.long))
        room -= keep
        start += int(length)
        if room <= 0 or start >= rows:
            break
    n = seq_len - room
    out_hs = torch.zeros(seq_len, aux_w, dtype=hs.dtype, device=dev)
    out_last = torch.zeros(seq_len, hidden_size, dtype=hs.dtype, device=dev)
    out_ids = torch.zeros(seq_len, dtype=torch.long, device=dev)
    mask = torch.zeros(seq_len, dtype=torch.bool, device=dev)
    position = torch.zeros(seq_len, dtype=torch.long, device=dev)
    document = torch.full((seq_len,), -1, dtype=torch.long, device=dev)
    if n > 0:
        src = torch.cat(src_parts).to(dev)
        out_hs[:n] = hs.index_select(0, src)[:, :aux_w]        # states of each document's tokens 0 .. len-2
        out_last[:n] = hs.index_select(0, src + 1)[:, aux_w:]  # verifier output at tokens 1 .. len-1
        out_ids[:n] = ids.index_select(0, src + 1)
        mask[:n] = True if loss_mask is None else loss_mask.to(dev).reshape(-1).index_select(0, src + 1).bool()
        position[:n] = torch.cat(pos_parts).to(dev)
        document[:n] = torch.cat(doc_parts).to(dev)
    return {
        "hidden_states": out_hs.unsqueeze(0), "input_ids": out_ids.unsqueeze(0), "verifier_last_hidden_states": out_last.unsqueeze(0),
        "loss_mask": mask.unsqueeze(0), "position_ids": position.unsqueeze(0), "document_ids": document.unsqueeze(0),
    }


class RingBatchLoader:
    """Loader-shaped (``__len__``, ``__iter__``, ``batch_sampler.set_epoch``): step ``i`` pops
    sample ``first_seq + i`` from ``ring`` and yields its batch.  ``mask_fn(token_ids) -> bool
    [rows]`` supplies the loss mask of a sample (default: every position)."""

    class _Sampler:
        def set_epoch(self, _epoch: int) -> None:
            pass

    def __init__(self, ring, num_steps: int, hidden_size: int, seq_len: int, first_seq: int = 1, timeout_s: float = 60.0, mask_fn=None,
                 meta_fn=None):
        """``meta_fn(i) -> (loss_mask [rows] or None, lengths or None)`` for the ``i``-th sample this loader pops
        (counted from 0 over its whole life): the per-token mask and the document lengths of a packed row, known
        to the trainer from the dataset; takes precedence over ``mask_fn``."""
        self.ring, self.num_steps, self.hidden_size, self.seq_len = ring, int(num_steps), int(hidden_size), int(seq_len)
        self.next_seq, self.timeout_s, self.mask_fn, self.meta_fn = int(first_seq), float(timeout_s), mask_fn, meta_fn
        self.popped = 0
        self.batch_sampler = self._Sampler()

    def __len__(self) -> int:
        return self.num_steps

    def next_batch(self) -> dict:
        sample = self.ring.pop(self.next_seq, self.timeout_s)
        self.next_seq += 1
        lengths = None
        if self.meta_fn is not None:
            mask, lengths = self.meta_fn(self.popped)
        else:
            mask = self.mask_fn(sample["token_ids"]) if self.mask_fn is not None else None
        self.popped += 1
        return batch_from_ring_sample(sample, self.hidden_size, self.seq_len, mask, lengths)

    def __iter__(self):
        for _ in range(self.num_steps):
            yield self.next_batch()
