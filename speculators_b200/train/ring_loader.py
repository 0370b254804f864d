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


def batch_from_ring_sample(sample: dict, hidden_size: int, seq_len: int, loss_mask: torch.Tensor | None = None) -> dict:
    """One post-collate batch (``[1, seq_len, ...]``, fixed shapes) from one ring sample, on the
    sample's device.  Applies the EAGLE-3 pairing (hidden state of token ``t - 1`` with token
    ``t``: drop the last hidden state and the first token, positions start at 1), keeps at most
    ``seq_len`` rows and pads the rest (document id -1, mask 0)."""
    hs, ids = sample["hidden_states"], sample["token_ids"].long()
    rows = hs.shape[0]
    width = hs.shape[1]
    aux_w = width - hidden_size
    n = max(0, min(rows - 1, seq_len))
    dev = hs.device
    out_hs = torch.zeros(seq_len, aux_w, dtype=hs.dtype, device=dev)
    out_last = torch.zeros(seq_len, hidden_size, dtype=hs.dtype, device=dev)
    out_ids = torch.zeros(seq_len, dtype=torch.long, device=dev)
    out_hs[:n] = hs[:n, :aux_w]            # states of tokens 0 .. n-1
    out_last[:n] = hs[1 : n + 1, aux_w:]   # verifier output at tokens 1 .. n
    out_ids[:n] = ids[1 : n + 1]
    idx = torch.arange(seq_len, device=dev)
    real = idx < n
    mask = real
    if loss_mask is not None:  # per-token mask of the sample: shifted like the ids
        shifted = torch.zeros(seq_len, dtype=torch.bool, device=dev)
        shifted[:n] = loss_mask.to(dev).reshape(-1)[1 : n + 1].bool()
        mask = shifted & real
    return {
        "hidden_states": out_hs.unsqueeze(0), "input_ids": out_ids.unsqueeze(0), "verifier_last_hidden_states": out_last.unsqueeze(0),
        "loss_mask": mask.unsqueeze(0), "position_ids": torch.where(real, idx + 1, torch.zeros_like(idx)).unsqueeze(0),
        "document_ids": torch.where(real, torch.zeros_like(idx), torch.full_like(idx, -1)).unsqueeze(0),
    }


class RingBatchLoader:
    """Loader-shaped (``__len__``, ``__iter__``, ``batch_sampler.set_epoch``): step ``i`` pops
    sample ``first_seq + i`` from ``ring`` and yields its batch.  ``mask_fn(token_ids) -> bool
    [rows]`` supplies the loss mask of a sample (default: every position)."""

    class _Sampler:
        def set_epoch(self, _epoch: int) -> None:
            pass

    def __init__(self, ring, num_steps: int, hidden_size: int, seq_len: int, first_seq: int = 1, timeout_s: float = 60.0, mask_fn=None):
        self.ring, self.num_steps, self.hidden_size, self.seq_len = ring, int(num_steps), int(hidden_size), int(seq_len)
        self.next_seq, self.timeout_s, self.mask_fn = int(first_seq), float(timeout_s), mask_fn
        self.batch_sampler = self._Sampler()

    def __len__(self) -> int:
        return self.num_steps

    def next_batch(self) -> dict:
        sample = self.ring.pop(self.next_seq, self.timeout_s)
        self.next_seq += 1
        mask = self.mask_fn(sample["token_ids"]) if self.mask_fn is not None else None
        return batch_from_ring_sample(sample, self.hidden_size, self.seq_len, mask)

    def __iter__(self):
        for _ in range(self.num_steps):
            yield self.next_batch()
