"""Multipack batch sampler: packs variable-length samples into per-rank batches
of at most ``batch_max_length`` tokens, with every data-parallel rank receiving
the same number of batches per epoch.

Algorithm (same as the reference's ``MultipackDistributedBatchSamplerV2``,
src/speculators/train/distributed_batch_sampler.py:47-250, so a given seed yields
the same assignment): shuffle with ``default_rng(seed + epoch)``; repeatedly take
the longest prefix of the remaining samples that longest-processing-time-first
(LPT) scheduling can fit into ``num_replicas`` bins of ``batch_max_length`` tokens
(binary search on the prefix length, bounded by the token budget); bin ``s`` of
the ``b``-th group goes to rank ``(s + b) % num_replicas`` so that the rank which
gets the largest sample rotates.  Leftover samples (< ``num_replicas``) are
dropped.  Over-long samples are truncated (default) or dropped.
"""

from __future__ import annotations

import heapq
import warnings

import numpy as np
from torch.utils.data import Sampler

__all__ = ["MultipackDistributedBatchSamplerV2", "lpt_bins"]


def lpt_bins(lengths: np.ndarray, max_len: int, num_bins: int) -> list[list[int]] | None:
    """LPT packing of ``lengths`` into ``num_bins`` bins; ``None`` if some bin would
    exceed ``max_len``.  Returns local indices per bin.  Ties between equally
    filled bins break on the lower bin id."""
    bins: list[list[int]] = [[] for _ in range(num_bins)]
    heap = [(0, slot) for slot in range(num_bins)]
    for idx in np.argsort(lengths)[::-1]:
        fill, slot = heap[0]
        new_fill = fill + int(lengths[idx])
        if new_fill > max_len:
            return None
        bins[slot].append(int(idx))
        heapq.heapreplace(heap, (new_fill, slot))
    return bins


def _pack_for_rank(lengths: np.ndarray, max_len: int, rank: int, replicas: int) -> list[list[int]]:
    csum = np.cumsum(lengths)
    out: list[list[int]] = []
    pos, consumed = 0, 0
    while len(lengths) - pos >= replicas:
        lo = 1
        hi = 1 + int(np.searchsorted(csum[pos:], consumed + max_len * replicas, "right"))
        slot = (rank - len(out)) % replicas
        best = None
        while hi - lo > 1 and hi > replicas:
            mid = (lo + hi) // 2
            bins = lpt_bins(lengths[pos : pos + mid], max_len, replicas)
            if bins is None:
                hi = mid
                best = None
            else:
                lo = mid
                best = bins
        if best is None:
            best = lpt_bins(lengths[pos : pos + lo], max_len, replicas)
        out.append([pos + i for i in best[slot]] if best is not None else None)
        pos += lo
        consumed = csum[pos - 1]
    return out


class MultipackDistributedBatchSamplerV2(Sampler):
    def __init__(self, batch_max_length: int, lengths, num_replicas: int, rank: int, truncate_long_samples: bool = True, seed: int = 0):
        self.num_replicas, self.rank, self.seed, self.epoch = num_replicas, rank, seed, 0
        self.batch_max_length = batch_max_length
        self.lengths = np.array(lengths)
        self.valid_indices = np.nonzero(self.lengths <= batch_max_length)[0]
        too_long = len(self.lengths) - len(self.valid_indices)
        if too_long:
            if truncate_long_samples:
                msg = (f"Found {too_long}/{len(self.lengths)} samples longer than batch_max_length. "
                       "These samples will be truncated to batch_max_length.")
                self.valid_indices = np.arange(len(self.lengths))
                self.lengths = np.clip(self.lengths, 0, batch_max_length)
            else:
                msg = (f"Dropping {too_long}/{len(self.lengths)} samples longer than batch_max_length. Ensure that "
                       "the right max_batch_length is used during data processing.")
            if rank == 0:
                warnings.warn(msg, stacklevel=1)
        self._cached_generated_batches: tuple[int, list] = (-1, [])

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch

    def _generate_batches(self, epoch: int) -> list:
        if self._cached_generated_batches[0] == epoch:
            return self._cached_generated_batches[1]
        order = np.random.default_rng(seed=self.seed + epoch).permutation(self.valid_indices)
        packed = _pack_for_rank(self.lengths[order], self.batch_max_length, self.rank, self.num_replicas)
        batches = [order[np.asarray(b, dtype=np.int64)] for b in packed]
        self._cached_generated_batches = (epoch, batches)
        return batches

    def __iter__(self):
        return iter(self._generate_batches(self.epoch))

    def __len__(self) -> int:
        return len(self._generate_batches(self.epoch))
