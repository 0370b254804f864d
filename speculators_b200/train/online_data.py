"""Which dataset rows every trainer rank trains on at every step of an online run.

In the reference's online mode a trainer worker asks the verifier server for the hidden states of
the rows its sampler handed it (src/speculators/train/data.py:220-255).  With the verifier inside
the job (``train/online.py``) nobody asks: every rank derives the same plan from the preprocessed
dataset and the seed - the multipack sampler of each trainer rank, epoch by epoch - so the
verifier ranks know which packed row to run for which trainer at which step, and a trainer rank
knows the loss mask and the document lengths of the row it is about to pop from its ring.
"""

from __future__ import annotations

from os import PathLike

import torch

from speculators_b200.train.data import RowWindow
from speculators_b200.train.distributed_batch_sampler import MultipackDistributedBatchSamplerV2

__all__ = ["OnlineBatchPlan"]


class OnlineBatchPlan:
    def __init__(self, datapath: str | PathLike, total_seq_len: int, n_trainer: int, seed: int = 0, train_ratio: float = 1.0,
                 split: str = "train"):
        from datasets import load_from_disk

        table = load_from_disk(str(datapath))
        self.window = RowWindow.of(len(table), train_ratio, split)
        self.data = table.select(range(self.window.start, self.window.stop)).with_format(None)
        self.total_seq_len, self.n_trainer = int(total_seq_len), int(n_trainer)
        lengths = [int(v) for v in self.data["seq_len"]]
        self.samplers = [MultipackDistributedBatchSamplerV2(self.total_seq_len, lengths, self.n_trainer, ti, seed=seed) for ti in range(self.n_trainer)]
        self._batches: list[list[list[int]]] = []
        self.epoch = -1
        self.set_epoch(0)

    def set_epoch(self, epoch: int) -> None:
        if epoch == self.epoch:
            return
        self.epoch = int(epoch)
        for sampler in self.samplers:
            sampler.set_epoch(self.epoch)
        self._batches = [[list(map(int, b)) for b in sampler] for sampler in self.samplers]

    @property
    def steps_per_epoch(self) -> int:
        return min(len(b) for b in self._batches)

    def row(self, step: int, trainer_index: int) -> dict:
        """The packed row trainer ``trainer_index`` trains on at ``step`` of the current epoch:
        ``input_ids`` / ``loss_mask`` / ``document_ids`` / ``position_ids`` (``[L]``, ``L <= total_seq_len``)
        and ``lengths`` (tokens per document; the document that crosses the limit is clipped)."""
        ids, mask, doc, pos, lengths = [], [], [], [], []
        room = self.total_seq_len
        for d, index in enumerate(self._batches[trainer_index][step]):
            sample = self.data[index]
            take = min(len(sample["input_ids"]), room)
            if take <= 0:
                break
            ids.append(torch.as_tensor(sample["input_ids"][:take], dtype=torch.long))
            mask.append(torch.as_tensor(sample["loss_mask"][:take]).bool())
            doc.append(torch.full((take,), d, dtype=torch.long))
            pos.append(torch.arange(take))
            lengths.append(take)
            room -= take
        if not ids:
            empty = torch.zeros(0, dtype=torch.long)
            return {"input_ids": empty, "loss_mask": empty.bool(), "document_ids": empty, "position_ids": empty, "lengths": []}
        return {"input_ids": torch.cat(ids), "loss_mask": torch.cat(mask), "document_ids": torch.cat(doc), "position_ids": torch.cat(pos),
                "lengths": lengths}
