"""Online training on one machine split between verifier GPUs and trainer GPUs.

The reference's online mode is a vLLM server on some GPUs (tensor parallel), the trainer on the
others, and hidden states travelling server -> store -> trainer dataloader -> CPU collate -> GPU
(scripts/launch_vllm.py:104-163; src/speculators/train/data.py:220-255;
docs/user_guide/tutorials/train.md:165-170).  ``OnlineSplit`` is the single-job counterpart: the
first half of the ranks run the verifier tensor-parallel (``TensorParallelVerifier``), the second
half train the draft (sharded optimizer among themselves); after every verifier forward one
verifier rank pushes the auxiliary + last hidden states of a sequence straight into the ring of
the trainer rank it is meant for (NVLink peer stores, ``hs_connectors/nvlink.py``), and the
trainer builds its batch from the ring slot on its own device (``RingBatchLoader``).  No hidden
state touches host memory.

Flow control is the ring itself: the verifier runs at most ``n_slots`` samples ahead of a
trainer; both sides wait with a bound (``timeout_s``) and raise on expiry.

Two sources of work: seeded random sequences through a random-init verifier (benchmarks), or the
packed rows of a preprocessed dataset (``OnlineBatchPlan``: every rank derives the same multipack
schedule, so the verifier ranks know which row to run for which trainer and the trainer ranks know
its loss mask and document lengths) through a verifier loaded from a checkpoint (``verifier_path``);
``serve`` / ``training_loader`` are the two halves of such a run (``train/entrypoint.py``,
``--online-verifier-gpus``).
"""

from __future__ import annotations

import time
from dataclasses import dataclass

import torch
import torch.distributed as dist

from speculators_b200.hs_connectors.nvlink import HiddenStateRing, HiddenStateRingWriter
from speculators_b200.train.ring_loader import RingBatchLoader
from speculators_b200.verifier.tp import TensorParallelVerifier

__all__ = ["OnlineSplit", "SplitTopology"]


@dataclass
class SplitTopology:
    world: int
    rank: int
    n_verifier: int

    @property
    def n_trainer(self) -> int:
        return self.world - self.n_verifier

    @property
    def is_verifier(self) -> bool:
        return self.rank < self.n_verifier

    @property
    def trainer_index(self) -> int:
        return self.rank - self.n_verifier

    def pusher_of(self, trainer_index: int) -> int:
        """Verifier rank that pushes the samples of trainer ``trainer_index`` (every verifier rank holds
        the complete hidden states after the tensor-parallel forward; the pushes are spread over them)."""
        return trainer_index % self.n_verifier


class OnlineSplit:
    def __init__(self, verifier_config: dict, aux_layers: list[int], seq_len: int, device: torch.device, *, n_verifier: int | None = None,
                 n_slots: int = 4, timeout_s: float = 120.0, seed: int = 0, resident: bool = True, sliced_init: bool = True,
                 sample_tokens: int | None = None, verifier_comm: str | None = None, verifier_path: str | None = None, plan=None,
                 transform=None):
        """``sample_tokens``: length of the sequences the verifier runs (default ``seq_len + 1``: the pairing
        shift consumes one token, so the trainer's ``seq_len`` positions are all real; ``seq_len`` keeps the
        verifier's row count a multiple of the GEMM tile and leaves the trainer one masked position).
        ``verifier_comm``: see ``TensorParallelVerifier`` (``None``: fused peer-memory exchange where possible).
        ``verifier_path``: checkpoint directory to load the verifier from (default: random-init from ``seed``).
        ``plan``: an ``OnlineBatchPlan`` (rows of a dataset) instead of seeded random sequences; samples are then
        packed rows of up to ``seq_len`` tokens.  ``transform``: applied to every trainer batch (noise)."""
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() < 2:
            raise RuntimeError("OnlineSplit needs at least two ranks (one verifier, one trainer)")
        world, rank = dist.get_world_size(), dist.get_rank()
        self.topo = SplitTopology(world, rank, n_verifier if n_verifier is not None else world // 2)
        t = self.topo
        self.device, self.seq_len, self.aux_layers, self.timeout_s, self.seed = device, int(seq_len), list(aux_layers), timeout_s, seed
        self.plan, self.transform = plan, transform
        self.sample_tokens = int(sample_tokens) if sample_tokens is not None else (self.seq_len if plan is not None else self.seq_len + 1)
        self.hidden = int(verifier_config["hidden_size"])
        self.vocab = int(verifier_config["vocab_size"])
        # both groups are created by every rank (a collective of the whole job)
        self.verifier_group = dist.new_group(list(range(t.n_verifier)))
        self.trainer_group = dist.new_group(list(range(t.n_verifier, world)))
        width = (len(self.aux_layers) + 1) * self.hidden
        self.ring = HiddenStateRing(n_slots, self.sample_tokens, width, device) if not t.is_verifier else None
        described: list = [None] * world
        dist.all_gather_object(described, self.ring.describe() if self.ring is not None else None)
        self.writers: dict[int, HiddenStateRingWriter] = {}
        self.verifier = None
        if t.is_verifier:
            for ti in range(t.n_trainer):
                if t.pusher_of(ti) == rank:
                    self.writers[ti] = HiddenStateRingWriter(described[t.n_verifier + ti], device)
            dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
            if verifier_path is not None:
                self.verifier = TensorParallelVerifier.from_pretrained(verifier_path, group=self.verifier_group, device=device, dtype=dtype,
                                                                       max_tokens=self.sample_tokens, comm=verifier_comm)
            else:
                self.verifier = TensorParallelVerifier(verifier_config, group=self.verifier_group, seed=seed, device=device, dtype=dtype,
                                                       resident=resident, sliced_init=sliced_init, max_tokens=self.sample_tokens, comm=verifier_comm)
        self._seq = 0
        self._loader: RingBatchLoader | None = None  # one per trainer rank for the whole job: sequence numbers run on across ``run`` calls

    # ------------------------------------------------------------------ data
    def tokens(self, step: int, trainer_index: int) -> torch.Tensor:
        """The sequence trainer ``trainer_index`` trains on at ``step`` (seeded, ``sample_tokens`` long)."""
        gen = torch.Generator().manual_seed(self.seed * 1_000_003 + step * 1009 + trainer_index)
        return torch.randint(0, self.vocab, (self.sample_tokens,), generator=gen)

    # ------------------------------------------------------------------ verifier side
    def verifier_step(self, step: int) -> None:
        """Forward of one sequence per trainer rank; the responsible rank pushes each into its ring."""
        t = self.topo
        self._seq += 1
        for ti in range(t.n_trainer):
            if self.plan is not None:
                row = self.plan.row(step, ti)
                ids = row["input_ids"].to(self.device)
                doc, pos = row["document_ids"], row["position_ids"]
            else:
                ids, doc, pos = self.tokens(step, ti).to(self.device), None, None
            if ids.numel() > 0:
                out = self.verifier.forward(ids, self.aux_layers, document_ids=doc, position_ids=pos)
                payload = torch.cat([out["hidden_states"], out["verifier_last_hidden_states"]], dim=-1)
            else:  # an empty row still takes its place in the sequence
                payload = torch.zeros(0, (len(self.aux_layers) + 1) * self.hidden, dtype=torch.bfloat16, device=self.device)
            if ti in self.writers:
                self.writers[ti].push(self._seq, payload, ids.to(torch.int32), timeout_s=self.timeout_s, check=False)

    def check_verifier(self) -> None:
        for w in self.writers.values():
            w.check_status()
        if self.verifier is not None and self.verifier.comm is not None:
            self.verifier.comm.check_status()

    # ------------------------------------------------------------------ trainer side
    def loader(self, num_steps: int) -> RingBatchLoader:
        return RingBatchLoader(self.ring, num_steps, self.hidden, self.seq_len, first_seq=1, timeout_s=self.timeout_s)

    # ------------------------------------------------------------------ a training run over a dataset plan
    def serve(self, first_epoch: int, num_epochs: int, max_steps: int | None = None) -> int:
        """Verifier ranks: run the rows of epochs ``first_epoch .. num_epochs - 1`` in the order the trainer ranks
        pop them (at most ``max_steps`` of them); returns the number of steps served."""
        served = 0
        for epoch in range(first_epoch, num_epochs):
            self.plan.set_epoch(epoch)
            for step in range(self.plan.steps_per_epoch):
                if max_steps is not None and served >= max_steps:
                    break
                self.verifier_step(step)
                served += 1
            self.check_verifier()
        return served

    def training_loader(self):
        """Trainer ranks: the loader ``Trainer`` iterates, one epoch of the plan per pass (``len`` = steps per
        epoch, ``batch_sampler.set_epoch`` moves the plan on)."""
        split = self

        class _PlanLoader(RingBatchLoader):
            class _Sampler:
                def set_epoch(self, epoch: int) -> None:
                    split.plan.set_epoch(epoch)
                    split._epoch_step = 0  # noqa: SLF001

            def __len__(self) -> int:
                return split.plan.steps_per_epoch

            def __iter__(self):
                for _ in range(len(self)):
                    yield self.next_batch()

        def meta(_popped: int):
            row = split.plan.row(split._epoch_step, split.topo.trainer_index)  # noqa: SLF001
            split._epoch_step += 1  # noqa: SLF001
            return row["loss_mask"], row["lengths"]

        self._epoch_step = 0
        loader = _PlanLoader(self.ring, self.plan.steps_per_epoch, self.hidden, self.seq_len, first_seq=1, timeout_s=self.timeout_s, meta_fn=meta)
        if self.transform is not None:
            build = loader.next_batch

            def with_transform():
                return self.transform(build())

            loader.next_batch = with_transform
        return loader

    # ------------------------------------------------------------------ a run of W + K steps
    def run(self, trainer_step, warmup: int, steps: int) -> float:
        """``trainer_step(batch)`` on trainer ranks; returns the K timed steps' milliseconds (max over all
        ranks: verifier and trainer halves overlap, the slower one sets the pace)."""
        cuda = self.device.type == "cuda"
        if self._loader is None and not self.topo.is_verifier:
            self._loader = self.loader(2**31)
        loader = self._loader

        def one(step):
            if self.topo.is_verifier:
                self.verifier_step(step)
            else:
                trainer_step(loader.next_batch())

        for s in range(warmup):
            one(s)
        if cuda:
            torch.cuda.synchronize()
        dist.barrier()
        t0 = time.perf_counter()
        if cuda:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        for s in range(steps):
            one(warmup + s)
        if cuda:
            end.record()
            torch.cuda.synchronize()
            ms = start.elapsed_time(end)
        else:
            ms = (time.perf_counter() - t0) * 1000.0
        if self.topo.is_verifier:
            self.check_verifier()
        t = torch.tensor([ms], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def close(self) -> None:
        if dist.is_initialized():
            if self.device.type == "cuda":
                torch.cuda.synchronize()
            dist.barrier()
        for w in self.writers.values():
            w.close()
        if self.ring is not None:
            self.ring.close()
        if self.verifier is not None and self.verifier.comm is not None:
            self.verifier.comm.check_status()
            self.verifier.comm.close()
