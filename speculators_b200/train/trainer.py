"""Training loop.

Same contract as src/speculators/train/trainer.py (``Trainer(model,
TrainerConfig, train_loader, val_loader).run_training()``, one optimizer step per
packed batch, gradient clipping at 1.0, metric reduction every ``log_freq`` steps,
epoch / fractional-epoch checkpoints, mid-epoch resume, best-epoch tracking), with
a different execution model:

* mixed precision, data parallelism and the optimizer live in ``TrainEngine``
  (flat bf16 compute weights, fp32 master + AdamW/Muon state, one collective per
  step) instead of autocast + DDP/FSDP2 wrappers + ``torch.optim``;
* on a GPU the step (zero-grad, forward, backward and, single-process, the
  optimizer) is captured once per input signature into a CUDA graph and replayed;
  batches are copied into the graph's static inputs from pinned host memory;
* step timing uses CUDA events on the training stream (device time), not
  ``synchronize`` + ``perf_counter``.
"""

from __future__ import annotations

import json
import logging
import os
import time
import warnings
from pathlib import Path
from typing import Literal, NamedTuple

import torch
import torch.distributed as dist

from speculators_b200.model import SpeculatorModel
from speculators_b200.parallel.distributed import get_local_rank, get_rank, is_distributed, set_training_group, training_rank
from speculators_b200.parallel.engine import EngineConfig, TrainEngine
from speculators_b200.train.checkpointer import Checkpointer
from speculators_b200.train.graceful_shutdown import with_graceful_shutdown
from speculators_b200.train.schedule import LRSchedule, resolve_scheduler_steps
from speculators_b200.train.schedule import resolve_scheduler_steps as _resolve_scheduler_steps  # noqa: F401  (the reference's name)
from speculators_b200.utils.util import nvtx_range
from speculators_b200.train.utils import normalize_counted_metrics

root_logger = logging.getLogger("speculators")
metric_logger = logging.getLogger("speculators.metrics")

__all__ = ["LossHandle", "Trainer", "TrainerConfig"]

MIN_STEP_PCT = 0.25
_VAL_SYNC_INTERVAL = 50  # barrier every N validation batches to bound rank skew


class TrainerConfig(NamedTuple):
    lr: float
    num_epochs: int
    save_path: str
    resume_from_checkpoint: bool = False
    train_call_kwargs: dict | None = None
    val_call_kwargs: dict | None = None
    optimizer: Literal["adamw", "muon"] = "adamw"
    weight_decay: float = 0.01
    muon_lr: float = 0.02
    muon_momentum: float = 0.95
    muon_weight_decay: float = 0.1
    muon_ns_steps: int = 5
    muon_adjust_lr_fn: str = "match_rms_adamw"
    scheduler_type: Literal["linear", "cosine", "none"] = "linear"
    scheduler_warmup_steps: int | None = None
    scheduler_warmup_ratio: float | None = None
    scheduler_total_steps: int | None = None
    scheduler_num_cosine_cycles: float = 0.5
    checkpoint_freq: float = 1
    save_best: bool = False
    hidden_states_dtype: torch.dtype = torch.bfloat16
    log_freq: int = 1
    fsdp_shard: bool = False
    max_steps: int | None = None
    max_grad_norm: float = 1.0
    use_cuda_graph: bool | None = None  # None: on when training on a GPU
    device: str | None = None  # None: cuda:<local_rank> when available, else cpu
    process_group: object | None = None  # ranks that train together (None: all); e.g. the trainer half of a verifier / trainer split


class _StepTimer:
    """Phase marks of one training step.  On CUDA each mark records an event on the
    current stream (no synchronisation until ``profile`` is read); on CPU it reads
    ``perf_counter``.  Enabled only on steps that will be logged."""

    def __init__(self, enabled: bool = False, device_type: str = "cpu"):
        self.enabled = enabled
        self.cuda = device_type == "cuda"
        self._marks: dict[str, object] = {}

    def reset(self, enabled: bool) -> None:
        self.enabled = enabled
        self._marks.clear()

    def mark(self, name: str) -> None:
        if not self.enabled:
            return
        if self.cuda:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            self._marks[name] = ev
        else:
            self._marks[name] = time.perf_counter()

    def snapshot(self) -> "_StepTimer":
        """Frozen copy of this step's marks: its ``profile`` can be read after the timer has
        been reset for the next step."""
        frozen = _StepTimer(self.enabled, "cuda" if self.cuda else "cpu")
        frozen._marks = dict(self._marks)
        return frozen

    def _between(self, a: str, b: str) -> float:
        ma, mb = self._marks.get(a), self._marks.get(b)
        if ma is None or mb is None:
            return 0.0
        if self.cuda:
            return float(ma.elapsed_time(mb))
        return (mb - ma) * 1000.0

    def profile(self, num_tokens: int, synchronize: bool = True) -> dict[str, float] | None:
        """``synchronize=False``: the caller knows that every mark's event has completed."""
        if not self.enabled:
            return None
        if self.cuda and synchronize:
            torch.cuda.current_stream().synchronize()
        fetch = self._between("start", "fetch")
        fwd = self._between("fetch", "fwd")
        bwd = self._between("fwd", "bwd")
        opt = self._between("bwd", "opt")
        step = self._between("start", "opt")
        return {
            "fetch_ms": fetch, "fwd_ms": fwd, "bwd_ms": bwd, "opt_ms": opt, "step_ms": step,
            "tokens_per_s": num_tokens / (step / 1000.0) if step > 0 else 0.0,
            "fetch_frac": fetch / step if step > 0 else 0.0,
        }


class LossHandle:
    """Loss of one ``train_step_async`` call on its way to the host."""

    RING = 4

    def __init__(self, host: torch.Tensor, event) -> None:  # noqa: ANN001
        self._host, self._event = host, event

    def value(self) -> float:
        if self._event is not None:
            self._event.synchronize()
        return float(self._host[0])


def _with_lookahead(iterable):
    """``(item, next_item_or_None)`` pairs: lets the trainer start the next batch's
    host-to-device copy while the current step runs."""
    it = iter(iterable)
    try:
        cur = next(it)
    except StopIteration:
        return
    for nxt in it:
        yield cur, nxt
        cur = nxt
    yield cur, None


class _GraphedStep:
    """CUDA-graph capture of forward + backward (+ optimizer) per input signature."""

    def __init__(self, trainer: "Trainer", capture_optimizer: bool):
        self.trainer = trainer
        self.capture_optimizer = capture_optimizer
        self.cache: dict[tuple, tuple] = {}
        self.launches_per_capture: dict[tuple, int] = {}  # own-kernel launches recorded per graph
        self.capture_launch_total = 0  # launches issued while warming up / capturing
        # input prefetch: host->device copy of the next batch on a side stream while the
        # current step computes; [host batch object, staged device tensors, event]
        self._copy_stream: torch.cuda.Stream | None = None
        self._staged: tuple | None = None
        self._staging: dict[tuple, dict] = {}
        self._consumed: torch.cuda.Event | None = None

    @staticmethod
    def signature(batch: dict) -> tuple:
        return tuple(sorted((k, tuple(v.shape), str(v.dtype)) for k, v in batch.items() if isinstance(v, torch.Tensor)))

    def _capture(self, batch: dict):
        tr = self.trainer
        dev = tr.device
        from speculators_b200 import ops

        count_before = ops.native().launch_count()
        static_in = {k: torch.empty(v.shape, dtype=v.dtype, device=dev) for k, v in batch.items() if isinstance(v, torch.Tensor)}
        for k, v in static_in.items():
            v.copy_(batch[k], non_blocking=True)
        kwargs = tr.config.train_call_kwargs or {}
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):  # warm-up without touching the weights
                tr.engine.zero_grad()
                _, loss, _ = tr.model(**static_in, **kwargs)
                loss.backward()
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        count_capture = ops.native().launch_count()
        with torch.cuda.graph(graph):
            tr.engine.zero_grad()
            _, loss, metrics = tr.model(**static_in, **kwargs)
            loss.backward()
            if self.capture_optimizer:
                tr.engine.apply()
        count_after = ops.native().launch_count()
        self.launches_per_capture[self.signature(batch)] = count_after - count_capture
        self.capture_launch_total += count_after - count_before
        return graph, static_in, loss, metrics

    def prefetch(self, batch: dict) -> None:
        """Start copying ``batch`` (host tensors, ideally pinned) to the device on a side
        stream.  The next ``run`` given this same dict object picks the staged copy up
        instead of copying on the training stream."""
        sig = self.signature(batch)
        if self._copy_stream is None:
            self._copy_stream = torch.cuda.Stream()
        stage = self._staging.get(sig)
        if stage is None:
            stage = {k: torch.empty(v.shape, dtype=v.dtype, device=self.trainer.device) for k, v in batch.items() if isinstance(v, torch.Tensor)}
            self._staging[sig] = stage
            self._copy_stream.wait_stream(torch.cuda.current_stream())  # the fresh memory may have belonged to work still queued on the training stream
        # the staging buffers may still be read by the device-to-device copy of the step
        # that consumed the previous prefetch (only that copy: not the step's compute)
        if self._consumed is not None:
            self._copy_stream.wait_event(self._consumed)
        with torch.cuda.stream(self._copy_stream):
            for k, v in stage.items():
                v.copy_(batch[k], non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        self._staged = (batch, stage, done)

    def run(self, batch: dict, lr: float | None, next_batch: dict | None = None):
        sig = self.signature(batch)
        entry = self.cache.get(sig)
        tr = self.trainer
        if entry is None:
            entry = self._capture(batch)
            self.cache[sig] = entry
        graph, static_in, loss, metrics = entry
        source = batch
        if self._staged is not None and self._staged[0] is batch:
            _, source, done = self._staged
            torch.cuda.current_stream().wait_event(done)
        self._staged = None
        for k, v in static_in.items():
            v.copy_(source[k], non_blocking=True)
        if source is not batch:
            self._consumed = torch.cuda.Event()
            self._consumed.record()
        tr.timer.mark("fetch")
        tr.engine.prepare_hyper(lr)
        graph.replay()
        tr.timer.mark("fwd")
        tr.timer.mark("bwd")
        if not self.capture_optimizer:
            tr.engine.apply()
        if next_batch is not None:
            self.prefetch(next_batch)
        return loss, metrics


class Trainer:
    def __init__(self, model: SpeculatorModel, config: TrainerConfig, train_loader, val_loader=None):
        self.model = model
        self.config = config
        self.local_rank = get_local_rank()
        if config.process_group is not None:
            set_training_group(config.process_group)
        self.rank = training_rank() if config.process_group is not None else get_rank()
        self.train_loader = train_loader
        self.val_loader = val_loader
        self.is_distributed = is_distributed() or (dist.is_available() and dist.is_initialized())
        self.resume_from_checkpoint = config.resume_from_checkpoint
        if config.device is not None:
            self.device = torch.device(config.device)
        elif torch.cuda.is_available():
            self.device = torch.device("cuda", self.local_rank)
        else:
            self.device = torch.device("cpu")
        self.device_type = self.device.type
        self.checkpointer = Checkpointer(config.save_path)
        self.timer = _StepTimer(False, self.device_type)
        self.setup_trainer()
        self.setup_model()
        self.setup_optimizer()

    # ------------------------------------------------------------------ setup
    def _training_state_path(self, epoch) -> Path:
        return self.checkpointer.path / str(epoch) / "training_state.json"

    def _save_training_state(self, epoch: int, local_step: int) -> None:
        if not self.is_distributed or training_rank() == 0:
            path = self._training_state_path(epoch)
            path.parent.mkdir(parents=True, exist_ok=True)
            path.write_text(json.dumps({"epoch": epoch, "local_step": local_step, "global_step": self.global_step}))

    def _load_training_state(self) -> dict:
        path = self._training_state_path(self.checkpointer.previous_epoch)
        if path.exists():
            try:
                return json.loads(path.read_text())
            except (json.JSONDecodeError, OSError) as err:
                root_logger.warning("Failed to read training state %s: %s", path, err)
        return {}

    def setup_trainer(self) -> None:
        """Decide where training starts: fresh, next epoch, or inside an epoch."""
        self.current_epoch = 0
        self._resume_local_step = 0
        self._resume_global_step = 0
        prev = self.checkpointer.previous_epoch
        if prev == -1:
            root_logger.info("No previous training checkpoint found in '%s'. Starting fresh training run.", self.checkpointer.path)
        elif not self.resume_from_checkpoint:
            root_logger.warning(
                "`resume_from_checkpoint` is False, starting training from scratch. This will overwrite the "
                "existing checkpoints in %s.", self.checkpointer.path,
            )
        else:
            root_logger.info("Found checkpoint at %s.", self.checkpointer.prev_path)
            state = self._load_training_state()
            mid_epoch = bool(state) and state.get("epoch") == prev and state.get("local_step", 0) > 0
            self._resume_global_step = state.get("global_step", 0) if state else 0
            if mid_epoch:
                self.current_epoch = state["epoch"]
                self._resume_local_step = state["local_step"]
                root_logger.info(
                    "Resuming mid-epoch from epoch=%d local_step=%d global_step=%d.",
                    self.current_epoch, self._resume_local_step, self._resume_global_step,
                )
            else:
                self.current_epoch = prev + 1
                root_logger.info("Resuming training on epoch %d.", self.current_epoch)
        self.global_step = self._resume_global_step
        self.best_val_loss = float("inf")
        if self.resume_from_checkpoint and prev != -1:
            saved = self.checkpointer.load_best_val_loss()
            if saved is not None:
                self.best_val_loss = saved
                root_logger.info("Restored best_val_loss=%.6f from checkpoint", saved)

    def _loading_checkpoint(self) -> bool:
        return self.resume_from_checkpoint and self.checkpointer.previous_epoch != -1

    def setup_model(self) -> None:
        SpeculatorModel.verify_training_compatible(self.model)
        if self._loading_checkpoint():
            self.checkpointer.load_model_state_dict(self.model)

    def setup_optimizer(self) -> None:
        cfg = self.config
        compute_dtype = cfg.hidden_states_dtype if self.device_type == "cuda" else torch.float32
        self.engine = TrainEngine(
            self.model,
            EngineConfig(
                lr=cfg.lr, weight_decay=cfg.weight_decay, max_grad_norm=cfg.max_grad_norm, optimizer=cfg.optimizer,
                muon_lr=cfg.muon_lr, muon_momentum=cfg.muon_momentum, muon_weight_decay=cfg.muon_weight_decay,
                muon_ns_steps=cfg.muon_ns_steps, muon_adjust_lr_fn=cfg.muon_adjust_lr_fn,
                compute_dtype=compute_dtype, shard=cfg.fsdp_shard or hasattr(self.model, "_sb200_shard_request"), broadcast_from_rank0=True,
                group=cfg.process_group,
            ),
            device=self.device,
        )
        self.optimizers = [self.engine]
        if self._loading_checkpoint():
            self.checkpointer.load_optimizer_state_dict(self.model, self.engine)
        if cfg.scheduler_type == "none":
            self.schedulers: list[LRSchedule] = []
        else:
            warmup, total = resolve_scheduler_steps(cfg, len(self.train_loader))
            self.schedulers = [LRSchedule(cfg.scheduler_type, cfg.lr, warmup, total, cfg.scheduler_num_cosine_cycles)]
            if self._loading_checkpoint():
                self.checkpointer.load_scheduler_state_dict(self.schedulers)
        use_graph = cfg.use_cuda_graph if cfg.use_cuda_graph is not None else self.device_type == "cuda"
        # only models whose forward has fixed shapes and no host synchronisation can be replayed
        use_graph = use_graph and bool(getattr(self.model, "cuda_graph_safe", False))
        if use_graph and hasattr(self.model, "graph_safe_with"):
            use_graph = bool(self.model.graph_safe_with(dict(cfg.train_call_kwargs or {})))
        if os.environ.get("SB200_DISABLE_CUDA_GRAPH") == "1":
            use_graph = False
        self._graphed = None
        if use_graph and self.device_type == "cuda":
            # the fused peer-memory optimizer step is two plain kernels: capturable as is
            capture_opt = (
                (not self.is_distributed) or getattr(self.engine, "p2p", False)
                or os.environ.get("SB200_GRAPH_COLLECTIVES") == "1"
            )
            if os.environ.get("SB200_GRAPH_OPTIMIZER") == "0":
                capture_opt = False
            self._graphed = _GraphedStep(self, capture_optimizer=capture_opt)

    # ------------------------------------------------------------------ one step
    def _current_lr(self) -> float:
        return self.schedulers[0].current_lr() if self.schedulers else self.config.lr

    def train_step(self, batch: dict, next_batch: dict | None = None) -> tuple[torch.Tensor, dict[str, torch.Tensor]]:
        """One optimizer step on ``batch`` (host or device tensors).  Returns the
        loss and metric tensors on the training device.  ``next_batch`` (optional, the
        dict that the following call will receive) has its host-to-device copy started
        on a side stream so that it overlaps this step's compute."""
        lr = self._current_lr()
        if self._graphed is not None and not self._graphed.cache:
            # first capture of this trainer: a model whose step turns out not to be capturable (a host read
            # in a rarely used branch) falls back to eager steps instead of ending the run
            try:
                with nvtx_range("step (graph capture)"):
                    loss, metrics = self._graphed.run(batch, lr, next_batch)
            except RuntimeError as err:
                if "captur" not in str(err).lower():
                    raise
                root_logger.warning("CUDA graph capture of the training step failed (%s); running eager steps", str(err).splitlines()[0])
                self._graphed = None
                torch.cuda.synchronize(self.device)
                return self.train_step(batch, next_batch)
        elif self._graphed is not None:
            with nvtx_range("step (graph replay)"):
                loss, metrics = self._graphed.run(batch, lr, next_batch)
        else:
            with nvtx_range("fetch"):
                dev_batch = self._eager_inputs(batch)
            self.timer.mark("fetch")
            with nvtx_range("forward"):
                self.engine.zero_grad()
                _, loss, metrics = self.model(**dev_batch, **(self.config.train_call_kwargs or {}))
            self.timer.mark("fwd")
            with nvtx_range("backward"):
                loss.backward()
            self.timer.mark("bwd")
            with nvtx_range("optimizer"):
                self.engine.account_comm(self.timer.enabled)  # collectives of a logged step are timed
                self.engine.step(lr)
            stage = self.__dict__.get("_eager_stage")
            if stage is not None and stage.get("in_use") is not None:  # this step read a staged set: free once its work has run
                freed = torch.cuda.Event()
                freed.record()
                stage["free"][stage["in_use"]] = freed
                stage["in_use"] = None
            if next_batch is not None:
                self._eager_prefetch(next_batch)
        for sched in self.schedulers:
            sched.step()
        self.timer.mark("opt")
        return loss, metrics

    # ------------------------------------------------------------------ eager steps: input prefetch
    # A step that is not replayed from a CUDA graph reads its device inputs until its backward pass ends, so the
    # copy of the following batch cannot reuse the same buffers: two sets alternate, and a set is written again
    # only after the step that read it has finished (an event on the training stream).
    def _eager_prefetch(self, batch: dict) -> None:
        """Start the host-to-device copy of ``batch`` (host tensors, ideally pinned) on a side stream; the next
        ``train_step`` given this same dict picks the copy up instead of copying on the training stream."""
        if (self.device_type != "cuda" or os.environ.get("SB200_EAGER_PREFETCH", "1") == "0"
                or any(isinstance(v, torch.Tensor) and v.is_cuda for v in batch.values())):
            return
        state = self.__dict__.setdefault("_eager_stage", {"stream": torch.cuda.Stream(device=self.device), "sets": [{}, {}], "free": [None, None],
                                                           "turn": 0, "ready": None, "in_use": None})
        turn = state["turn"]
        state["turn"] = turn ^ 1
        sig = _GraphedStep.signature(batch)
        slot = state["sets"][turn]
        if slot.get("sig") != sig:
            slot.clear()
            slot.update(sig=sig, tensors={k: torch.empty(v.shape, dtype=v.dtype, device=self.device) for k, v in batch.items() if isinstance(v, torch.Tensor)})
            # The allocator may hand out memory that temporaries of the step in flight gave back in the training stream's
            # order: another stream may write it only after that stream has caught up (once per set, at its allocation).
            state["stream"].wait_stream(torch.cuda.current_stream(self.device))
        if state["free"][turn] is not None:  # the step that read this set two steps ago must have ended
            state["stream"].wait_event(state["free"][turn])
        with torch.cuda.stream(state["stream"]):
            for k, v in slot["tensors"].items():
                v.copy_(batch[k], non_blocking=True)
            done = torch.cuda.Event()
            done.record()
        state["ready"] = (batch, turn, done)

    def _eager_inputs(self, batch: dict) -> dict:
        state = self.__dict__.get("_eager_stage")
        if state is not None and state["ready"] is not None and state["ready"][0] is batch:
            _, turn, done = state["ready"]
            state["ready"] = None
            torch.cuda.current_stream().wait_event(done)
            staged = state["sets"][turn]["tensors"]
            state["in_use"] = turn  # ``train_step`` records the event that frees the set after the step's last kernel
            return {k: staged.get(k, v) if isinstance(v, torch.Tensor) else v for k, v in batch.items()}
        return {k: v.to(self.device, non_blocking=True) if isinstance(v, torch.Tensor) else v for k, v in batch.items()}

    def train_step_async(self, batch: dict, next_batch: dict | None = None) -> "LossHandle":
        """``train_step`` that does not make the host wait for the step: the loss is copied to
        pinned host memory behind the step on the training stream and returned as a handle
        whose ``value()`` waits for just that copy.  Reading the handle of step ``n`` after
        step ``n + 1`` has been enqueued keeps the device busy while the host reads.  At most
        ``LossHandle.RING`` handles may be outstanding."""
        loss, _ = self.train_step(batch, next_batch)
        if not hasattr(self, "_loss_ring"):
            pin = self.device.type == "cuda"
            self._loss_ring = [torch.zeros(1, dtype=torch.float32, pin_memory=pin) for _ in range(LossHandle.RING)]
            self._loss_ring_pos = 0
        slot = self._loss_ring[self._loss_ring_pos % LossHandle.RING]
        self._loss_ring_pos += 1
        slot.copy_(loss.detach().reshape(1), non_blocking=True)
        event = None
        if self.device.type == "cuda":
            event = torch.cuda.Event()
            event.record()
        return LossHandle(slot, event)

    # ------------------------------------------------------------------ epochs
    def _prepare_resume_skip(self, epoch: int) -> int:
        skip = 0
        if epoch == getattr(self, "current_epoch", epoch):
            skip = getattr(self, "_resume_local_step", 0)
            self._resume_local_step = 0
        sampler = getattr(self.train_loader, "batch_sampler", None)
        fast = hasattr(sampler, "_generate_batches") and hasattr(sampler, "_cached_generated_batches")
        if skip > 0 and fast:
            remaining = sampler._generate_batches(epoch)[skip:]  # noqa: SLF001
            sampler._cached_generated_batches = (epoch, remaining)  # noqa: SLF001
            root_logger.info("Fast-skipping %d batches via sampler slice. epoch=%d, global_step=%d.", skip, epoch, self.global_step)
        elif skip > 0:
            root_logger.warning("Sampler lacks fast-skip API; resume will replay %d batches from the start of the epoch.", skip)
        return skip

    def train_epoch(self, epoch: int) -> None:
        self.model.train()
        sampler = getattr(self.train_loader, "batch_sampler", None)
        if hasattr(sampler, "set_epoch"):
            sampler.set_epoch(epoch)
        num_steps = len(self.train_loader)
        skip_steps = self._prepare_resume_skip(epoch)
        cfg = self.config
        step_interval = max(1, round(num_steps * cfg.checkpoint_freq)) if cfg.checkpoint_freq < 1 else None
        loader = self.train_loader
        if self.rank == 0 and os.environ.get("SB200_NO_TQDM") != "1":
            try:
                from tqdm import tqdm

                loader = tqdm(loader, desc=f"Epoch {epoch}")
            except ImportError:
                pass
        self.timer.reset(self.global_step % cfg.log_freq == 0)
        self.timer.mark("start")
        for rel, (batch, upcoming) in enumerate(_with_lookahead(loader), 1):
            local_step = rel + skip_steps
            loss, metrics = self.train_step(batch, upcoming)
            lr_now = self._current_lr()
            if self.timer.enabled:
                # the record of the previous logged step is complete by now: emit it, then queue
                # this step's (its values are copied to pinned memory behind the step)
                self._flush_step_log()
                self._queue_step_log(epoch, lr_now, metrics, batch)
            self.global_step += 1
            self.timer.reset(self.global_step % cfg.log_freq == 0)
            self.timer.mark("start")
            if cfg.max_steps is not None and self.global_step >= cfg.max_steps:
                break
            if (
                step_interval is not None and not cfg.save_best and local_step % step_interval == 0
                and num_steps - local_step >= step_interval * MIN_STEP_PCT
            ):
                self._flush_step_log()
                self.maybe_save_checkpoint(epoch, local_step=local_step)
        self._flush_step_log()
        self.check_device_status()

    # ------------------------------------------------------------------ step logging
    def _queue_step_log(self, epoch: int, lr_now: float, metrics: dict, batch) -> None:  # noqa: ANN001
        """Start moving a step's metrics to the host without waiting for the step: one stacked
        device tensor (summed over ranks when distributed), copied to pinned memory behind the
        step on the training stream.  ``_flush_step_log`` reads it when the next logged step
        comes around (or at the end of the epoch), so logging every step does not put a host
        synchronisation between consecutive steps."""
        keys = list(metrics)
        entries = [metrics[k].detach().float().reshape(()) for k in keys]
        doc = batch.get("document_ids") if isinstance(batch, dict) else None
        num_tokens = 0
        if doc is not None and doc.device.type == "cpu":
            num_tokens = int((doc != -1).sum())
        elif doc is not None:
            entries.append((doc != -1).sum().float())  # counted on the device, read with the rest
        has_count = doc is not None and doc.device.type != "cpu"
        words = self._status_words()
        status = torch.cat([w.reshape(1) for _, w, _ in words]).float() if words else None
        host = event = None
        n_metrics = len(keys)
        if entries or status is not None:
            stacked = torch.stack(entries) if entries else torch.zeros(0, device=self.device)
            if self.is_distributed and n_metrics:
                head = stacked[:n_metrics].clone()
                group = self.config.process_group
                dist.reduce(head, dst=dist.get_global_rank(group, 0) if group is not None else 0, op=dist.ReduceOp.SUM, group=group)
                stacked = torch.cat([head, stacked[n_metrics:]])
            if status is not None:
                stacked = torch.cat([stacked, status])
            host = torch.empty(stacked.shape, dtype=torch.float32, pin_memory=self.device_type == "cuda")
            host.copy_(stacked, non_blocking=True)
            if self.device_type == "cuda":
                event = torch.cuda.Event()
                event.record()
        self._pending_step_log = {
            "keys": keys, "host": host, "event": event, "timer": self.timer.snapshot(), "epoch": epoch, "lr": lr_now,
            "engine": self.engine if self._graphed is None else None,
            "global_step": self.global_step, "num_tokens": num_tokens, "has_count": has_count, "status_checks": [(label, check) for label, _, check in words],
        }

    def _status_words(self) -> list:
        """``(label, device int32 word, check(code))`` of everything on this rank that reports
        a bounded wait running out: the tcgen05 kernels, the peer-memory optimizer step, every
        expert-parallel exchange.  Their values ride along with the logged step's record; a
        non-zero value stops training (the step that set it did no update, or read stale rows)."""
        if self.device_type != "cuda":
            return []
        from speculators_b200.ops import check_gemm_status, gemm_status

        words = [("tcgen05", gemm_status(self.device), lambda _code: check_gemm_status())]
        words.append(("optimizer", self.engine.status, self.engine.check_status))
        for name, mod in self.model.named_modules():
            comm = getattr(mod, "_comm", None)
            if comm is not None and hasattr(comm, "status") and hasattr(comm, "check_status"):
                words.append((f"expert exchange {name}", comm.status, comm.check_status))
        return words

    def check_device_status(self) -> None:
        """Read every status word now (one host synchronisation) and raise on the first that is
        set.  Called before a checkpoint is written and at the end of an epoch, so that weights
        produced after a failed wait are never saved as if they were good."""
        words = self._status_words()
        if not words:
            return
        codes = torch.cat([w.reshape(1) for _, w, _ in words]).tolist()
        for (label, _, check), code in zip(words, codes):
            if code != 0:
                root_logger.error("device status word '%s' = %d: stopping", label, int(code))
                check(int(code))

    def _flush_step_log(self) -> None:
        pending = getattr(self, "_pending_step_log", None)
        if pending is None:
            return
        self._pending_step_log = None
        if pending["event"] is not None:
            pending["event"].synchronize()
        raw = pending["host"].tolist() if pending["host"] is not None else []
        keys = pending["keys"]
        values = dict(zip(keys, raw[: len(keys)]))
        rest = raw[len(keys):]
        num_tokens = pending["num_tokens"]
        if pending["has_count"]:
            num_tokens = int(rest.pop(0))
        checks = pending["status_checks"]
        for (label, check), code in zip(checks, rest[len(rest) - len(checks):] if checks else []):
            if code != 0:
                root_logger.error("device status word '%s' = %d at global step %d: stopping", label, int(code), pending["global_step"])
                check(int(code))  # raises with the meaning of the code
        profile = pending["timer"].profile(num_tokens, synchronize=pending["event"] is None)  # the marks precede the copy's event
        if profile is not None and pending.get("engine") is not None:
            comm = pending["engine"].exposed_comm_ms()  # library collectives of that step; None: none timed
            if comm is not None:
                profile["comm_ms"] = comm
                profile["comm_frac"] = comm / profile["step_ms"] if profile["step_ms"] > 0 else 0.0
        world = dist.get_world_size(self.config.process_group) if self.is_distributed else 1
        metric_logger.info(
            {"train": normalize_counted_metrics(values, world), "profile": profile, "epoch": pending["epoch"], "lr": pending["lr"],
             "global_step": pending["global_step"]},
            extra={"step": pending["global_step"]},
        )

    def _maybe_val_sync(self, batch_index: int) -> None:
        if not self.is_distributed or _VAL_SYNC_INTERVAL <= 0:
            return
        if batch_index > 0 and batch_index % _VAL_SYNC_INTERVAL == 0:
            dist.barrier(group=getattr(getattr(self, "config", None), "process_group", None))

    @torch.no_grad()
    def val_epoch(self, epoch: int) -> dict[str, float] | None:
        if self.val_loader is None:
            return None
        self.model.eval()
        sampler = getattr(self.val_loader, "batch_sampler", None)
        if hasattr(sampler, "set_epoch"):
            sampler.set_epoch(epoch)
        accumulated: dict[str, torch.Tensor] = {}
        num_batches = len(self.val_loader)
        device = getattr(self, "device", None)
        if device is None:  # a trainer assembled by hand (tests): what ``__init__`` would have chosen
            device = torch.device("cuda", self.local_rank) if self.device_type == "cuda" else torch.device(self.device_type)
        for i, batch in enumerate(self.val_loader):
            self._maybe_val_sync(i)
            dev_batch = {k: v.to(device, non_blocking=True) if isinstance(v, torch.Tensor) else v for k, v in batch.items()}
            _, _loss, metrics = self.model(**dev_batch, **(self.config.val_call_kwargs or {}))
            for k, v in metrics.items():
                accumulated[k] = v.float() if k not in accumulated else accumulated[k] + v.float()
        val_metrics: dict[str, float] = {}
        if accumulated:
            stacked = torch.stack([v.reshape(()) for v in accumulated.values()])
            if self.is_distributed:
                dist.all_reduce(stacked, op=dist.ReduceOp.SUM, group=self.config.process_group)
            val_metrics = dict(zip(accumulated, stacked.tolist(), strict=True))
        world = dist.get_world_size(self.config.process_group) if self.is_distributed else 1
        val_metrics = {k: v / max(1, num_batches) for k, v in val_metrics.items()}
        val_metrics = {f"{k}_epoch": v for k, v in normalize_counted_metrics(val_metrics, world).items()}
        metric_logger.info({"val": val_metrics, "epoch": epoch}, extra={"step": self.global_step})
        return val_metrics

    # ------------------------------------------------------------------ checkpoints
    def maybe_save_checkpoint(self, epoch, local_step: int = 0) -> None:
        cfg = self.config
        if epoch != "interrupted" and (
            cfg.save_best
            or (cfg.checkpoint_freq >= 1 and isinstance(epoch, int) and epoch != 0 and (epoch + 1) % cfg.checkpoint_freq != 0)
        ):
            return
        if epoch != "interrupted":
            self.check_device_status()
        root_logger.info("Saving checkpoint to %s", self.checkpointer.path / str(epoch))
        self.checkpointer.save_checkpoint(self.model, self.engine, epoch)
        if self.schedulers:
            self.checkpointer.save_scheduler_state_dict(self.schedulers, epoch)
        if isinstance(epoch, int):
            self._save_training_state(epoch, local_step)
            if not self.is_distributed or training_rank() == 0:
                root = self.checkpointer.path
                for old in root.glob(f"epoch{epoch}_*"):
                    if old.is_symlink():
                        old.unlink()
                suffix = f"step{local_step}" if local_step > 0 else "end"
                (root / f"epoch{epoch}_{suffix}").symlink_to(Path(str(epoch)))
        root_logger.info("Checkpoint saved to %s", self.checkpointer.path / str(epoch))

    def maybe_update_best(self, epoch: int, val_metrics: dict | None) -> None:
        if val_metrics is None or "loss_epoch" not in val_metrics:
            return
        if val_metrics["loss_epoch"] >= self.best_val_loss:
            return
        cfg = self.config
        if cfg.save_best:
            self.checkpointer.save_checkpoint(self.model, self.engine, epoch)
            if self.schedulers:
                self.checkpointer.save_scheduler_state_dict(self.schedulers, epoch)
        elif cfg.checkpoint_freq >= 1 and not (epoch == 0 or (epoch + 1) % int(cfg.checkpoint_freq) == 0):
            return
        self.best_val_loss = val_metrics["loss_epoch"]
        self.checkpointer.save_val_metrics(epoch, val_metrics)
        self.checkpointer.update_best_symlink(epoch)
        root_logger.info("Updated checkpoint_best -> %s (loss_epoch=%.6f)", epoch, self.best_val_loss)
        if cfg.save_best:
            self.checkpointer.cleanup_keep_only_best(best_epoch=epoch)

    def _barrier(self) -> None:
        if self.is_distributed:
            dist.barrier(group=self.config.process_group)

    @with_graceful_shutdown()
    def run_training(self) -> None:
        n_epochs = self.config.num_epochs
        for epoch in range(self.current_epoch, n_epochs):
            root_logger.info("Training epoch %d/%d started", epoch + 1, n_epochs)
            self.train_epoch(epoch)
            root_logger.info("Training epoch %d/%d completed", epoch + 1, n_epochs)
            self._barrier()
            self.maybe_save_checkpoint(epoch)
            self._barrier()
            val_metrics = None
            if self.val_loader is None:
                root_logger.warning("No val loader, skipping validation epoch")
            else:
                val_metrics = self.val_epoch(epoch)
            self._barrier()
            self.maybe_update_best(epoch, val_metrics)
            self._barrier()
            if self.config.max_steps is not None and self.global_step >= self.config.max_steps:
                break
