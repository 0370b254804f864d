"""Trainer internals on CPU: step timer, LR schedules and their step resolution, lookahead
iteration, graceful shutdown, checkpoint bookkeeping (best link, keep-only-best), mid-epoch
resume state, validation metric normalisation."""

import json
import os
import signal
import warnings

import pytest
import torch

import speculators_b200 as sb
from speculators_b200.train import Trainer, TrainerConfig
from speculators_b200.train.checkpointer import Checkpointer
from speculators_b200.train.graceful_shutdown import GracefulShutdownHandler, TrainingInterrupted, with_graceful_shutdown
from speculators_b200.train.schedule import LRSchedule, resolve_scheduler_steps
from speculators_b200.train.synthetic import SyntheticLoader
from speculators_b200.train.trainer import _StepTimer, _with_lookahead

from conftest import make_tiny_batch, make_tiny_eagle3


def test_step_timer_phases():
    t = _StepTimer(enabled=False)
    t.mark("start")
    assert t.profile(10) is None
    t.reset(True)
    for name in ("start", "fetch", "fwd", "bwd", "opt"):
        t.mark(name)
    prof = t.profile(1000)
    assert set(prof) == {"fetch_ms", "fwd_ms", "bwd_ms", "opt_ms", "step_ms", "tokens_per_s", "fetch_frac"}
    assert prof["step_ms"] >= prof["fetch_ms"] >= 0 and abs(prof["step_ms"] - sum(prof[k] for k in ("fetch_ms", "fwd_ms", "bwd_ms", "opt_ms"))) < 1e-6
    t.reset(True)
    t.mark("start")
    assert t.profile(5)["tokens_per_s"] == 0.0  # missing marks read as zero-length phases


def test_lookahead_pairs():
    assert list(_with_lookahead([])) == []
    assert list(_with_lookahead("a")) == [("a", None)]
    assert list(_with_lookahead([1, 2, 3])) == [(1, 2), (2, 3), (3, None)]


def _cfg(**kw):
    base = dict(lr=1.0, num_epochs=2, save_path="unused", scheduler_total_steps=None, scheduler_warmup_steps=None, scheduler_warmup_ratio=None)
    return TrainerConfig(**{**base, **kw})


def test_scheduler_step_resolution_and_shapes():
    assert resolve_scheduler_steps(_cfg(), 50) == (1, 100)  # 1 % warm-up of epochs x loader length
    assert resolve_scheduler_steps(_cfg(scheduler_total_steps=400, scheduler_warmup_ratio=0.25), 50) == (100, 400)
    with warnings.catch_warnings(record=True) as caught:
        warnings.simplefilter("always")
        assert resolve_scheduler_steps(_cfg(scheduler_warmup_steps=7, scheduler_warmup_ratio=0.5), 50) == (7, 100)
    assert any("using scheduler_warmup_steps" in str(w.message) for w in caught)
    with pytest.raises(ValueError):
        resolve_scheduler_steps(_cfg(scheduler_warmup_ratio=1.5), 50)
    lin = LRSchedule("linear", 2.0, warmup_steps=4, total_steps=12)
    lrs = []
    for _ in range(13):
        lrs.append(lin.current_lr())
        lin.step()
    assert lrs[0] == 0.0 and lrs[2] == 1.0 and lrs[4] == 2.0 and lrs[8] == 1.0 and lrs[12] == 0.0
    cos = LRSchedule("cosine", 1.0, warmup_steps=0, total_steps=10)
    cos.last_step = 5
    assert abs(cos.current_lr() - 0.5) < 1e-9
    again = LRSchedule("cosine", 1.0, total_steps=10)
    again.load_state_dict(cos.state_dict())
    assert again.last_step == 5 and LRSchedule("none", 3.0).current_lr() == 3.0
    with pytest.raises(ValueError):
        LRSchedule("exp", 1.0)


def test_graceful_shutdown_saves_interrupted_checkpoint():
    calls = []

    class FakeTrainer:
        def maybe_save_checkpoint(self, tag):
            calls.append(tag)

        @with_graceful_shutdown(timeout_s=30)
        def run_training(self):
            os.kill(os.getpid(), signal.SIGTERM)
            for _ in range(10**6):  # the handler raises inside this loop
                pass
            return "finished"

    before = signal.getsignal(signal.SIGTERM)
    with pytest.raises(SystemExit) as stop:
        FakeTrainer().run_training()
    assert stop.value.code == 128 + signal.SIGTERM and calls == ["interrupted"]
    assert signal.getsignal(signal.SIGTERM) is before  # handlers restored
    with GracefulShutdownHandler() as h:
        with pytest.raises(TrainingInterrupted):
            os.kill(os.getpid(), signal.SIGINT)
            for _ in range(10**6):
                pass
        h._handle(signal.SIGINT, None)  # a repeat while shutting down is ignored, not raised
    assert h.triggered == signal.SIGINT


def test_checkpointer_best_link_and_cleanup(tmp_path):
    ck = Checkpointer(tmp_path)
    assert ck._get_previous_epoch() == -1 and ck.read_best_epoch() is None and ck.load_best_val_loss() is None
    for epoch, loss in ((0, 3.0), (1, 2.0), (2, 2.5)):
        ck.model_path(epoch).parent.mkdir(parents=True, exist_ok=True)
        ck.model_path(epoch).write_text("w")
        ck.save_val_metrics(epoch, {"loss_epoch": loss})
    (tmp_path / "interrupted").mkdir()
    assert ck._get_previous_epoch() == 2
    ck.update_best_symlink(1)
    assert ck.read_best_epoch() == 1 and ck.load_best_val_loss() == 2.0 and os.path.islink(ck.best_path())
    ck.update_best_symlink(0)  # re-pointing replaces the link
    assert ck.read_best_epoch() == 0
    ck.update_best_symlink(1)
    ck.cleanup_keep_only_best(1)
    assert sorted(p.name for p in tmp_path.iterdir() if p.is_dir() and not p.is_symlink() and p.name.isdigit()) == ["1"]


def test_mid_epoch_checkpoint_and_resume(tiny_verifier_dir, tiny_vocab_maps, tmp_path):
    """checkpoint_freq < 1 saves inside the epoch with the local step; a new trainer over
    the same directory resumes at that step and finishes the epoch."""
    kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=2, ttt_step_loss_decay=1.0)
    batches = [make_tiny_batch(T=40, seed=s) for s in range(4)]

    class Crash(RuntimeError):
        pass

    class IndexSampler:
        """The slice of the multipack sampler's interface that fast resume uses."""

        def __init__(self, n):
            self.n, self.epoch, self._cached_generated_batches = n, 0, None

        def set_epoch(self, epoch):
            self.epoch = epoch

        def _generate_batches(self, epoch):
            return [[i] for i in range(self.n)]

        def __iter__(self):
            cached = self._cached_generated_batches
            yield from (cached[1] if cached and cached[0] == self.epoch else self._generate_batches(self.epoch))

    class IndexedLoader:
        crash_at = None

        def __init__(self, data, n):
            self.data, self.batch_sampler = data, IndexSampler(n)

        def __len__(self):
            return self.batch_sampler.n

        def __iter__(self):
            for (i,) in self.batch_sampler:
                if self.crash_at is not None and i == self.crash_at:
                    raise Crash("node lost")
                yield self.data[i]

    class CrashingLoader(IndexedLoader):
        crash_at = 3

    def trainer(loader_cls=IndexedLoader):
        model = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
        return Trainer(model, TrainerConfig(lr=1e-3, num_epochs=1, save_path=str(tmp_path), train_call_kwargs=kwargs, val_call_kwargs=kwargs,
                                            scheduler_type="none", checkpoint_freq=0.5, log_freq=1, device="cpu", resume_from_checkpoint=True),
                       loader_cls(batches, 4), SyntheticLoader(batches[:2], 2))

    first = trainer(CrashingLoader)
    with pytest.raises(Crash):
        first.run_training()  # dies on the fourth batch, after the half-epoch checkpoint
    state = json.loads((tmp_path / "0" / "training_state.json").read_text())
    assert state["epoch"] == 0 and state["local_step"] == 2 and state["global_step"] == 2
    assert (tmp_path / "epoch0_step2").is_symlink()
    second = trainer()
    assert second.global_step == 2 and second._resume_local_step == 2 and second.current_epoch == 0
    second.run_training()
    assert second.global_step == 4
    final = json.loads((tmp_path / "0" / "training_state.json").read_text())
    assert final["global_step"] == 4
    val = second.val_epoch(0)
    assert val is not None and all(k.endswith("_epoch") for k in val) and "loss_epoch" in val and 0.0 <= val["full_acc_0_epoch"] <= 1.0


def test_async_step_handles_on_cpu(tiny_verifier_dir, tiny_vocab_maps, tmp_path):
    """The handle API also works without a GPU (no event, plain host tensor)."""
    import copy

    import speculators_b200 as sb
    from speculators_b200.train import Trainer, TrainerConfig
    from speculators_b200.train.synthetic import SyntheticLoader
    from tests.conftest import make_tiny_batch, make_tiny_eagle3

    base = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
    batch = make_tiny_batch(T=32)
    kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=2, ttt_step_loss_decay=1.0)

    def make(model):
        return Trainer(model, TrainerConfig(lr=1e-3, num_epochs=1, save_path=str(tmp_path / str(id(model))), train_call_kwargs=kwargs,
                                            scheduler_type="none", log_freq=10**9, device="cpu"), SyntheticLoader([batch], 3))

    a, b = make(copy.deepcopy(base)), make(copy.deepcopy(base))
    want = [float(a.train_step(batch)[0].item()) for _ in range(3)]
    handles = [b.train_step_async(batch) for _ in range(3)]
    # on the CPU every handle holds its own value only until the ring wraps; three fit
    assert [h.value() for h in handles] == pytest.approx(want, rel=1e-6)


def test_step_records_are_emitted_in_order_one_step_late_and_flushed(tiny_verifier_dir, tiny_vocab_maps, tmp_path):
    """Per-step logging does not wait for the step: the record of step n is emitted when step
    n + 1 is queued, and the last one when the epoch ends; nothing is lost or reordered."""
    import logging

    import speculators_b200 as sb
    from speculators_b200.train import Trainer, TrainerConfig
    from speculators_b200.train import trainer as trainer_mod
    from speculators_b200.train.synthetic import SyntheticLoader
    from tests.conftest import make_tiny_batch, make_tiny_eagle3

    records = []

    class Capture(logging.Handler):
        def emit(self, record):
            if isinstance(record.msg, dict) and "train" in record.msg:
                records.append(record.msg)

    handler = Capture()
    trainer_mod.metric_logger.addHandler(handler)
    old_level = trainer_mod.metric_logger.level
    trainer_mod.metric_logger.setLevel(logging.INFO)
    try:
        model = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
        batch = make_tiny_batch(T=32)
        kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=2, ttt_step_loss_decay=1.0)
        trainer = Trainer(model, TrainerConfig(lr=1e-3, num_epochs=1, save_path=str(tmp_path), train_call_kwargs=kwargs, scheduler_type="none",
                                               log_freq=1, device="cpu"), SyntheticLoader([batch], 4))
        import os

        os.environ["SB200_NO_TQDM"] = "1"
        trainer.train_epoch(0)
    finally:
        trainer_mod.metric_logger.removeHandler(handler)
        trainer_mod.metric_logger.setLevel(old_level)
    assert [r["global_step"] for r in records] == [0, 1, 2, 3]
    assert all("loss" in r["train"] and r["profile"] is not None and r["profile"]["step_ms"] >= 0 for r in records)
    losses = [r["train"]["loss"] for r in records]
    assert losses[-1] < losses[0]
    assert getattr(trainer, "_pending_step_log", None) is None


@pytest.mark.parametrize("log_freq", [1, 10**9])
def test_device_status_word_stops_training(tiny_verifier_dir, tiny_vocab_maps, tmp_path, log_freq):
    """A status word that a bounded device wait set (here: injected on the host) must end the
    run with an error: on the next logged step when steps are logged, else at the end of the
    epoch, and before any checkpoint is written."""
    kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=2, ttt_step_loss_decay=1.0)
    batches = [make_tiny_batch(T=32, seed=s) for s in range(3)]
    model = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
    tr = Trainer(model, TrainerConfig(lr=1e-3, num_epochs=1, save_path=str(tmp_path), train_call_kwargs=kwargs, scheduler_type="none",
                                      log_freq=log_freq, device="cpu"), SyntheticLoader(batches, 3))
    word = torch.zeros(1, dtype=torch.int32)
    tr._status_words = lambda: [("optimizer", word, tr.engine.check_status)]
    tr.train_epoch(0)  # all clear: runs through
    word.fill_(11)
    with pytest.raises(RuntimeError, match="fused optimizer step timed out waiting at the gradient barrier"):
        tr.train_epoch(0)
    with pytest.raises(RuntimeError, match="timed out"):
        tr.maybe_save_checkpoint(0)
    assert not (tmp_path / "0").exists()


def test_optimizer_state_formats(tiny_verifier_dir, tiny_vocab_maps, tmp_path, caplog):
    """A torch.optim-format state dict (what the reference's checkpoints hold) is recognised
    and refused with a warning instead of being skipped silently."""
    import logging

    from speculators_b200.parallel.engine import EngineConfig, TrainEngine

    eng = TrainEngine(make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps), EngineConfig(compute_dtype=torch.float32), device="cpu")
    eng.step_count = 5
    own = eng.optimizer_state_dict(first_rank_only=True)
    assert own["step"] == 5 and set(own["state"]) == set(eng.names)
    with caplog.at_level(logging.WARNING):
        eng.load_optimizer_state_dict({"state": {0: {"step": torch.tensor(3.0)}}, "param_groups": [{"lr": 1e-4, "params": [0]}]})
    assert "torch.optim format" in caplog.text and eng.step_count == 5
    caplog.clear()
    with caplog.at_level(logging.WARNING):
        eng.load_optimizer_state_dict({"step": 2, "state": {"no.such.weight": {}}})
    assert "matches none" in caplog.text and eng.step_count == 2
    eng.load_optimizer_state_dict(own)
    assert eng.step_count == 5


# ---- "rank 0" duties follow the training sub-group when one is declared ------------------------------
def _training_group_worker(rank, world, port, out_dir):
    import os

    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from speculators_b200.parallel import distributed as topo
    from speculators_b200.train import checkpointer
    from speculators_b200.train.logger import IsRank0Filter

    before = (topo.training_rank(), checkpointer._is_rank0())  # noqa: SLF001
    group = dist.new_group([1, 2])  # every rank takes part in the creation
    topo.set_training_group(group)
    topo.training_barrier()  # members only; rank 0 returns at once
    after = (topo.training_rank(), checkpointer._is_rank0(), IsRank0Filter()._rank())  # noqa: SLF001
    topo.set_training_group(None)
    with open(os.path.join(out_dir, f"{rank}.txt"), "w") as fh:
        fh.write(repr((before, after)))
    dist.barrier()
    dist.destroy_process_group()
    os._exit(0)


def test_rank0_duties_follow_the_training_group(tmp_path):
    import ast

    import torch.multiprocessing as mp

    mp.spawn(_training_group_worker, args=(3, 29771, str(tmp_path)), nprocs=3, join=True)
    seen = {r: ast.literal_eval((tmp_path / f"{r}.txt").read_text()) for r in range(3)}
    assert [seen[r][0] for r in range(3)] == [(0, True), (1, False), (2, False)]  # the job's rank 0 before a group is declared
    assert seen[0][1] == (-1, False, -1)  # outside the training group: no duties
    assert seen[1][1] == (0, True, 0) and seen[2][1] == (1, False, 1)
