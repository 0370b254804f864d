"""Checkpoint layout, save / load, best-epoch bookkeeping.

On disk (same directory layout as src/speculators/train/checkpointer.py:54-68; every epoch
directory is directly ``vllm serve``-able).  ``config.json`` and ``model.safetensors`` are
interchangeable with the reference.  ``optimizer_state_dict.pt`` and
``scheduler_state_dict.pt`` are not: they hold this engine's name-keyed fp32 master / moment
tensors and an ``LRSchedule`` state, where the reference stores ``torch.optim`` state dicts
keyed by parameter index; loading the other format restarts the optimizer with a warning::

    <save_path>/<epoch>/config.json, model.safetensors (bf16),
                        optimizer_state_dict.pt, scheduler_state_dict.pt,
                        training_state.json, val_metrics.json, train_command.txt
    <save_path>/epoch<E>_{end|step<K>} -> <E>      descriptive symlink
    <save_path>/checkpoint_best        -> <E>
    <save_path>/interrupted/                       written on graceful shutdown

One class serves single-process, replicated and sharded training: the engine
gathers ``master_state_dict`` on every rank (every rank's model copy stays complete) and the
optimizer state on rank 0 only, rank 0 writes, everyone meets at a barrier.
The reference needs two classes because FSDP2 state lives in DTensors
(``DistributedCheckpointer``, :359-438); both names are kept as aliases.
"""

from __future__ import annotations

import json
import logging
import shutil
from pathlib import Path

import torch
import torch.distributed as dist
from safetensors.torch import load_file

log = logging.getLogger("speculators")

__all__ = [
    "BaseCheckpointer", "Checkpointer", "DistributedCheckpointer", "SingleGPUCheckpointer",
    "convert_float_dtype", "load_safetensors_state_dict", "patch_config_dtype",
]

TRAIN_COMMAND_FILENAME = "train_command.txt"


def _is_rank0() -> bool:
    """The writer of checkpoint files: rank 0 of the training ranks (of the whole job unless a training
    sub-group is declared, ``parallel.distributed.set_training_group``)."""
    from speculators_b200.parallel.distributed import training_rank

    return not (dist.is_available() and dist.is_initialized()) or training_rank() == 0


def _barrier() -> None:
    from speculators_b200.parallel.distributed import training_barrier

    training_barrier()


def convert_float_dtype(obj, dtype: torch.dtype):
    """Recursively cast floating tensors in nested dict / list structures."""
    if isinstance(obj, torch.Tensor):
        return obj.to(dtype) if obj.is_floating_point() else obj
    if isinstance(obj, dict):
        return {k: convert_float_dtype(v, dtype) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(convert_float_dtype(v, dtype) for v in obj)
    return obj


def load_safetensors_state_dict(path: str | Path, device: str = "cpu") -> dict[str, torch.Tensor]:
    return load_file(str(path), device=device)


def patch_config_dtype(checkpoint_dir: str | Path, dtype: torch.dtype) -> None:
    """Make ``config.json`` advertise the dtype the weights were saved in."""
    cfg = Path(checkpoint_dir) / "config.json"
    if not cfg.exists():
        return
    data = json.loads(cfg.read_text())
    name = str(dtype).removeprefix("torch.")
    data["torch_dtype"] = name
    if "dtype" in data:
        data["dtype"] = name
    cfg.write_text(json.dumps(data, indent=2, sort_keys=True) + "\n")


class Checkpointer:
    def __init__(self, path: Path | str):
        self.path = Path(path)
        self.previous_epoch = self._get_previous_epoch()
        self.prev_path: Path | None = self.path / str(self.previous_epoch) if self.previous_epoch != -1 else None

    # ---- paths ---------------------------------------------------------------
    def _get_previous_epoch(self) -> int:
        if not self.path.exists():
            return -1
        newest = -1
        for entry in self.path.iterdir():
            if entry.is_symlink() or not entry.is_dir():
                continue
            if entry.name == "interrupted":
                log.warning(
                    "Found interrupted checkpoint at %s. To resume from it, rename it to an epoch number "
                    "(e.g., 'mv interrupted 5' to resume as epoch 5).", entry,
                )
                continue
            if entry.name.isdigit():
                newest = max(newest, int(entry.name))
        return newest

    def model_path(self, epoch) -> Path:
        return self.path / str(epoch) / "model.safetensors"

    def optimizer_path(self, epoch) -> Path:
        return self.path / str(epoch) / "optimizer_state_dict.pt"

    def scheduler_path(self, epoch) -> Path:
        return self.path / str(epoch) / "scheduler_state_dict.pt"

    def val_metrics_path(self, epoch) -> Path:
        return self.path / str(epoch) / "val_metrics.json"

    def best_path(self) -> Path:
        return self.path / "checkpoint_best"

    # ---- save ------------------------------------------------------------------
    def save_checkpoint(self, model, engine, epoch, float_dtype: torch.dtype = torch.bfloat16) -> None:
        """``engine`` is a ``TrainEngine`` (or ``None`` for a model-only save).  The
        model is written from the fp32 master weights cast to ``float_dtype``."""
        target = self.path / str(epoch)
        state = {k: v.detach() for k, v in _unwrap(model).state_dict().items()}
        opt_state = None
        if engine is not None:
            for name, tensor in engine.master_state_dict().items():  # collective in sharded mode
                _assign_master(state, name, tensor)
            opt_state = engine.optimizer_state_dict(first_rank_only=True)  # collective in sharded mode
        if _is_rank0():
            target.mkdir(parents=True, exist_ok=True)
            inner = _unwrap(model)
            tensors = {k: (v.to(float_dtype) if v.is_floating_point() else v) for k, v in state.items()}
            inner.save_pretrained(target, state_dict=tensors)
            patch_config_dtype(target, float_dtype)
            if opt_state is not None:
                torch.save(convert_float_dtype(opt_state, float_dtype), self.optimizer_path(epoch))
            src = self.path / TRAIN_COMMAND_FILENAME
            if src.exists():
                shutil.copy2(src, target / TRAIN_COMMAND_FILENAME)
        _barrier()

    def save_scheduler_state_dict(self, schedulers, epoch) -> None:
        if _is_rank0():
            items = schedulers if isinstance(schedulers, (list, tuple)) else [schedulers]
            states = [s.state_dict() for s in items]
            self.scheduler_path(epoch).parent.mkdir(parents=True, exist_ok=True)
            torch.save(states[0] if len(states) == 1 else states, self.scheduler_path(epoch))
        _barrier()

    def save_val_metrics(self, epoch: int, val_metrics: dict[str, float]) -> None:
        if _is_rank0():
            path = self.val_metrics_path(epoch)
            path.parent.mkdir(parents=True, exist_ok=True)
            path.write_text(json.dumps(val_metrics))
        _barrier()

    # ---- load ------------------------------------------------------------------
    def load_model_state_dict(self, model, float_dtype: torch.dtype | None = None) -> None:
        sd = load_safetensors_state_dict(self.model_path(self.previous_epoch))
        if float_dtype is not None:
            sd = convert_float_dtype(sd, float_dtype)
        # verifier-derived weights are not in the file; strict=False keeps what is loaded
        _unwrap(model).load_state_dict(sd, strict=False)

    def load_model_state_dict_for_epoch(self, model, epoch: int, float_dtype: torch.dtype | None = None) -> None:
        previous = self.previous_epoch
        try:
            self.previous_epoch = epoch
            self.load_model_state_dict(model, float_dtype=float_dtype)
        finally:
            self.previous_epoch = previous

    def load_optimizer_state_dict(self, model, engine, float_dtype: torch.dtype | None = None) -> None:
        del model
        path = self.optimizer_path(self.previous_epoch)
        if not path.exists():
            log.warning("No optimizer state at %s; the optimizer starts fresh.", path)
            return
        sd = torch.load(path, weights_only=True, map_location="cpu")
        engine.load_optimizer_state_dict(convert_float_dtype(sd, float_dtype or torch.float32))

    def load_scheduler_state_dict(self, schedulers) -> None:
        path = self.scheduler_path(self.previous_epoch)
        if not path.exists():
            return
        loaded = torch.load(path, weights_only=True)
        items = schedulers if isinstance(schedulers, (list, tuple)) else [schedulers]
        states = loaded if isinstance(loaded, list) else [loaded]
        for sched, state in zip(items, states, strict=True):
            sched.load_state_dict(state)

    # ---- best-epoch bookkeeping ------------------------------------------------------
    def read_best_epoch(self) -> int | None:
        link = self.best_path()
        if not link.is_symlink():
            return None
        try:
            return int(Path(link.readlink()).name)
        except (OSError, ValueError):
            return None

    def load_best_val_loss(self) -> float | None:
        best = self.read_best_epoch()
        if best is None:
            return None
        path = self.val_metrics_path(best)
        try:
            return float(json.loads(path.read_text())["loss_epoch"])
        except (OSError, json.JSONDecodeError, KeyError, ValueError, TypeError):
            return None

    def update_best_symlink(self, epoch: int) -> None:
        if _is_rank0():
            link = self.best_path()
            if link.is_symlink() or link.is_file():
                link.unlink()
            elif link.is_dir():
                shutil.rmtree(link)
            link.symlink_to(Path(str(epoch)), target_is_directory=True)
        _barrier()

    def cleanup_keep_only_best(self, best_epoch: int) -> None:
        """Delete everything under the save path except the best epoch directory,
        the ``checkpoint_best`` link and the run-level ``train_command.txt``."""
        if _is_rank0():
            keep = self.path / str(best_epoch)
            if not keep.is_dir():
                raise FileNotFoundError(f"Best epoch dir does not exist: {keep}")
            protected = {keep, self.best_path(), self.path / TRAIN_COMMAND_FILENAME}
            for child in self.path.iterdir():
                if child in protected:
                    continue
                try:
                    if child.is_symlink() or child.is_file():
                        child.unlink()
                    elif child.is_dir():
                        shutil.rmtree(child)
                except OSError as exc:
                    raise RuntimeError(f"Failed to delete {child}") from exc
        _barrier()


def _unwrap(model):
    return getattr(model, "module", model)


def _assign_master(state: dict, param_name: str, tensor: torch.Tensor) -> None:
    """Route a master tensor (keyed by parameter name, fused layout) into a
    ``state_dict`` whose fused projections were split by the save hook."""
    if param_name in state:
        state[param_name] = tensor
        return
    for fused, parts in (("qkv_proj", ("q_proj", "k_proj", "v_proj")), ("gate_up_proj", ("gate_proj", "up_proj")), ("kv_proj", ("k_proj", "v_proj"))):
        token = f".{fused}."
        if token not in param_name and not param_name.startswith(fused + "."):
            continue
        off = 0
        for part in parts:
            key = param_name.replace(fused, part, 1) if token not in param_name else param_name.replace(token, f".{part}.")
            if key not in state:
                return
            rows = state[key].shape[0]
            state[key] = tensor[off : off + rows]
            off += rows
        return


BaseCheckpointer = Checkpointer
SingleGPUCheckpointer = Checkpointer
DistributedCheckpointer = Checkpointer
