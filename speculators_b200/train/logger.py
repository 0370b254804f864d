"""Console and metric logging.

Two logger names, as in the reference (src/speculators/train/logger.py:624-738):

* ``speculators``          : human-readable log lines (Rich console when available),
  rank 0 only unless a record carries ``extra={"override_rank0_filter": True}``;
* ``speculators.metrics``  : dict payloads.  Every record whose message is a mapping
  fans out to the configured backends (``tensorboard``, ``wandb``, ``trackio``,
  ``mlflow``; imported lazily, so an unused backend is not a dependency).
  ``extra={"step": n}`` sets the x-axis, ``extra={"hparams": True}`` marks a
  hyper-parameter record.

Run names accept the placeholders ``{time}``, ``{utc_time}``, ``{rank}``,
``{local_rank}``.
"""

from __future__ import annotations

import json
import logging
import numbers
import os
from collections.abc import Mapping
from datetime import datetime, timezone
from pathlib import Path
from typing import Any

import torch

__all__ = [
    "FormatDictFilter", "IsMappingFilter", "IsRank0Filter", "MLFlowHandler", "TensorBoardHandler", "TrackioHandler",
    "WandbHandler", "log_run_config", "setup_metric_logger", "setup_root_logger",
]


def _substitute_placeholders(run_name: str | None, default_template: str = "{time}") -> str:
    name = default_template if run_name is None else run_name
    values = {
        "{time}": datetime.now().isoformat(timespec="seconds"),
        "{utc_time}": datetime.now(timezone.utc).isoformat(timespec="seconds"),
        "{rank}": int(os.environ.get("RANK", "0")),
        "{local_rank}": int(os.environ.get("LOCAL_RANK", "0")),
    }
    for key, value in values.items():
        name = name.replace(key, str(value))
    return name


def _flatten_dict(d: Mapping, sep: str = "/", prefix: str = "") -> dict[str, Any]:
    flat: dict[str, Any] = {}
    for key, value in d.items():
        path = f"{prefix}{sep}{key}" if prefix else str(key)
        if isinstance(value, Mapping):
            flat.update(_flatten_dict(value, sep, path))
        else:
            flat[path] = value
    return flat


def _scalars(d: Mapping) -> dict[str, float]:
    out = {}
    for key, value in _flatten_dict(d).items():
        if isinstance(value, bool):
            out[key] = float(value)
        elif isinstance(value, numbers.Number):
            out[key] = float(value)
        elif hasattr(value, "item") and getattr(value, "numel", lambda: 2)() == 1:
            out[key] = float(value.item())
    return out


class IsMappingFilter(logging.Filter):
    def filter(self, record: logging.LogRecord) -> bool:
        return isinstance(record.msg, Mapping)


class IsRank0Filter(logging.Filter):
    """Pass records only on (local) rank 0; ``extra={"override_rank0_filter": True}``
    lets a record through on every rank."""

    def __init__(self, rank_val: int | None = None, local_rank: bool = False):
        super().__init__()
        self.rank_val, self.local_rank = rank_val, local_rank

    def _rank(self) -> int:
        if self.rank_val is not None:
            return self.rank_val
        if not self.local_rank:
            from speculators_b200.parallel.distributed import get_training_group, training_rank

            if get_training_group() is not None:  # the training ranks are a sub-group of the job: its first rank speaks
                return training_rank()
        return int(os.environ.get("LOCAL_RANK" if self.local_rank else "RANK", "0"))

    def filter(self, record: logging.LogRecord) -> bool:
        return bool(getattr(record, "override_rank0_filter", False)) or self._rank() == 0


class FormatDictFilter(logging.Filter):
    """Render mapping messages as aligned ``key: value`` lines for the console."""

    @staticmethod
    def _fmt(v: Any) -> str:
        if isinstance(v, float):
            return f"{v:.6g}"
        return str(v)

    def filter(self, record: logging.LogRecord) -> bool:
        if isinstance(record.msg, Mapping):
            flat = _flatten_dict(record.msg)
            record.msg = "\n".join(f"  {k}: {self._fmt(v)}" for k, v in flat.items())
            record.args = None
        return True


class _LazyHandler(logging.Handler):
    def __init__(self, log_dir: str | os.PathLike = "logs", run_name: str | None = None):
        super().__init__()
        self.log_dir = Path(log_dir)
        self.run_name = _substitute_placeholders(run_name)
        self._ready = False

    def _setup(self) -> None:
        raise NotImplementedError

    def _ensure(self) -> None:
        if not self._ready:
            self._setup()
            self._ready = True


# hyper-parameter values TensorBoard's hparams plugin takes as they are; anything else (lists,
# nested dicts) is JSON-encoded before it is handed over
TB_SUPPORTED_TYPES = (int, float, str, bool, torch.Tensor, type(None))


class TensorBoardHandler(_LazyHandler):
    def _setup(self) -> None:
        from torch.utils.tensorboard import SummaryWriter

        self.writer = SummaryWriter(log_dir=str(self.log_dir / self.run_name))

    def emit(self, record: logging.LogRecord) -> None:
        if not isinstance(record.msg, Mapping):
            return
        self._ensure()
        if getattr(record, "hparams", False):
            flat = _flatten_dict(record.msg)
            self.writer.add_text("hparams", "\n".join(f"    {k}: {v}" for k, v in flat.items()))
            self.writer.add_hparams(self._scalarise(flat), {}, run_name=".")  # the hparams tab of the same run
            return
        step = getattr(record, "step", None)
        for key, value in _scalars(record.msg).items():
            self.writer.add_scalar(key, value, global_step=step)

    @staticmethod
    def _scalarise(d: Mapping) -> dict:
        return {k: (v if isinstance(v, TB_SUPPORTED_TYPES) else json.dumps(v, default=str)) for k, v in d.items()}

    def flush(self) -> None:
        if self._ready:
            self.writer.flush()

    def close(self) -> None:
        if self._ready:
            self.writer.close()
        super().close()


class WandbHandler(_LazyHandler):
    _module = "wandb"

    def _setup(self) -> None:
        import importlib

        self._backend = importlib.import_module(self._module)
        self._run = self._backend.init(dir=str(self.log_dir), name=self.run_name, project=os.environ.get("WANDB_PROJECT", "speculators"))

    def emit(self, record: logging.LogRecord) -> None:
        if not isinstance(record.msg, Mapping):
            return
        self._ensure()
        if getattr(record, "hparams", False):
            try:
                self._run.config.update(_flatten_dict(record.msg), allow_val_change=True)
            except Exception:  # noqa: BLE001
                pass
            return
        self._backend.log(_scalars(record.msg), step=getattr(record, "step", None))


class TrackioHandler(WandbHandler):
    _module = "trackio"

    def _setup(self) -> None:
        import importlib

        self._backend = importlib.import_module(self._module)
        self._run = self._backend.init(project=os.environ.get("TRACKIO_PROJECT", "speculators"), name=self.run_name)


class MLFlowHandler(_LazyHandler):
    def _setup(self) -> None:
        import mlflow

        self._mlflow = mlflow
        if uri := os.environ.get("MLFLOW_TRACKING_URI"):
            mlflow.set_tracking_uri(uri)
        else:
            mlflow.set_tracking_uri(f"file://{(self.log_dir / 'mlruns').resolve()}")
        mlflow.set_experiment(os.environ.get("MLFLOW_EXPERIMENT_NAME", "speculators"))
        self._run = mlflow.start_run(run_name=self.run_name)

    def emit(self, record: logging.LogRecord) -> None:
        if not isinstance(record.msg, Mapping):
            return
        self._ensure()
        if getattr(record, "hparams", False):
            params = {k: str(v)[:500] for k, v in _flatten_dict(record.msg).items()}
            self._mlflow.log_params(params)
            return
        clean = {k.replace("/", "."): v for k, v in _scalars(record.msg).items()}
        self._mlflow.log_metrics(clean, step=getattr(record, "step", None))

    def close(self) -> None:
        if self._ready:
            self._mlflow.end_run()
        super().close()


_HANDLERS = {"tensorboard": TensorBoardHandler, "wandb": WandbHandler, "trackio": TrackioHandler, "mlflow": MLFlowHandler}


def setup_root_logger(level: str | int = "INFO") -> None:
    try:
        from rich.logging import RichHandler

        handler: logging.Handler = RichHandler()
    except ImportError:
        handler = logging.StreamHandler()
    handler.addFilter(FormatDictFilter())
    handler.addFilter(IsRank0Filter())
    logging.basicConfig(level=level, format="%(message)s", datefmt="[%X]", handlers=[handler], force=True)
    logging.getLogger("httpx").propagate = False


def setup_metric_logger(loggers, run_name, output_dir) -> None:
    """``loggers``: comma-separated string or list of backend names ("" = console only)."""
    if isinstance(loggers, str):
        loggers = [part.strip() for part in loggers.split(",") if part.strip()]
    unknown = [name for name in loggers if name not in _HANDLERS]
    if unknown:
        raise ValueError(f"unknown metric logger(s) {unknown}; choose from {sorted(_HANDLERS)}")
    metrics = logging.getLogger("speculators.metrics")
    for old in list(metrics.handlers):
        if isinstance(old, _LazyHandler):
            metrics.removeHandler(old)
            old.close()
    if not any(isinstance(f, IsMappingFilter) for f in metrics.filters):
        metrics.addFilter(IsMappingFilter())
    for name in loggers:
        handler = _HANDLERS[name](log_dir=output_dir, run_name=run_name)
        handler.addFilter(IsMappingFilter())
        handler.addFilter(IsRank0Filter())
        metrics.addHandler(handler)
    metrics.setLevel(logging.INFO)
    metrics.propagate = True
    logging.getLogger("speculators").setLevel(logging.INFO)


def log_run_config(cfg) -> None:
    resolved = cfg.model_dump(mode="json")
    if getattr(cfg, "backend_args", None):
        resolved["hidden_states_backend_args"] = dict(cfg.backend_args)
    logging.getLogger("speculators.metrics").info(resolved, extra={"hparams": True})
