"""Reproducibility artifacts written next to the checkpoints: ``run.yaml`` (the
resolved config, re-loadable with ``--config``) and ``train_command.txt``.

Only values supplied by a flag or the YAML file are emitted (defaults are
re-derived on reload): persisting materialised defaults would make a
``--from-pretrained`` run reject its own ``run.yaml``, because YAML-supplied
decoder-shaping keys count as explicit.  Parity:
src/speculators/train/config/artifacts.py:18-84."""

from __future__ import annotations

from pathlib import Path

import yaml

from speculators_b200.train.config.schema import TrainConfig, nest_flat

__all__ = ["dump_yaml", "save"]


def dump_yaml(cfg: TrainConfig) -> str:
    from speculators_b200.train.config.resolution import BACKEND_DESTS

    resolved = cfg.flatten()
    if cfg.provenance:
        provided = {d: v for d, v in resolved.items() if cfg.provenance.get(d, "default") != "default"}
    else:  # built off-argv (from_flat): "customised" = differs from a default-constructed config
        baseline = type(cfg)().flatten()
        provided = {d: v for d, v in resolved.items() if v != baseline.get(d)}
    nested = nest_flat({k: v for k, v in provided.items() if k not in BACKEND_DESTS})
    backend = {k: v for k, v in provided.items() if k in BACKEND_DESTS}
    if backend:
        nested["backend"] = backend
    return yaml.safe_dump({"train": nested}, sort_keys=False, default_flow_style=False)


def save(cfg: TrainConfig, save_dir: str) -> None:
    from speculators_b200.train.utils import save_train_command

    out = Path(save_dir)
    out.mkdir(parents=True, exist_ok=True)
    (out / "run.yaml").write_text(dump_yaml(cfg))
    save_train_command(save_dir, argv=list(cfg.argv) or None)
