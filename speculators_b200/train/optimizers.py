"""Optimizer construction.

The reference returns ``[AdamW]`` or ``[Muon, AdamW]`` torch optimizers
(src/speculators/train/optimizers.py:61-110).  Here the optimizer, mixed precision and
the data-parallel reduction are one object, ``TrainEngine`` (flat bf16 weight / gradient
buffers, fp32 master weights and moments, fused AdamW, Newton-Schulz Muon for the matrix
region); ``build_optimizers`` builds it from a ``TrainerConfig`` and returns it in a list
so callers written against the reference's API (``for opt in optimizers: opt.step()``)
keep their shape.
"""

from __future__ import annotations

import torch
from torch import nn

from speculators_b200.parallel.engine import EngineConfig, TrainEngine, split_named_params_for_muon

__all__ = ["build_optimizers", "engine_config_from_trainer_config", "split_named_params_for_muon"]


def engine_config_from_trainer_config(config, compute_dtype: torch.dtype = torch.bfloat16) -> EngineConfig:
    if config.optimizer not in ("adamw", "muon"):
        raise ValueError(f"Unsupported optimizer: {config.optimizer!r}")
    return EngineConfig(
        lr=config.lr, weight_decay=config.weight_decay, max_grad_norm=getattr(config, "max_grad_norm", 1.0), optimizer=config.optimizer,
        muon_lr=config.muon_lr, muon_momentum=config.muon_momentum, muon_weight_decay=config.muon_weight_decay,
        muon_ns_steps=config.muon_ns_steps, muon_adjust_lr_fn=config.muon_adjust_lr_fn, compute_dtype=compute_dtype,
        shard=bool(getattr(config, "fsdp_shard", False)),
    )


def build_optimizers(model: nn.Module, config, device: torch.device | str | None = None,
                     compute_dtype: torch.dtype | None = None) -> list[TrainEngine]:
    """``[TrainEngine]`` for ``config.optimizer`` in {"adamw", "muon"}.  Raises
    ``ValueError`` for another name or a model without trainable parameters."""
    dev = torch.device(device) if device is not None else next(model.parameters()).device
    if compute_dtype is None:
        compute_dtype = torch.bfloat16 if dev.type == "cuda" else torch.float32
    return [TrainEngine(model, engine_config_from_trainer_config(config, compute_dtype), device=dev)]
