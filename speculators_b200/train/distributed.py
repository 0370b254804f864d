"""Process-topology helpers under the reference's module path
(src/speculators/train/distributed.py).  The implementation lives in
``speculators_b200.parallel``; sharded training is done by ``TrainEngine`` (flat buffers,
sharded optimizer state), so ``apply_fully_sharded`` only marks the model for it."""

from __future__ import annotations

import torch

from speculators_b200.parallel.distributed import (
    get_dp_group, get_dp_rank, get_dp_size, get_local_rank, get_rank, get_sp_group, get_sp_rank, get_sp_size, get_world_size,
    is_distributed, maybe_destroy_distributed, maybe_setup_distributed,
)

__all__ = [
    "apply_fully_sharded", "get_dp_group", "get_dp_rank", "get_dp_size", "get_local_rank", "get_rank", "get_sp_group", "get_sp_rank",
    "get_sp_size", "get_world_size", "is_distributed", "maybe_destroy_distributed", "maybe_setup_distributed",
]


def apply_fully_sharded(model: torch.nn.Module, param_dtype: torch.dtype = torch.bfloat16) -> torch.nn.Module:
    """Request sharded training for ``model``.  The reference wraps every decoder layer in
    FSDP2 here; in this package the ``Trainer`` builds a ``TrainEngine`` that shards the fp32
    master weights and optimizer state over the data-parallel group and keeps the
    ``param_dtype`` compute weights resident, so the model is returned unwrapped with the
    request recorded on it (``TrainerConfig.fsdp_shard`` / ``--fsdp-shard`` is the usual way
    to ask for the same thing)."""
    model._sb200_shard_request = {"param_dtype": param_dtype}  # noqa: SLF001 - read by Trainer
    return model
