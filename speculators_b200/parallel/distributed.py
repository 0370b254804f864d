"""Process topology: one process per GPU, ``torch.distributed`` for the plumbing.

``maybe_setup_distributed`` is a no-op outside ``torchrun`` (``LOCAL_RANK`` unset).
Under ``torchrun`` it binds the process to its GPU, initialises the default group
(NCCL over NVLink on CUDA, gloo on CPU) and creates the data-parallel and
sequence-parallel sub-groups: SP groups are contiguous ranks, DP groups are strided
(``sp_size=2, world=4``: SP {0,1},{2,3}; DP {0,2},{1,3}).  Getter names match
src/speculators/train/distributed.py:43-80 so call sites port unchanged.
"""

from __future__ import annotations

import datetime
import logging
import os

import torch
import torch.distributed as dist

log = logging.getLogger("speculators")

__all__ = [
    "get_dp_group", "get_dp_rank", "get_dp_size", "get_local_rank", "get_rank", "get_sp_group",
    "get_sp_rank", "get_sp_size", "get_world_size", "is_distributed", "maybe_destroy_distributed",
    "maybe_setup_distributed",
]


class _Topology:
    def __init__(self) -> None:
        self.reset()

    def reset(self) -> None:
        self.local_rank = 0
        self.rank = 0
        self.world_size = 1
        self.distributed = False
        self.sp_size = 1
        self.sp_rank = 0
        self.dp_size = 1
        self.dp_rank = 0
        self.sp_group = None
        self.dp_group = None
        self.train_group = None  # the ranks that train, when they are a sub-group of the job (online verifier / trainer split)


_T = _Topology()


def get_local_rank() -> int:
    return _T.local_rank


def get_rank() -> int:
    return _T.rank


def get_world_size() -> int:
    return _T.world_size


def is_distributed() -> bool:
    return _T.distributed


def set_training_group(group) -> None:
    """Declare the process group of the training ranks when other ranks of the job do something else (run
    the verifier): "rank 0" duties (checkpoint files, progress bar, metric sinks) and the barriers around
    them then refer to this group."""
    _T.train_group = group


def get_training_group():
    return _T.train_group


def training_rank() -> int:
    """Rank inside the training group (the job's rank when none is declared); -1 outside of it."""
    if _T.train_group is None or not (dist.is_available() and dist.is_initialized()):
        return dist.get_rank() if (dist.is_available() and dist.is_initialized()) else _T.rank
    return dist.get_rank(_T.train_group)


def training_barrier() -> None:
    if not (dist.is_available() and dist.is_initialized()):
        return
    if _T.train_group is None:
        dist.barrier()
    elif dist.get_rank(_T.train_group) >= 0:
        dist.barrier(group=_T.train_group)


def get_sp_group():
    return _T.sp_group


def get_dp_group():
    return _T.dp_group


def get_sp_size() -> int:
    return _T.sp_size


def get_sp_rank() -> int:
    return _T.sp_rank


def get_dp_size() -> int:
    return _T.dp_size


def get_dp_rank() -> int:
    return _T.dp_rank


def _init_sp_process_groups(rank: int, world_size: int, sp_size: int) -> None:
    if sp_size <= 0:
        raise ValueError(f"sp_size must be positive, got {sp_size}")
    if world_size % sp_size:
        raise ValueError(f"world_size ({world_size}) must be divisible by sp_size ({sp_size})")
    dp_size = world_size // sp_size
    mine_sp = mine_dp = None
    for block in range(dp_size):  # every rank creates every group, in the same order
        members = list(range(block * sp_size, (block + 1) * sp_size))
        group = dist.new_group(members)
        if rank in members:
            mine_sp = group
    for lane in range(sp_size):
        members = list(range(lane, world_size, sp_size))
        group = dist.new_group(members)
        if rank in members:
            mine_dp = group
    if mine_sp is None or mine_dp is None:
        raise RuntimeError("Failed to initialize SP/DP process groups")
    _T.sp_group, _T.dp_group = mine_sp, mine_dp
    _T.sp_size, _T.sp_rank = sp_size, rank % sp_size
    _T.dp_size, _T.dp_rank = dp_size, rank // sp_size


def maybe_setup_distributed(sp_size: int = 1, backend: str | None = None, timeout_s: float | None = None) -> None:
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    _T.local_rank = local_rank
    _T.distributed = "LOCAL_RANK" in os.environ
    if not _T.distributed:
        return
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    if use_cuda:
        torch.cuda.set_device(local_rank)
    backend = backend or ("nccl" if use_cuda else "gloo")
    kwargs = {}
    if timeout_s is not None:
        kwargs["timeout"] = datetime.timedelta(seconds=timeout_s)
    if use_cuda:
        kwargs["device_id"] = torch.device("cuda", local_rank)
    if not dist.is_initialized():
        dist.init_process_group(backend, **kwargs)
    _T.rank, _T.world_size = dist.get_rank(), dist.get_world_size()
    _init_sp_process_groups(_T.rank, _T.world_size, sp_size)
    log.info(
        "Started distributed with local_rank=%d, dp_size=%d, sp_size=%d", local_rank, _T.dp_size, _T.sp_size,
        extra={"override_rank0_filter": True},
    )


def maybe_destroy_distributed() -> None:
    if not _T.distributed:
        return
    if dist.is_initialized():
        dist.destroy_process_group()
    log.info("Destroyed distributed process group", extra={"override_rank0_filter": True})
    _T.reset()
