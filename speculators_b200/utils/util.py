"""Small device helpers (parity: src/speculators/utils/util.py).  This framework
targets CUDA (B200) with a CPU path for tests; there is no NPU branch."""

from __future__ import annotations

import contextlib
import os

import torch

__all__ = ["empty_cache", "get_current_device", "get_device_name", "is_npu_available", "mem_get_info", "nvtx_range"]


def is_npu_available() -> bool:
    """Ascend NPUs are not a target of this package (sm_100a only): always False.  Kept so that
    code written against the reference's helper keeps importing."""
    return False


def get_device_name() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def get_current_device() -> torch.device:
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    return torch.device("cpu")


def mem_get_info() -> tuple[int, int]:
    if torch.cuda.is_available():
        return torch.cuda.mem_get_info()
    import psutil

    vm = psutil.virtual_memory()
    return vm.available, vm.total


def empty_cache() -> None:
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


NVTX_ENABLED = os.environ.get("SB200_NVTX", "0") == "1"


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range around a phase of the step (``SB200_NVTX=1``; a no-op otherwise and on
    machines without CUDA), so that a timeline capture shows fetch / forward / backward /
    optimizer / collective phases by name."""
    active = NVTX_ENABLED and torch.cuda.is_available()
    if active:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if active:
            torch.cuda.nvtx.range_pop()
