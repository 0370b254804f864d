"""Torch helpers for data generation.

Reference surface: src/speculators/data_generation/torch_utils.py:13.
"""

from __future__ import annotations

import contextlib
import os

import torch

__all__ = ["set_default_torch_num_threads"]


@contextlib.contextmanager
def set_default_torch_num_threads(num_threads: int | None = None):
    """Temporarily pin torch's intra-op thread count.  ``None`` takes
    ``OMP_NUM_THREADS`` (1 when unset or not an integer), which keeps multimodal
    preprocessing workers from oversubscribing the host cores."""
    if num_threads is None:
        try:
            num_threads = int(os.environ.get("OMP_NUM_THREADS", "1"))
        except ValueError:
            num_threads = 1
    before = torch.get_num_threads()
    torch.set_num_threads(max(1, num_threads))
    try:
        yield
    finally:
        torch.set_num_threads(before)
