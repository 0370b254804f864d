"""DataLoader factory: train / validation ``ArrowDataset`` splits, multipack
sampler over the data-parallel ranks, packing collate, pinned memory, spawned
persistent workers (src/speculators/train/dataloader.py:31-168)."""

from __future__ import annotations

import os
from collections.abc import Callable
from typing import Literal

import torch
from torch.utils.data import DataLoader

from speculators_b200.hs_connectors import HiddenStatesTransfer
from speculators_b200.parallel.distributed import get_dp_rank, get_dp_size
from speculators_b200.train.data import ArrowDataset, BaseDataset, BatchType, CollateFn
from speculators_b200.train.distributed_batch_sampler import MultipackDistributedBatchSamplerV2
from speculators_b200.train.noise_transforms import AddUniformNoise

__all__ = ["create_train_val_loaders", "setup_dataloader"]


def _limit_worker_threads() -> None:
    """Workers only do I/O and slicing; one thread each avoids oversubscription.
    Must run before numpy / torch are imported in the workers to take effect."""
    for var in ("OPENBLAS_NUM_THREADS", "OMP_NUM_THREADS", "MKL_NUM_THREADS"):
        os.environ.setdefault(var, "1")


def _worker_init_fn(worker_id: int) -> None:  # noqa: ARG001
    torch.set_num_threads(1)


def setup_dataloader(dataset: BaseDataset, total_seq_len: int, hidden_size: int, num_workers: int = 12, num_target_layers: int = 3,
                     prefetch_factor: int | None = 4, preprocess: Callable[[BatchType], BatchType] | None = None) -> DataLoader:
    sampler = MultipackDistributedBatchSamplerV2(
        batch_max_length=total_seq_len, lengths=dataset.approx_lengths, num_replicas=get_dp_size(), rank=get_dp_rank()
    )
    workers = num_workers > 0
    return DataLoader(
        dataset, batch_sampler=sampler, num_workers=num_workers, prefetch_factor=prefetch_factor if workers else None,
        pin_memory=torch.cuda.is_available(),
        collate_fn=CollateFn(total_seq_len, hidden_size, num_target_layers=num_target_layers, dtype=dataset.hidden_states_dtype, preprocess=preprocess),
        persistent_workers=workers, multiprocessing_context="spawn" if workers else None,
        worker_init_fn=_worker_init_fn if workers else None,
    )


def create_train_val_loaders(*, data_path: str, total_seq_len: int, hidden_states_dtype: torch.dtype, noise_std: float,
                             transfer: HiddenStatesTransfer | None = None, vllm_endpoint: str,
                             on_missing: Literal["generate", "skip", "warn", "raise"], on_generate: Literal["cache", "delete"],
                             verifier_name_or_path: str, request_timeout: float | None, max_retries: int, hidden_size: int,
                             num_target_layers: int, num_workers: int, prefetch_factor: int,
                             preprocess: Callable[[BatchType], BatchType] | None, train_data_ratio: float = 0.9):
    _limit_worker_threads()
    if not 0.0 < train_data_ratio < 1.0:
        raise ValueError(f"train_data_ratio must be in (0, 1), got {train_data_ratio}")
    common = dict(datapath=data_path, max_len=total_seq_len, transfer=transfer, vllm_endpoint=vllm_endpoint, on_missing=on_missing,
                  on_generate=on_generate, train_ratio=train_data_ratio, model=verifier_name_or_path,
                  hidden_states_dtype=hidden_states_dtype, request_timeout=request_timeout, max_retries=max_retries)
    train = ArrowDataset(split="train", transform=AddUniformNoise(std=noise_std), **common)
    val = ArrowDataset(split="val", **common)
    kw = dict(num_target_layers=num_target_layers, num_workers=num_workers, prefetch_factor=prefetch_factor, preprocess=preprocess)
    return setup_dataloader(train, total_seq_len, hidden_size, **kw), setup_dataloader(val, total_seq_len, hidden_size, **kw)
