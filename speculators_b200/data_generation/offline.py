"""Helpers for offline hidden-state generation: payload validation, resume by
existing files, per-node index split (src/speculators/data_generation/offline.py)."""

from __future__ import annotations

import logging
import re
from pathlib import Path

import torch

log = logging.getLogger(__name__)

__all__ = ["check_hidden_states", "get_existing_hidden_state_indices", "get_indices_to_process"]

_ROWS_PER_CHUNK = 256
_HS_FILE = re.compile(r"^hs_(\d+)\.safetensors$")


def check_hidden_states(data: dict, tokens: list[int]) -> None:
    """Raise ``ValueError`` unless ``data`` holds ``token_ids`` equal to ``tokens`` and
    finite ``hidden_states`` with one row per token.  The finite scan walks 256 rows
    at a time so no full-size boolean temporary is created for long samples."""
    missing = {"token_ids", "hidden_states"} - data.keys()
    if missing:
        raise ValueError(f"Hidden-state payload is missing keys: {missing}")
    if data["token_ids"].tolist() != list(tokens):
        raise ValueError(f"Token ids don't match expected token ids {tokens}")
    hs = data["hidden_states"]
    if not isinstance(hs, torch.Tensor):
        raise ValueError(f"Hidden states must be a tensor, got {type(hs).__name__}")
    if hs.shape[0] != len(tokens):
        raise ValueError(f"Sequence length of hidden states {hs.shape[0]} doesn't match num tokens {len(tokens)}")
    nans = infs = 0
    bad_layers: set[int] = set()
    for start in range(0, hs.shape[0], _ROWS_PER_CHUNK):
        chunk = hs[start : start + _ROWS_PER_CHUNK]
        finite = torch.isfinite(chunk)
        if bool(finite.all()):
            continue
        nans += int(torch.isnan(chunk).sum())
        infs += int(torch.isinf(chunk).sum())
        if hs.ndim >= 3:
            bad_layers.update((~finite).flatten(start_dim=2).any(dim=(0, 2)).nonzero().flatten().tolist())
    if nans or infs:
        details = f"shape={tuple(hs.shape)}, dtype={hs.dtype}, nan_count={nans}, inf_count={infs}"
        if bad_layers:
            details += f", affected layer slots={sorted(bad_layers)}"
        raise ValueError(f"Hidden states contain non-finite values ({details})")


def get_existing_hidden_state_indices(output_path: Path) -> list[int]:
    if not Path(output_path).exists():
        return []
    found = {int(m.group(1)) for p in Path(output_path).iterdir() if (m := _HS_FILE.match(p.name))}
    return sorted(found)


def get_indices_to_process(num_samples: int, max_samples: int | None, existing: list[int], world_size: int, rank: int) -> list[int]:
    """Contiguous share of ``[0, target)`` for ``rank`` (earlier ranks take the
    remainder), minus indices that already have a file."""
    target = min(max_samples, num_samples) if max_samples is not None else num_samples
    if target <= 0:
        return []
    base, rem = divmod(target, world_size)
    start = rank * base + min(rank, rem)
    end = start + base + (1 if rank < rem else 0)
    done = set(existing)
    todo = [i for i in range(start, end) if i not in done]
    already = len(done & set(range(start, end)))
    if not todo:
        log.info("All samples for this rank already processed!")
    elif already:
        log.info("Found %d existing samples for rank %d.", already, rank)
    return todo


# --------------------------------------------------------------------------- async runner
import asyncio  # noqa: E402
import shutil  # noqa: E402
import time  # noqa: E402
from dataclasses import dataclass, field  # noqa: E402
from typing import Any, Awaitable, Callable  # noqa: E402

__all__ += ["OfflineRunConfig", "OfflineRunStats", "run_offline_generation"]


@dataclass
class OfflineRunConfig:
    """Knobs of one offline run (scripts/data_generation_offline.py:58 of the
    reference lists the same CLI surface)."""

    output_dir: Path
    concurrency: int = 32
    validate_outputs: bool = False
    request_timeout: float | None = 120.0
    max_retries: int = 3
    fail_on_error: bool = False
    max_consecutive_errors: int | None = None  # default: concurrency


@dataclass
class OfflineRunStats:
    ok: int = 0
    errors: int = 0
    request_s: float = 0.0
    write_s: float = 0.0
    skipped: list[int] = field(default_factory=list)
    elapsed_s: float = 0.0

    def summary(self) -> str:
        if not self.ok:
            return f"0 samples saved, {self.errors} errors in {self.elapsed_s:.1f}s"
        return (
            f"{self.ok} samples in {self.elapsed_s:.1f}s ({self.ok / max(self.elapsed_s, 1e-9):.1f}/s), "
            f"avg request {self.request_s / self.ok * 1e3:.0f} ms, avg file move {self.write_s / self.ok * 1e3:.0f} ms, "
            f"{self.errors} errors"
        )


class ConsecutiveFailureAbort(RuntimeError):
    """Too many samples in a row failed after their retries: the server is probably down."""


async def run_offline_generation(
    indices: list[int],
    make_item: Callable[[int], dict],
    request: Callable[[dict], Awaitable[str]],
    cfg: OfflineRunConfig,
    on_progress: Callable[[OfflineRunStats], None] | None = None,
) -> OfflineRunStats:
    """Fetch hidden states for ``indices`` and file them as ``hs_<idx>.safetensors``.

    ``request(item)`` performs one extraction (with its own retries) and returns the
    path the server wrote; a sliding window of ``concurrency`` requests is kept in
    flight (samples are materialised only when a slot frees up, so memory stays
    bounded).  A failed sample is recorded and skipped, unless ``fail_on_error`` (the
    first failure is re-raised) or ``max_consecutive_errors`` failures happen without a
    success in between (``ConsecutiveFailureAbort``; pending requests are cancelled).
    """
    from speculators_b200.hs_connectors.transfer import wait_for_lock

    out_dir = Path(cfg.output_dir)
    out_dir.mkdir(parents=True, exist_ok=True)
    stats = OfflineRunStats()
    t0 = time.perf_counter()
    limit = cfg.max_consecutive_errors if cfg.max_consecutive_errors is not None else cfg.concurrency
    streak = 0

    async def one(idx: int) -> tuple[float, float]:
        item = make_item(idx)
        t_req = time.perf_counter()
        src = await request(item)
        t_req = time.perf_counter() - t_req
        lock = src + ".lock"
        if Path(lock).exists():  # the producer still holds the file
            await asyncio.to_thread(wait_for_lock, lock)
        dst = out_dir / f"hs_{idx}.safetensors"
        t_wr = time.perf_counter()
        await asyncio.to_thread(shutil.move, src, dst)
        t_wr = time.perf_counter() - t_wr
        if cfg.validate_outputs:
            def verify():
                from safetensors.torch import load_file

                check_hidden_states(load_file(dst), item["input_ids"])

            await asyncio.to_thread(verify)
        return t_req, t_wr

    pending: dict[asyncio.Task, int] = {}
    todo = iter(indices)
    exhausted = False
    try:
        while True:
            while not exhausted and len(pending) < max(1, cfg.concurrency):
                idx = next(todo, None)
                if idx is None:
                    exhausted = True
                    break
                pending[asyncio.create_task(one(idx))] = idx
            if not pending:
                break
            done, _ = await asyncio.wait(pending.keys(), return_when=asyncio.FIRST_COMPLETED)
            for task in done:
                idx = pending.pop(task)
                err = task.exception()
                if err is None:
                    t_req, t_wr = task.result()
                    stats.ok += 1
                    stats.request_s += t_req
                    stats.write_s += t_wr
                    streak = 0
                else:
                    if cfg.fail_on_error:
                        raise err
                    log.warning("Skipping sample %d due to error: %s", idx, err)
                    stats.errors += 1
                    stats.skipped.append(idx)
                    streak += 1
                    if limit and streak >= limit:
                        raise ConsecutiveFailureAbort(
                            f"Aborting: {limit} consecutive samples errored out. The server may be unreachable."
                        ) from err
                stats.elapsed_s = time.perf_counter() - t0
                if on_progress is not None:
                    on_progress(stats)
    finally:
        for task in pending:
            task.cancel()
        if pending:
            await asyncio.gather(*pending.keys(), return_exceptions=True)
        stats.elapsed_s = time.perf_counter() - t0
    return stats
