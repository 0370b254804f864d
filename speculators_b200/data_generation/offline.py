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
