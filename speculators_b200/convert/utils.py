"""Shared helpers for checkpoint converters (src/speculators/convert/utils.py):
locate a checkpoint, read its config and its weights (safetensors, sharded or not;
``pytorch_model.bin`` as a fallback), find the vocabulary size in nested configs."""

from __future__ import annotations

import json
import logging
from pathlib import Path

import torch
from safetensors.torch import load_file

log = logging.getLogger("speculators")

__all__ = ["download_checkpoint_from_hub", "ensure_checkpoint_is_local", "find_vocab_size", "load_checkpoint_config", "load_checkpoint_weights"]


def download_checkpoint_from_hub(model_id: str, cache_dir: str | None = None) -> Path:
    """Fetch the config / weight files of a hub checkpoint; ``FileNotFoundError`` when that
    is not possible (no ``huggingface_hub``, no network, unknown id)."""
    try:
        from huggingface_hub import snapshot_download
    except ImportError as err:
        raise FileNotFoundError(f"Checkpoint '{model_id}' is not a local path and huggingface_hub is unavailable") from err
    try:
        local = snapshot_download(repo_id=model_id, cache_dir=cache_dir, allow_patterns=["*.json", "*.safetensors", "*.bin", "*.index.json"])
    except Exception as err:  # noqa: BLE001 - the hub raises several unrelated exception types
        raise FileNotFoundError(f"Checkpoint not found: {model_id}") from err
    return Path(local)


def ensure_checkpoint_is_local(path: str | Path, cache_dir: str | Path | None = None) -> Path:
    """An existing local path as it is; anything else is taken for a hub id and downloaded."""
    p = Path(path)
    if p.exists():
        return p
    return download_checkpoint_from_hub(str(path), cache_dir=str(cache_dir) if cache_dir else None)


def load_checkpoint_config(path: str | Path) -> dict:
    cfg = Path(path) / "config.json"
    if not cfg.exists():
        raise FileNotFoundError(f"No config.json found at {path}")
    return json.loads(cfg.read_text())


def load_checkpoint_weights(path: str | Path) -> dict[str, torch.Tensor]:
    root = Path(path)
    index = root / "model.safetensors.index.json"
    if index.exists():
        out: dict[str, torch.Tensor] = {}
        for shard in sorted(set(json.loads(index.read_text())["weight_map"].values())):
            out.update(load_file(str(root / shard)))
        return out
    single = root / "model.safetensors"
    if single.exists():
        return load_file(str(single))
    legacy = root / "pytorch_model.bin"
    if legacy.exists():
        return torch.load(legacy, map_location="cpu", weights_only=True)
    raise FileNotFoundError(f"No weights found at {path} (looked for model.safetensors[.index.json] and pytorch_model.bin)")


def find_vocab_size(config: dict) -> int | None:
    if "vocab_size" in config:
        return int(config["vocab_size"])
    for value in config.values():
        if isinstance(value, dict):
            found = find_vocab_size(value)
            if found is not None:
                return found
    return None
