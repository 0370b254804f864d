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

__all__ = ["ensure_checkpoint_is_local", "find_vocab_size", "load_checkpoint_config", "load_checkpoint_weights"]


def ensure_checkpoint_is_local(path: str | Path, cache_dir: str | Path | None = None) -> Path:
    p = Path(path)
    if p.exists():
        return p
    try:
        from huggingface_hub import snapshot_download
    except ImportError as err:
        raise FileNotFoundError(f"Checkpoint '{path}' is not a local path and huggingface_hub is unavailable") from err
    return Path(snapshot_download(repo_id=str(path), cache_dir=cache_dir, allow_patterns=["*.json", "*.safetensors", "*.bin"]))


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
