"""Selective reads from safetensors checkpoints.

A draft model only needs three tensors of its verifier (token embeddings, LM
head, final norm), so nothing here ever loads a full checkpoint: the shard index
is consulted and only the shards that hold a requested tensor are opened.
Behaviour parity: src/speculators/utils/loading.py (exact -> suffix -> alias key
resolution :11-26, config-only directory test :29-53, key listing :56-79,
``load_model_layers`` :82-136).
"""

from __future__ import annotations

import json
import logging
from collections import defaultdict
from pathlib import Path

import torch
from safetensors import safe_open

log = logging.getLogger("speculators")

__all__ = ["is_config_only_dir", "list_checkpoint_keys", "load_model_layers", "resolve_checkpoint_file"]

# alternative spellings used by some verifier families
_ALIASES: dict[str, tuple[str, ...]] = {
    "embed_tokens.weight": ("tok_embeddings.weight", "llm.embed.weight"),
    "lm_head.weight": ("output.weight", "llm.unembed.weight"),
    "model.norm.weight": ("norm.weight",),
}
_INDEX = "model.safetensors.index.json"
_SINGLE = "model.safetensors"


def _match(name: str, keys) -> str | None:
    for cand in (name, *_ALIASES.get(name, ())):
        if cand in keys:
            return cand
        for key in keys:
            if key.endswith(cand):
                return key
    return None


def resolve_checkpoint_file(model_path: str | Path, file_name: str) -> Path:
    """Local directory lookup; a hub id is fetched through ``huggingface_hub`` when
    that package and a network are available."""
    root = Path(model_path)
    if root.is_dir():
        path = root / file_name
        if not path.exists():
            raise FileNotFoundError(f"Expected local file missing: {path}")
        return path
    try:
        from huggingface_hub import hf_hub_download
    except ImportError as err:  # pragma: no cover
        raise FileNotFoundError(f"{model_path!r} is not a local directory and huggingface_hub is absent") from err
    return Path(hf_hub_download(repo_id=str(model_path), filename=file_name))


def is_config_only_dir(path: str | Path) -> bool:
    root = Path(path)
    if not root.is_dir() or not (root / "config.json").is_file():
        return False
    patterns = ("*.safetensors", "*.bin", "*.safetensors.index.json", "*.bin.index.json")
    return not any(any(root.glob(p)) for p in patterns)


def _weight_map(model_path: str | Path) -> dict[str, str]:
    try:
        index = resolve_checkpoint_file(model_path, _INDEX)
        return json.loads(Path(index).read_text())["weight_map"]
    except Exception as err:  # noqa: BLE001 - hub 404s come in several exception types
        if not isinstance(err, FileNotFoundError) and type(err).__name__ != "EntryNotFoundError":
            raise
    single = resolve_checkpoint_file(model_path, _SINGLE)
    with safe_open(str(single), framework="pt", device="cpu") as fh:
        return dict.fromkeys(fh.keys(), _SINGLE)


def list_checkpoint_keys(checkpoint_dir: str | Path) -> list[str]:
    root = Path(checkpoint_dir)
    if not (root / _INDEX).exists() and not (root / _SINGLE).exists():
        raise FileNotFoundError(f"No safetensors checkpoint found at {root} (looked for {_INDEX} and {_SINGLE}).")
    return list(_weight_map(root).keys())


def load_model_layers(layer_names: list[str], model_path: str | Path) -> dict[str, torch.Tensor]:
    """Return ``{requested name: tensor}`` for every name that resolves."""
    wmap = _weight_map(model_path)
    by_shard: dict[str, list[tuple[str, str]]] = defaultdict(list)
    for name in layer_names:
        key = _match(name, wmap)
        if key is None:
            log.warning("Tensor '%s' not found in the checkpoint of %s.", name, model_path)
            continue
        by_shard[wmap[key]].append((name, key))
    if not by_shard:
        raise ValueError("None of the requested tensor names were found in the index.")
    out: dict[str, torch.Tensor] = {}
    for shard, pairs in by_shard.items():
        with safe_open(str(resolve_checkpoint_file(model_path, shard)), framework="pt", device="cpu") as fh:
            for name, key in pairs:
                out[name] = fh.get_tensor(key)
    return out


# the reference's private names for the two lookups above (its tests and some downstream code use them)
_resolve_key = _match
_resolve_file = resolve_checkpoint_file
