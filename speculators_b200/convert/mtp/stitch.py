"""Merge a fine-tuned MTP draft back into its verifier checkpoint.

The draft checkpoint stores the MTP head under this package's names
(``mtp_layers.0.*``, packed 3-D expert tensors); a deployable verifier checkpoint wants
them under the verifier's own ``mtp.*`` names with one tensor per expert.  ``stitch``
copies the verifier directory, drops the frozen tensors (embeddings, LM head), unpacks
the experts, maps names back and rewrites only the shards that hold a changed tensor.

Reference surface: scripts/stitch_mtp.py:86 (_unfuse_moe_experts), :239 (stitch).
"""

from __future__ import annotations

import json
import logging
import re
import shutil
from pathlib import Path

import torch

from speculators_b200.convert.mtp.converter import MTP_EXACT_REMAP, MTP_PREFIX_REMAP

__all__ = ["FROZEN_KEYS", "load_draft_weights", "native_key", "stitch", "unfuse_moe_experts"]

log = logging.getLogger(__name__)

FROZEN_KEYS = frozenset({"embed_tokens.weight", "lm_head.weight"})
_TO_NATIVE_EXACT = {ours: theirs for theirs, ours in MTP_EXACT_REMAP.items()}
_TO_NATIVE_PREFIX = [(ours, theirs) for theirs, ours in MTP_PREFIX_REMAP]
_PACKED = re.compile(r"^(?P<stem>.+\.experts)\.(?P<kind>gate_up_proj|down_proj)$")


def native_key(key: str) -> str:
    """Draft-checkpoint tensor name -> verifier-checkpoint tensor name."""
    if key in _TO_NATIVE_EXACT:
        return _TO_NATIVE_EXACT[key]
    for ours, theirs in _TO_NATIVE_PREFIX:
        if key.startswith(ours):
            return theirs + key[len(ours):]
    return key


def unfuse_moe_experts(weights: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """``experts.gate_up_proj [E, 2I, H]`` / ``experts.down_proj [E, H, I]`` ->
    ``experts.<e>.{gate,up,down}_proj.weight``.  Inverse of the converter's packing."""
    packed: dict[str, dict[str, torch.Tensor]] = {}
    out: dict[str, torch.Tensor] = {}
    for key, tensor in weights.items():
        m = _PACKED.match(key)
        if m:
            packed.setdefault(m["stem"], {})[m["kind"]] = tensor
        else:
            out[key] = tensor
    for stem, pair in packed.items():
        if "gate_up_proj" not in pair:
            raise ValueError(f"Found down_proj without matching gate_up_proj at: {stem}")
        if "down_proj" not in pair:
            raise ValueError(f"Found gate_up_proj at '{stem}' but missing down_proj")
        gate_up, down = pair["gate_up_proj"], pair["down_proj"]
        if gate_up.shape[0] != down.shape[0]:
            raise ValueError(f"Expert count mismatch at '{stem}': gate_up_proj has {gate_up.shape[0]} but down_proj has {down.shape[0]}")
        inter = gate_up.shape[1] // 2
        for e in range(gate_up.shape[0]):
            out[f"{stem}.{e}.gate_proj.weight"] = gate_up[e, :inter].contiguous()
            out[f"{stem}.{e}.up_proj.weight"] = gate_up[e, inter:].contiguous()
            out[f"{stem}.{e}.down_proj.weight"] = down[e].contiguous()
        log.info("Unfused %d experts at %s", gate_up.shape[0], stem)
    return out


def _read_shard(path: Path) -> tuple[dict[str, torch.Tensor], dict | None]:
    from safetensors import safe_open

    with safe_open(str(path), framework="pt") as fh:
        return {k: fh.get_tensor(k) for k in fh.keys()}, fh.metadata()  # noqa: SIM118


def load_draft_weights(checkpoint_dir: Path) -> dict[str, torch.Tensor]:
    checkpoint_dir = Path(checkpoint_dir)
    index = checkpoint_dir / "model.safetensors.index.json"
    if index.exists():
        shards = sorted(set(json.loads(index.read_text())["weight_map"].values()))
    elif (checkpoint_dir / "model.safetensors").exists():
        shards = ["model.safetensors"]
    else:
        raise FileNotFoundError(f"No safetensors found at {checkpoint_dir}")
    weights: dict[str, torch.Tensor] = {}
    for shard in shards:
        weights.update(_read_shard(checkpoint_dir / shard)[0])
    return weights


def _resolve_verifier(path: Path) -> Path:
    if Path(path).exists():
        return Path(path)
    from huggingface_hub import snapshot_download

    log.info("Verifier path %s not found locally, downloading", path)
    return Path(snapshot_download(repo_id=str(path), allow_patterns=["*.json", "*.safetensors", "*.bin", "*.index.json"]))


def _rewrite(path: Path, updates: dict[str, torch.Tensor]) -> None:
    from safetensors.torch import save_file

    tensors, meta = _read_shard(path)
    tensors.update(updates)
    save_file(tensors, str(path), metadata=meta)


def stitch(finetuned_checkpoint: Path, verifier_path: Path, output_path: Path) -> Path:
    """Write ``output_path`` = verifier checkpoint with the trained MTP tensors swapped in."""
    verifier_path = _resolve_verifier(verifier_path)
    weights = load_draft_weights(Path(finetuned_checkpoint))
    trained = {k: v for k, v in weights.items() if k not in FROZEN_KEYS}
    log.info("Loaded %d tensors (%d frozen skipped)", len(weights), len(weights) - len(trained))
    native = {native_key(k): v for k, v in unfuse_moe_experts(trained).items()}
    output_path = Path(output_path)
    shutil.copytree(verifier_path, output_path, dirs_exist_ok=True)
    index = output_path / "model.safetensors.index.json"
    if index.exists():
        weight_map = json.loads(index.read_text())["weight_map"]
        by_shard: dict[str, dict[str, torch.Tensor]] = {}
        for key, tensor in native.items():
            if key not in weight_map:
                raise ValueError(f"Finetuned key '{key}' not found in verifier weight map. The finetuned checkpoint may not match the verifier.")
            by_shard.setdefault(weight_map[key], {})[key] = tensor
        for shard, updates in by_shard.items():
            _rewrite(output_path / shard, updates)
    elif (output_path / "model.safetensors").exists():
        _rewrite(output_path / "model.safetensors", native)
    else:
        raise FileNotFoundError(f"No safetensors checkpoint found at {output_path}")
    log.info("Stitched checkpoint saved to %s", output_path)
    return output_path
