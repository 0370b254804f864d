"""Small helpers of the EAGLE checkpoint converters (parity:
src/speculators/convert/eagle/utils.py): where a research checkpoint keeps its vocabulary
size, which optional tensors it carries, and how rotary / dtype settings are spelled for
the decoder config."""

from __future__ import annotations

import logging
from typing import Any

import torch

from speculators_b200.convert.utils import find_vocab_size

__all__ = ["build_llama_config_dtype_kwarg", "build_llama_config_rope_kwargs", "detect_fusion_bias_and_layernorms", "find_vocab_size"]

log = logging.getLogger("speculators")


def build_llama_config_dtype_kwarg(torch_dtype: str | None) -> dict[str, Any]:
    """``{"torch_dtype": ...}`` for the decoder config, nothing when the checkpoint names no dtype."""
    return {} if torch_dtype is None else {"torch_dtype": torch_dtype}


def build_llama_config_rope_kwargs(rope_theta: float = 10000.0, rope_scaling: dict[str, Any] | None = None) -> dict[str, Any]:
    """Rotary settings in both spellings the decoder config reads: the flat ``rope_theta`` /
    ``rope_scaling`` pair and the merged ``rope_parameters`` dict (``rope_type`` taken from
    ``rope_type`` or the older ``type`` key, ``"default"`` without scaling)."""
    merged: dict[str, Any] = {"rope_theta": rope_theta, "rope_type": "default"}
    out: dict[str, Any] = {"rope_theta": rope_theta}
    if rope_scaling is not None:
        out["rope_scaling"] = rope_scaling
        merged["rope_type"] = rope_scaling.get("rope_type", rope_scaling.get("type", "default"))
        merged.update({k: v for k, v in rope_scaling.items() if k not in ("rope_type", "type")})
    out["rope_parameters"] = merged
    return out


def detect_fusion_bias_and_layernorms(weights: dict[str, torch.Tensor]) -> tuple[bool, bool]:
    """(checkpoint has a bias on the fusion layer ``fc``, checkpoint has the extra embedding layer norms)."""
    has_bias = "fc.bias" in weights
    has_norms = any(name in weights for name in ("embed_layernorm.weight", "post_embedding_layernorm.weight"))
    if has_bias:
        log.info("Detected fusion bias in checkpoint")
    if has_norms:
        log.info("Detected extra layernorms in checkpoint")
    return has_bias, has_norms
