"""Helpers shared by the algorithm implementations (parity:
src/speculators/models/utils.py:20-111)."""

from __future__ import annotations

import warnings

from speculators_b200.layer_config import TransformerLayerConfig, read_config_json, unwrap_text_config

__all__ = [
    "DEFAULT_TARGET_LAYER_IDS_WARNING",
    "flatten_rope_parameters",
    "conditional_torch_compile",
    "get_verifier_config",
    "resolve_draft_intermediate_size",
    "resolve_target_layer_ids",
]


def conditional_torch_compile(fn=None, **_compile_kwargs):
    """Kept for API parity with the reference (src/speculators/models/utils.py:12-17),
    which compiles hot functions when CUDA is present.  This package has no tracing
    compiler in its hot path (CUDA kernels + CUDA graphs), so the function comes back
    unchanged; usable bare or with arguments."""
    if fn is None:
        return lambda f: f
    return fn


DEFAULT_TARGET_LAYER_IDS_WARNING = (
    "--target-layer-ids is not explicitly set. Setting target layers to {ids}. If custom target "
    "layers were used when launching vllm datagen, please set them explicitly."
)


def get_verifier_config(verifier_name_or_path: str, trust_remote_code: bool = False) -> TransformerLayerConfig:
    """Language-model part of the verifier's config.json (``text_config`` unwrapped)."""
    del trust_remote_code  # nothing is executed from the checkpoint directory
    return TransformerLayerConfig(**unwrap_text_config(read_config_json(verifier_name_or_path)))


def resolve_target_layer_ids(target_layer_ids: list[int] | None, verifier_name_or_path: str, trust_remote_code: bool = False) -> list[int]:
    """Explicit ids win; otherwise ``[2, n // 2, n - 3]`` for an ``n``-layer verifier."""
    if target_layer_ids is not None:
        return list(target_layer_ids)
    n = int(get_verifier_config(verifier_name_or_path, trust_remote_code).num_hidden_layers)
    ids = [2, n // 2, n - 3]
    warnings.warn(DEFAULT_TARGET_LAYER_IDS_WARNING.format(ids=ids), stacklevel=3)
    return ids


def flatten_rope_parameters(config):
    """Configs that keep one rotary setting per layer type (``rope_parameters`` keyed by
    ``sliding_attention`` / ``full_attention``) become a deep copy whose ``rope_parameters``
    is the ``sliding_attention`` entry, which is what a rotary table is built from; any other
    config is returned as it is (src/speculators/models/utils.py:60-74)."""
    import copy

    rope = getattr(config, "rope_parameters", None)
    if not rope or "sliding_attention" not in rope:
        return config
    out = copy.deepcopy(config)
    out.rope_parameters = rope["sliding_attention"]
    return out


def resolve_draft_intermediate_size(verifier_config) -> int:
    """Dense verifiers: mirror ``intermediate_size``.  MoE verifiers expose none, so the
    dense draft uses ``3 * hidden_size``."""
    cfg = TransformerLayerConfig.from_any(verifier_config)
    if "intermediate_size" in cfg and cfg.intermediate_size is not None:
        return int(cfg.intermediate_size)
    if "hidden_size" not in cfg:
        raise ValueError(
            "Verifier config exposes neither `intermediate_size` nor `hidden_size`, so a draft "
            "intermediate_size cannot be inferred. Pass --draft-config to set the draft architecture explicitly."
        )
    size = 3 * int(cfg.hidden_size)
    warnings.warn(
        f"Verifier config has no dense intermediate_size (likely MoE); using draft intermediate_size={size} "
        f"(3 x hidden_size = {cfg.hidden_size}). Pass --draft-config to override.",
        stacklevel=3,
    )
    return size
