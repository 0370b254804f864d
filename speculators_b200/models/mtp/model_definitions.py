"""MTP layer: ``input_proj(cat[token_norm(embedding), hidden_norm(hidden)])`` ->
one decoder block of the verifier's architecture -> ``final_layernorm``
(src/speculators/models/mtp/model_definitions.py:73-116).  The 2H -> H projection
happens *before* attention, so q/k/v keep the standard width.

Supported block types: dense ``qwen3`` / ``llama`` blocks, and the gated-attention
+ mixture-of-experts block of ``qwen3_next`` / ``qwen3_5_moe_text`` verifiers
(``speculators_b200.models.moe``).
"""

from __future__ import annotations

import torch
from torch import nn

from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.models.layers import DecoderLayer, Linear, RMSNorm

__all__ = ["MTPLayer", "MTPLayerMixin", "build_mtp_layer", "mtp_model_classes", "resolve_model_type"]

_DENSE_TYPES = ("qwen3", "llama", "qwen2")
_MOE_TYPES = ("qwen3_next", "qwen3_5_moe_text", "qwen3_5_text")


def resolve_model_type(model_type: str) -> str:
    if model_type in _DENSE_TYPES or model_type in _MOE_TYPES:
        return model_type
    raise ValueError(f"Unsupported MTP model type '{model_type}'. Supported types: {sorted(_DENSE_TYPES + _MOE_TYPES)}")


class _MTPMixin:
    def _setup_mtp_modules(self, config: TransformerLayerConfig, norm_cls=RMSNorm) -> None:
        H, eps = config.hidden_size, config.rms_norm_eps
        self.hidden_layernorm = norm_cls(H, eps)
        self.token_layernorm = norm_cls(H, eps)
        self.input_proj = Linear(2 * H, H, bias=False)
        self.final_layernorm = norm_cls(H, eps)

    def combine(self, hidden_states: torch.Tensor, token_embeddings: torch.Tensor) -> torch.Tensor:
        return self.input_proj(torch.cat([self.token_layernorm(token_embeddings), self.hidden_layernorm(hidden_states)], dim=-1))


class MTPLayer(_MTPMixin, DecoderLayer):
    """Dense decoder block variant."""

    def __init__(self, config: TransformerLayerConfig, layer_idx: int = 0):
        DecoderLayer.__init__(self, config, layer_idx)
        self._setup_mtp_modules(config)

    def forward(self, hidden_states, token_embeddings, positions, rotary, spec):
        x = self.combine(hidden_states, token_embeddings)
        return self.final_layernorm(DecoderLayer.forward(self, x, positions, rotary, spec))


MTPLayerMixin = _MTPMixin  # public name (src/speculators/models/mtp/model_definitions.py:73)


class _LazyMTPClasses(dict):
    """``model_type -> ModelComponents`` with the MTP layer as ``first_layer_class``
    (src/speculators/models/mtp/model_definitions.py:152-190).  Filled on first use: the
    MoE layer module imports this one."""

    def _fill(self) -> None:
        if dict.__len__(self):
            return
        from speculators_b200.models import base_components
        from speculators_b200.models.moe import MoEMTPLayer

        for kind in _DENSE_TYPES:
            dict.__setitem__(self, kind, base_components.override_components(kind, first_layer_class=MTPLayer))
        for kind in _MOE_TYPES:
            dict.__setitem__(self, kind, base_components.override_components(kind, first_layer_class=MoEMTPLayer))

    def __getitem__(self, key):
        self._fill()
        return dict.__getitem__(self, key)

    def __contains__(self, key) -> bool:
        self._fill()
        return dict.__contains__(self, key)

    def __iter__(self):
        self._fill()
        return dict.__iter__(self)

    def __len__(self) -> int:
        self._fill()
        return dict.__len__(self)

    def keys(self):
        self._fill()
        return dict.keys(self)

    def items(self):
        self._fill()
        return dict.items(self)

    def values(self):
        self._fill()
        return dict.values(self)


mtp_model_classes = _LazyMTPClasses()


def build_mtp_layer(config: TransformerLayerConfig, layer_idx: int = 0, ep_group=None) -> nn.Module:
    kind = resolve_model_type(config.model_type)
    if kind in _MOE_TYPES and int(config.get("num_experts", 0) or 0) > 0 or kind == "qwen3_next":
        from speculators_b200.models.moe import MoEMTPLayer

        return MoEMTPLayer(config, layer_idx, ep_group=ep_group)
    return MTPLayer(config, layer_idx)
