"""Building blocks per verifier architecture.

The reference keeps a table ``model_type -> (first_layer, decoder_layer, norm, rotary)``
of HF classes (src/speculators/models/base_components.py:17-118) and lets an algorithm
swap single entries (``override_components``).  The same table here points at this
package's own blocks: one ``DecoderLayer`` implementation covers Llama and Qwen3 (per-head
q/k norms switch on by ``model_type`` / config), ``MoEDecoderLayer`` covers the
gated-attention + sparse-MoE blocks of the ``qwen3_next`` / ``qwen3_5`` families, and a
single rotary table class handles default / linear / llama3 scaling and partial rotation.
"""

from __future__ import annotations

from typing import NamedTuple

from speculators_b200.models.layers import DecoderLayer, RMSNorm, RotaryTable
from speculators_b200.models.moe import MoEDecoderLayer, ZeroCenteredRMSNorm

__all__ = ["ModelComponents", "model_classes", "override_components"]


class ModelComponents(NamedTuple):
    first_layer_class: type  # an algorithm may replace just this one (EAGLE-3's 2H-input layer)
    decoder_layer_class: type
    norm_class: type
    rotary_emb_class: type


_DENSE = ModelComponents(DecoderLayer, DecoderLayer, RMSNorm, RotaryTable)
_GATED_MOE = ModelComponents(MoEDecoderLayer, MoEDecoderLayer, ZeroCenteredRMSNorm, RotaryTable)

model_classes: dict[str, ModelComponents] = {
    "llama": _DENSE,
    "qwen2": _DENSE,
    "qwen3": _DENSE,
    "qwen3_next": _GATED_MOE,
    "qwen3_5_text": _GATED_MOE,
    "qwen3_5_moe_text": _GATED_MOE,
}


def override_components(model_type: str, **overrides) -> ModelComponents:
    """The architecture's components with some fields replaced, e.g.
    ``override_components("llama", first_layer_class=Eagle3FirstLayer)``."""
    if model_type not in model_classes:
        raise KeyError(f"Unknown model type '{model_type}'. Known: {sorted(model_classes)}")
    return model_classes[model_type]._replace(**overrides)
