"""Per-architecture component table of the EAGLE-3 draft under the reference's module path
(src/speculators/models/eagle3/model_definitions.py).  The reference patches Hugging Face
decoder layers (one mixin, one subclass per architecture); here a single block,
``Eagle3FirstLayer`` (``models/eagle3/core.py``), serves every dense architecture because
the blocks of this package are architecture-parametrised through their config (q/k norms,
biases, rotary variant).  The architecture-specific names are kept as aliases."""

from __future__ import annotations

from speculators_b200.models import base_components
from speculators_b200.models.eagle3.core import Eagle3FirstLayer

__all__ = ["Eagle3FirstLayerMixin", "LlamaDecoderEagle3FirstLayer", "Qwen3DecoderEagle3FirstLayer", "model_classes"]

# the 2H-input behaviour is the block itself here, not a mixin over a library layer
Eagle3FirstLayerMixin = Eagle3FirstLayer
LlamaDecoderEagle3FirstLayer = Eagle3FirstLayer
Qwen3DecoderEagle3FirstLayer = Eagle3FirstLayer

model_classes: dict[str, base_components.ModelComponents] = {
    kind: base_components.override_components(kind, first_layer_class=Eagle3FirstLayer) for kind in ("llama", "qwen2", "qwen3")
}
