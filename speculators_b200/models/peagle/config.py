"""P-EAGLE configuration: EAGLE-3 plus a mask token and trainable embeddings
(src/speculators/models/peagle/config.py:13-43)."""

from __future__ import annotations

from typing import Literal

from pydantic import Field

from speculators_b200.config import SpeculatorModelConfig
from speculators_b200.models.eagle3.config import Eagle3SpeculatorConfig

__all__ = ["PEagleSpeculatorConfig"]


@SpeculatorModelConfig.register("peagle")
class PEagleSpeculatorConfig(Eagle3SpeculatorConfig):
    speculators_model_type: Literal["peagle"] = "peagle"  # type: ignore[assignment]
    architectures: list[str] = Field(default_factory=lambda: ["PEagleSpeculator"])
    mask_token_id: int | None = None
    embed_requires_grad: bool = True
