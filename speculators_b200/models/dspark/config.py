"""DSpark configuration: DFlash plus a low-rank Markov logit-bias head and a
confidence head (src/speculators/models/dspark/config.py:13-67)."""

from __future__ import annotations

from typing import Literal

from pydantic import Field

from speculators_b200.config import SpeculatorModelConfig
from speculators_b200.models.dflash.config import DFlashSpeculatorConfig

__all__ = ["DSparkSpeculatorConfig"]


@SpeculatorModelConfig.register("dspark")
class DSparkSpeculatorConfig(DFlashSpeculatorConfig):
    speculators_model_type: Literal["dspark"] = "dspark"  # type: ignore[assignment]
    architectures: list[str] = Field(default_factory=lambda: ["DSparkSpeculator"])
    sample_from_anchor: bool = True
    markov_rank: int = 256  # 0 disables the sequential head
    markov_head_type: Literal["vanilla", "gated", "rnn"] = "vanilla"
    enable_confidence_head: bool = True
    confidence_head_with_markov: bool = True
