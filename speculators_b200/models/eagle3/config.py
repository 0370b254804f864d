"""EAGLE-3 draft configuration (fields and defaults:
src/speculators/models/eagle3/config.py:27-96)."""

from __future__ import annotations

from typing import Any, Literal

from pydantic import Field, field_serializer, field_validator, model_validator

from speculators_b200.config import SpeculatorModelConfig
from speculators_b200.layer_config import TransformerLayerConfig

__all__ = ["Eagle3SpeculatorConfig"]


@SpeculatorModelConfig.register("eagle3")
class Eagle3SpeculatorConfig(SpeculatorModelConfig):
    speculators_model_type: Literal["eagle3"] = "eagle3"
    architectures: list[str] = Field(default_factory=lambda: ["Eagle3Speculator"])
    transformer_layer_config: TransformerLayerConfig = Field(default_factory=lambda: TransformerLayerConfig(model_type="qwen3"))
    draft_vocab_size: int = 32000
    norm_before_residual: bool = False
    target_hidden_size: int | None = None
    eagle_aux_hidden_state_layer_ids: list[int] | None = None
    norm_before_fc: bool = False  # one RMSNorm over the concatenated aux states
    fc_norm: bool = False  # one RMSNorm per aux state before concatenation
    norm_output: bool = False  # feed post-norm hidden states to the next TTT step
    embed_requires_grad: bool = False

    @field_validator("transformer_layer_config", mode="before")
    @classmethod
    def _coerce_tl(cls, value: Any) -> Any:
        return cls._coerce_layer_config(value)

    @field_serializer("transformer_layer_config")
    def _dump_tl(self, value: TransformerLayerConfig) -> dict:
        return value.to_dict()

    @model_validator(mode="after")
    def _norm_flags_exclusive(self) -> "Eagle3SpeculatorConfig":
        if self.norm_before_fc and self.fc_norm:
            raise ValueError("norm_before_fc and fc_norm are mutually exclusive — enable one or the other, not both.")
        return self

    @property
    def target_vocab_size(self) -> int:
        return self.transformer_layer_config.vocab_size
