"""MTP (multi-token prediction head) configuration
(src/speculators/models/mtp/config.py:18-101): full verifier vocabulary, exactly
one prediction layer, speculative depth taken from the greedy proposal config."""

from __future__ import annotations

from typing import Any, Literal

from pydantic import Field, field_serializer, field_validator

from speculators_b200.config import SpeculatorModelConfig
from speculators_b200.layer_config import TransformerLayerConfig

__all__ = ["MTPSpeculatorConfig"]


@SpeculatorModelConfig.register("mtp")
class MTPSpeculatorConfig(SpeculatorModelConfig):
    speculators_model_type: Literal["mtp"] = "mtp"
    architectures: list[str] = Field(default_factory=lambda: ["MTPDraftModel"])
    transformer_layer_config: TransformerLayerConfig = Field(default_factory=lambda: TransformerLayerConfig(model_type="qwen3"))
    num_nextn_predict_layers: int = 1  # vLLM reads this to size its MTP head list

    @field_validator("transformer_layer_config", mode="before")
    @classmethod
    def _coerce_tl(cls, value: Any) -> Any:
        return cls._coerce_layer_config(value)

    @field_serializer("transformer_layer_config")
    def _dump_tl(self, value: TransformerLayerConfig) -> dict:
        return value.to_dict()

    @field_validator("num_nextn_predict_layers")
    @classmethod
    def _one_layer(cls, value: int) -> int:
        if value != 1:
            raise ValueError(f"MTP currently supports 1 layer, got {value}.")
        return value

    @property
    def hidden_size(self) -> int:
        return self.transformer_layer_config.hidden_size

    @property
    def vocab_size(self) -> int:
        return self.transformer_layer_config.vocab_size

    @property
    def draft_vocab_size(self) -> int:
        return self.vocab_size

    @property
    def num_speculative_steps(self) -> int:
        if self.speculators_config is None or not self.speculators_config.proposal_methods:
            raise ValueError(
                "Cannot determine num_speculative_steps: speculators_config is missing or has no proposal_methods. "
                "Provide a SpeculatorsConfig with at least one proposal method."
            )
        return self.speculators_config.proposal_methods[0].speculative_tokens
