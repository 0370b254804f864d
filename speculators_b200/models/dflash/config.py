"""DFlash configuration (fields / defaults:
src/speculators/models/dflash/config.py:16-82)."""

from __future__ import annotations

from typing import Any, Literal

from pydantic import Field, field_serializer, field_validator

from speculators_b200.config import SpeculatorModelConfig
from speculators_b200.layer_config import TransformerLayerConfig

__all__ = ["DFlashSpeculatorConfig"]


@SpeculatorModelConfig.register("dflash")
class DFlashSpeculatorConfig(SpeculatorModelConfig):
    speculators_model_type: Literal["dflash"] = "dflash"
    architectures: list[str] = Field(default_factory=lambda: ["DFlashSpeculator"])
    transformer_layer_config: TransformerLayerConfig = Field(default_factory=lambda: TransformerLayerConfig(model_type="qwen3"))
    draft_vocab_size: int = 32000
    block_size: int = 8  # draft tokens predicted per forward pass of the model
    target_hidden_size: int | None = None
    aux_hidden_state_layer_ids: list[int] | None = None
    mask_token_id: int | None = None
    sliding_window_non_causal: bool = False  # sliding layers attend bidirectionally inside a block
    sample_from_anchor: bool = False  # True: slot 0 already predicts (block_size speculative tokens)

    @field_validator("transformer_layer_config", mode="before")
    @classmethod
    def _coerce_tl(cls, value: Any) -> Any:
        return cls._coerce_layer_config(value)

    @field_serializer("transformer_layer_config")
    def _dump_tl(self, value: TransformerLayerConfig) -> dict:
        return value.to_dict()

    @property
    def target_vocab_size(self) -> int:
        return self.transformer_layer_config.vocab_size
