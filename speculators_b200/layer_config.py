"""Decoder-layer hyper-parameters of a draft (or verifier) model.

The checkpoint format stores the draft's decoder description as a nested dict
``transformer_layer_config`` with Hugging Face key names (``model_type``,
``hidden_size``, ``num_attention_heads`` ...; reference:
src/speculators/models/eagle3/config.py:98-114 writes it with ``to_diff_dict``).
The reference materialises that dict as a ``transformers.PretrainedConfig``
subclass; this framework owns its decoder blocks, so it only needs the numbers.
``TransformerLayerConfig`` is an attribute bag over the dict that

* keeps every key it was given (unknown keys round-trip untouched, which keeps
  a file written here loadable by vLLM and by the reference),
* supplies the Hugging Face defaults for keys that were omitted (a diff-dict
  omits defaults), and
* accepts a ``PretrainedConfig`` instance or a verifier ``config.json`` path.
"""

from __future__ import annotations

import copy
import json
import os
from typing import Any

__all__ = ["TransformerLayerConfig", "read_config_json", "unwrap_text_config"]

# Hugging Face defaults of the config classes the reference supports
# (LlamaConfig, Qwen3Config and the Qwen3-Next / Qwen3.5 text configs).
_COMMON_DEFAULTS: dict[str, Any] = {
    "hidden_act": "silu",
    "rms_norm_eps": 1e-6,
    "attention_bias": False,
    "attention_dropout": 0.0,
    "mlp_bias": False,
    "max_position_embeddings": 32768,
    "rope_theta": 10000.0,
    "rope_scaling": None,
    "sliding_window": None,
    "layer_types": None,
    "tie_word_embeddings": False,
    "pad_token_id": None,
    "partial_rotary_factor": 1.0,
}
_MODEL_DEFAULTS: dict[str, dict[str, Any]] = {
    "llama": {
        "vocab_size": 32000, "hidden_size": 4096, "intermediate_size": 11008,
        "num_hidden_layers": 32, "num_attention_heads": 32, "max_position_embeddings": 2048,
    },
    "qwen3": {
        "vocab_size": 151936, "hidden_size": 4096, "intermediate_size": 22016,
        "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 32,
        "head_dim": 128, "max_position_embeddings": 32768,
    },
    "qwen3_next": {
        "vocab_size": 151936, "hidden_size": 2048, "intermediate_size": 5632,
        "num_hidden_layers": 48, "num_attention_heads": 16, "num_key_value_heads": 2,
        "head_dim": 256, "partial_rotary_factor": 0.25, "num_experts": 512,
        "num_experts_per_tok": 10, "moe_intermediate_size": 512,
        "shared_expert_intermediate_size": 512, "norm_topk_prob": True,
    },
}
_MODEL_DEFAULTS["qwen3_5_text"] = dict(_MODEL_DEFAULTS["qwen3_next"], num_experts=0)
_MODEL_DEFAULTS["qwen3_5_moe_text"] = dict(_MODEL_DEFAULTS["qwen3_next"])

_DROP_ON_SAVE = ("_name_or_path", "transformers_version", "architectures", "torch_dtype", "dtype")


def read_config_json(name_or_path: str | os.PathLike) -> dict[str, Any]:
    """Read ``config.json`` of a local model directory (or a direct file path).

    There is no hub access in an offline deployment, so a bare hub id raises a
    ``FileNotFoundError`` naming what was looked for.
    """
    path = os.fspath(name_or_path)
    candidate = os.path.join(path, "config.json") if os.path.isdir(path) else path
    if not os.path.isfile(candidate):
        raise FileNotFoundError(
            f"no config.json at {candidate!r}; pass a local directory that contains the "
            "model's config.json (hub ids need to be downloaded first)"
        )
    with open(candidate) as fh:
        return json.load(fh)


def unwrap_text_config(cfg: dict[str, Any]) -> dict[str, Any]:
    """Multimodal verifiers nest the language model under ``text_config``
    (reference: src/speculators/models/utils.py:20-30)."""
    inner = cfg.get("text_config")
    return inner if isinstance(inner, dict) else cfg


class TransformerLayerConfig:
    def __init__(self, **kwargs: Any):
        object.__setattr__(self, "_data", {})
        for key, value in kwargs.items():
            self._data[key] = value
        self._data.setdefault("model_type", "qwen3")
        # transformers >= 5 nests rope settings; flatten for the rotary table builder
        rope = self._data.get("rope_parameters")
        if isinstance(rope, dict):
            flat = rope.get("sliding_attention") if "sliding_attention" in rope else rope
            if isinstance(flat, dict) and "rope_theta" in flat and "rope_theta" not in self._data:
                self._data["rope_theta"] = flat["rope_theta"]

    # ---- construction helpers -------------------------------------------------
    @classmethod
    def from_any(cls, value: Any) -> "TransformerLayerConfig":
        if isinstance(value, TransformerLayerConfig):
            return value
        if isinstance(value, dict):
            return cls(**value)
        if isinstance(value, (str, os.PathLike)):
            return cls(**unwrap_text_config(read_config_json(value)))
        to_dict = getattr(value, "to_dict", None)
        if callable(to_dict):  # a transformers.PretrainedConfig
            data = to_dict()
            if isinstance(data.get("text_config"), dict):
                data = data["text_config"]
            return cls(**data)
        if hasattr(value, "__dict__"):  # any plain attribute holder (argparse / SimpleNamespace stand-ins)
            return cls(**{k: v for k, v in vars(value).items() if not k.startswith("_")})
        raise TypeError(f"cannot build a TransformerLayerConfig from {type(value)!r}")

    # ---- attribute protocol ---------------------------------------------------
    def _default(self, key: str) -> Any:
        model_defaults = _MODEL_DEFAULTS.get(self._data.get("model_type", ""), {})
        if key in model_defaults:
            return model_defaults[key]
        if key in _COMMON_DEFAULTS:
            return _COMMON_DEFAULTS[key]
        if key == "num_key_value_heads":
            return self.num_attention_heads
        if key == "head_dim":
            return self.hidden_size // self.num_attention_heads
        raise AttributeError(key)

    def __getattr__(self, key: str) -> Any:
        if key.startswith("__"):
            raise AttributeError(key)
        data = object.__getattribute__(self, "_data")
        if key in data and not (key == "head_dim" and data[key] is None):
            return data[key]
        return self._default(key)

    def __setattr__(self, key: str, value: Any) -> None:
        self._data[key] = value

    def get(self, key: str, default: Any = None) -> Any:
        try:
            return getattr(self, key)
        except AttributeError:
            return default

    def __contains__(self, key: str) -> bool:
        return key in self._data

    def __eq__(self, other: object) -> bool:
        return isinstance(other, TransformerLayerConfig) and self.to_dict() == other.to_dict()

    def __repr__(self) -> str:
        return f"TransformerLayerConfig({self._data!r})"

    def __deepcopy__(self, memo):  # noqa: ANN001
        return TransformerLayerConfig(**copy.deepcopy(self._data, memo))

    def copy(self, **overrides: Any) -> "TransformerLayerConfig":
        data = copy.deepcopy(self._data)
        data.update(overrides)
        return TransformerLayerConfig(**data)

    # ---- serialisation ----------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        out = {k: v for k, v in self._data.items() if k not in _DROP_ON_SAVE and not k.startswith("_")}
        # written explicitly so readers never have to derive them
        out.setdefault("num_key_value_heads", self.num_key_value_heads)
        out.setdefault("head_dim", self.head_dim)
        return out

    to_diff_dict = to_dict

    # ---- derived quantities -------------------------------------------------------
    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * float(self.partial_rotary_factor))

    def layer_type(self, idx: int) -> str:
        types = self.layer_types
        if types and idx < len(types):
            return types[idx]
        return "full_attention"
