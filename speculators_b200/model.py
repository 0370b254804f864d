"""Base classes of every draft ("speculator") model.

``SpeculatorModel`` is an ``nn.Module`` with the slice of the Hugging Face
``PreTrainedModel`` surface that users of the reference rely on:
``from_pretrained`` (polymorphic over the registry, optional auto-conversion of
external checkpoints, then ``load_vocab_mappings`` + ``load_verifier_weights``),
``save_pretrained`` (``config.json`` + ``model.safetensors`` in the layout vLLM
loads), ``from_training_args`` / ``get_trainer_kwargs`` / 
``verify_training_compatible``.  Reference: src/speculators/model.py:202-575.

``DraftVocabMixin`` owns the reduced draft vocabulary: ``t2d`` (bool mask over the
verifier vocabulary), ``d2t`` (int64 offsets ``target_id - draft_id``), the frozen
token embedding and the two LM heads, all NaN-initialised so that a weight that
was never loaded is impossible to miss (src/speculators/model.py:20-199).
"""

from __future__ import annotations

import json
import os
import warnings
from typing import Any, ClassVar

import torch
from safetensors.torch import load_file, save_file
from torch import nn

from speculators_b200.config import SpeculatorModelConfig
from speculators_b200.utils import ClassRegistryMixin

__all__ = ["DraftVocabMixin", "SpeculatorModel"]

_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}


class DraftVocabMixin(nn.Module):
    t2d: torch.Tensor | None
    d2t: torch.Tensor | None

    def _init_vocab(self, config) -> None:
        tl = config.transformer_layer_config
        self.draft_vocab_size = int(config.draft_vocab_size)
        self.verifier_vocab_size = int(tl.vocab_size)
        self.hidden_size = int(tl.hidden_size)
        self.use_draft_vocab = self.draft_vocab_size != self.verifier_vocab_size
        if self.use_draft_vocab:
            self.register_buffer("t2d", torch.zeros(self.verifier_vocab_size, dtype=torch.bool))
            self.register_buffer("d2t", torch.zeros(self.draft_vocab_size, dtype=torch.long))
        else:
            self.register_buffer("t2d", None)
            self.register_buffer("d2t", None)
        self.embed_tokens = nn.Embedding(self.verifier_vocab_size, self.hidden_size, padding_idx=tl.get("pad_token_id"))
        self.lm_head = nn.Linear(self.hidden_size, self.draft_vocab_size, bias=False)
        self.verifier_lm_head = nn.Linear(self.hidden_size, self.draft_vocab_size, bias=False)
        for mod in (self.embed_tokens, self.lm_head, self.verifier_lm_head):
            mod.weight.requires_grad_(False)
            with torch.no_grad():
                mod.weight.fill_(float("nan"))

    def load_vocab_mappings(self, t2d: torch.Tensor | None, d2t: torch.Tensor | None) -> None:
        if t2d is None and d2t is None:
            return
        if t2d is None or d2t is None:
            raise ValueError(
                "Both t2d and d2t must be provided together, or both must be None. "
                f"Got t2d={'provided' if t2d is not None else 'None'}, d2t={'provided' if d2t is not None else 'None'}"
            )
        if not self.use_draft_vocab:
            return  # identity mappings next to an unpruned checkpoint are accepted and ignored
        if t2d.shape[0] != self.verifier_vocab_size:
            raise ValueError(f"t2d.shape[0] ({t2d.shape[0]}) must match verifier_vocab_size ({self.verifier_vocab_size}).")
        kept = int(t2d.sum(dtype=torch.long).item())
        if kept != self.draft_vocab_size:
            raise ValueError(f"t2d has {kept} non-zero values, expected {self.draft_vocab_size}.")
        if d2t.shape[0] != self.draft_vocab_size:
            raise ValueError(f"d2t.shape[0] ({d2t.shape[0]}) must match draft_vocab_size ({self.draft_vocab_size}).")
        with torch.no_grad():
            self.t2d.copy_(t2d.to(torch.bool))
            self.d2t.copy_(d2t.to(torch.long))

    def load_verifier_weights(self) -> None:
        from speculators_b200.utils.loading import load_model_layers

        spec_cfg = getattr(getattr(self, "config", None), "speculators_config", None)
        if spec_cfg is None or spec_cfg.verifier.name_or_path is None:
            return
        path = spec_cfg.verifier.name_or_path
        wanted = ["embed_tokens.weight", "lm_head.weight"]
        if hasattr(self, "verifier_norm"):
            wanted.append("model.norm.weight")
        got = load_model_layers(wanted, path)
        embed = got["embed_tokens.weight"]
        head = got.get("lm_head.weight", embed)  # tied embeddings
        with torch.no_grad():
            if self.embed_tokens.weight.isnan().any():
                self.embed_tokens.weight.copy_(embed)
            if self.use_draft_vocab:
                if self.t2d is None or not bool(self.t2d.any()):
                    raise ValueError(
                        "t2d tensor hasn't been set. Please call `.load_vocab_mappings(t2d, d2t)` "
                        "before `.load_verifier_weights()`"
                    )
                head = head[self.t2d.to(head.device)]
            if self.lm_head.weight.isnan().any():
                self.lm_head.weight.copy_(head)
            self.verifier_lm_head.weight.copy_(head)
            if hasattr(self, "verifier_norm"):
                if "model.norm.weight" in got:
                    self.verifier_norm.weight.copy_(got["model.norm.weight"])
                else:
                    warnings.warn(
                        f"Could not find final norm weights in {path}. Using default initialization (weight=1.0).",
                        UserWarning, stacklevel=2,
                    )
        for mod in (self.embed_tokens, self.lm_head, self.verifier_lm_head):
            mod.weight.requires_grad_(False)
        if hasattr(self, "verifier_norm"):
            self.verifier_norm.weight.requires_grad_(False)


class SpeculatorModel(ClassRegistryMixin, nn.Module):
    config_class: ClassVar[type[SpeculatorModelConfig]] = SpeculatorModelConfig
    main_input_name: ClassVar[str] = "input_ids"
    base_model_prefix: ClassVar[str] = "model"
    # algorithms register themselves when this package's ``models`` sub-packages are imported
    auto_package: ClassVar[str] = "speculators_b200.models"
    registry_auto_discovery: ClassVar[bool] = True
    _keys_to_ignore_on_load_missing: ClassVar[list[str]] = []
    _keys_to_ignore_on_save: ClassVar[list[str]] = []

    def __init__(self, config: SpeculatorModelConfig, **_: Any):
        if not config:
            raise ValueError("Config must be provided to initialize a SpeculatorModel.")
        if not isinstance(config, SpeculatorModelConfig):
            raise TypeError(f"Expected config to be an instance of SpeculatorModelConfig, got {type(config)} {config}.")
        nn.Module.__init__(self)
        config.tie_word_embeddings = False
        self.config = config

    def post_init(self) -> None:
        """End-of-constructor hook (the convention of ``transformers`` models, which
        subclasses written against the reference follow): applies ``_init_weights`` to every
        sub-module when the subclass defines it."""
        init = getattr(self, "_init_weights", None)
        if callable(init):
            self.apply(init)

    # ------------------------------------------------------------------ abstract API
    def forward(self, *args, **kwargs):
        raise NotImplementedError("The forward method is only supported on concrete speculator model subclasses.")

    @classmethod
    def from_training_args(cls, verifier_config, **kwargs) -> "SpeculatorModel":
        raise NotImplementedError(f"{cls.__name__} must implement from_training_args() classmethod to support training infrastructure.")

    @staticmethod
    def get_trainer_kwargs(**kwargs) -> tuple[dict, dict]:
        raise NotImplementedError("Model must implement get_trainer_kwargs() staticmethod to support training infrastructure.")

    # ------------------------------------------------------------------ registry helpers
    @classmethod
    def registered_model_class_from_config(cls, config: SpeculatorModelConfig) -> type["SpeculatorModel"]:
        if not isinstance(config, SpeculatorModelConfig):
            raise TypeError(f"Expected config to be an instance of SpeculatorModelConfig, got {type(config)} {config}.")
        if type(config) is SpeculatorModelConfig:
            raise TypeError(f"Received a SpeculatorModelConfig instance but expected a subclass. Received: {type(config)} {config}")
        table = SpeculatorModel.registry
        if not table:
            raise ValueError("No registered model classes found. Register models with `SpeculatorModel.register(NAME)`.")
        for klass in table.values():
            if type(config) is klass.config_class:
                return klass
        raise ValueError(f"No registered model class found for config type {type(config)}. Available registered model classes: {list(table)}.")

    @classmethod
    def verify_training_compatible(cls, model: "SpeculatorModel") -> None:
        if not isinstance(model, SpeculatorModel):
            raise TypeError(f"Model must be a SpeculatorModel, got {type(model).__name__}")
        table = SpeculatorModel.registry or {}
        if type(model) not in table.values():
            raise ValueError(f"Model {type(model).__name__} is not registered in SpeculatorModel.registry. Available models: {list(table)}")
        if not hasattr(model, "layers"):
            raise AttributeError(f"Model {type(model).__name__} must have a 'layers' attribute containing decoder layers for FSDP wrapping")

    # ------------------------------------------------------------------ persistence
    def saveable_state_dict(self, dtype: torch.dtype | None = None) -> dict[str, torch.Tensor]:
        skip = set(self._keys_to_ignore_on_save)
        out = {}
        for key, value in self.state_dict().items():
            if key in skip:
                continue
            if dtype is not None and value.is_floating_point():
                value = value.to(dtype)
            out[key] = value.detach().contiguous().cpu()
        return out

    def save_pretrained(self, save_directory: str | os.PathLike, state_dict: dict[str, torch.Tensor] | None = None, **_: Any) -> None:
        os.makedirs(save_directory, exist_ok=True)
        tensors = state_dict if state_dict is not None else self.saveable_state_dict()
        tensors = {k: v.detach().contiguous().cpu() for k, v in tensors.items() if k not in set(self._keys_to_ignore_on_save)}
        floats = {str(v.dtype).removeprefix("torch.") for v in tensors.values() if v.is_floating_point()}
        if len(floats) == 1:
            self.config.torch_dtype = floats.pop()
        self.config.save_pretrained(save_directory)
        save_file(tensors, os.path.join(save_directory, "model.safetensors"), metadata={"format": "pt"})

    @classmethod
    def from_pretrained(
        cls,
        pretrained_model_name_or_path: str | os.PathLike | None,
        *model_args: Any,
        config: SpeculatorModelConfig | str | os.PathLike | None = None,
        t2d: torch.Tensor | None = None,
        d2t: torch.Tensor | None = None,
        verifier: str | None = None,
        state_dict: dict[str, torch.Tensor] | None = None,
        torch_dtype: torch.dtype | str | None = None,
        **kwargs: Any,
    ) -> "SpeculatorModel":
        if not config:
            if not pretrained_model_name_or_path:
                raise ValueError("Either `config` or `pretrained_model_name_or_path` must be provided to load a SpeculatorModel.")
            from speculators_b200.layer_config import read_config_json

            raw = read_config_json(pretrained_model_name_or_path)
            if "speculators_model_type" not in raw:
                from speculators_b200.convert.entrypoints import maybe_convert_external_checkpoint

                pretrained_model_name_or_path = maybe_convert_external_checkpoint(
                    pretrained_model_name_or_path, verifier=verifier, config_dict=raw
                )
            config = SpeculatorModelConfig.from_pretrained(pretrained_model_name_or_path)
        elif isinstance(config, (str, os.PathLike)) and os.path.exists(os.fspath(config)):
            config = SpeculatorModelConfig.from_pretrained(config)  # a config directory / file on disk; anything else must be a config object
        if not isinstance(config, SpeculatorModelConfig):
            raise TypeError(f"Expected config to be an instance of SpeculatorModelConfig, got {type(config)}.")
        if not pretrained_model_name_or_path and not state_dict:
            raise ValueError("Either `pretrained_model_name_or_path` or `state_dict` must be provided to load a SpeculatorModel.")
        if cls is SpeculatorModel:
            klass = cls.registered_model_class_from_config(config)
            return klass.from_pretrained(
                pretrained_model_name_or_path, *model_args, config=config, t2d=t2d, d2t=d2t,
                verifier=verifier, state_dict=state_dict, torch_dtype=torch_dtype, **kwargs,
            )
        model = cls(config)
        if state_dict is None:
            state_dict = _read_safetensors_dir(pretrained_model_name_or_path)
        result = model.load_state_dict(state_dict, strict=False)
        tolerated = set(cls._keys_to_ignore_on_load_missing)
        missing = [k for k in result.missing_keys if k not in tolerated]
        if missing:
            warnings.warn(f"Weights missing from checkpoint {pretrained_model_name_or_path}: {missing}", stacklevel=2)
        if result.unexpected_keys:
            warnings.warn(f"Unexpected weights in checkpoint {pretrained_model_name_or_path}: {result.unexpected_keys}", stacklevel=2)
        if isinstance(torch_dtype, str):
            torch_dtype = _DTYPES.get(torch_dtype)
        if torch_dtype is not None:
            model.to(torch_dtype)
        if hasattr(model, "load_vocab_mappings"):
            model.load_vocab_mappings(t2d, d2t)
        if hasattr(model, "load_verifier_weights"):
            model.load_verifier_weights()
        config.name_or_path = str(pretrained_model_name_or_path) if pretrained_model_name_or_path else None
        return model


def _read_safetensors_dir(path: str | os.PathLike) -> dict[str, torch.Tensor]:
    root = os.fspath(path)
    index = os.path.join(root, "model.safetensors.index.json")
    if os.path.exists(index):
        with open(index) as fh:
            shards = sorted(set(json.load(fh)["weight_map"].values()))
        out: dict[str, torch.Tensor] = {}
        for shard in shards:
            out.update(load_file(os.path.join(root, shard)))
        return out
    single = os.path.join(root, "model.safetensors")
    if not os.path.exists(single):
        raise FileNotFoundError(f"no model.safetensors (or shard index) under '{root}'.")
    return load_file(single)
