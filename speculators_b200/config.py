"""Configuration objects that map one-to-one onto a saved ``config.json``.

``SpeculatorModelConfig`` is the polymorphic root (discriminator
``speculators_model_type``); ``SpeculatorsConfig`` names the algorithm, its token
proposal methods and the verifier the draft was trained against;
``VerifierConfig`` is the verifier reference.  Field names, defaults and the
default-proposal validator match src/speculators/config.py:40-161,257-287 so a
file written by either implementation loads in the other and in vLLM.

Unlike the reference these are plain pydantic models: nothing here inherits from
``transformers.PretrainedConfig``.  The small part of that API that callers use
(``from_pretrained``, ``save_pretrained``, ``to_dict``, ``from_dict``,
``to_json_string``) is implemented directly on top of ``json``.
"""

from __future__ import annotations

import json
import os
from typing import Any, ClassVar

from pydantic import BaseModel, ConfigDict, Field, field_serializer, field_validator, model_validator

from speculators_b200.layer_config import TransformerLayerConfig, read_config_json
from speculators_b200.proposals import TokenProposalConfig
from speculators_b200.utils import PydanticClassRegistryMixin, ReloadableBaseModel
from speculators_b200.version import __version__

__all__ = [
    "SpeculatorModelConfig",
    "SpeculatorsConfig",
    "VerifierConfig",
    "reload_schemas",
]


class VerifierConfig(BaseModel):
    name_or_path: str | None = Field(description="local path (or hub id) of the verifier")
    architectures: list[str] = Field(description="`architectures` of the verifier's config.json")

    @classmethod
    def from_config(cls, config: Any, name_or_path: str | None = "UNSET") -> "VerifierConfig":
        """Extract the reference from an already-loaded config object or dict."""
        data = config if isinstance(config, dict) else config.to_dict()
        if name_or_path == "UNSET":
            name_or_path = (
                getattr(config, "name_or_path", None)
                or data.get("_name_or_path")
                or data.get("name_or_path")
            )
        return cls(name_or_path=name_or_path, architectures=data.get("architectures") or [])

    @classmethod
    def from_pretrained(cls, name_or_path: str, **_: Any) -> "VerifierConfig":
        """Read the verifier's own config.json so ``architectures`` is the real one."""
        data = read_config_json(name_or_path)
        return cls(name_or_path=str(name_or_path), architectures=data.get("architectures") or [])


class SpeculatorsConfig(ReloadableBaseModel):
    algorithm: str
    proposal_methods: list[TokenProposalConfig]
    default_proposal_method: str
    verifier: VerifierConfig

    @field_validator("proposal_methods", mode="before")
    @classmethod
    def _polymorphic_proposals(cls, value: Any) -> Any:
        if isinstance(value, (list, tuple)):
            return [TokenProposalConfig.model_validate(v) if isinstance(v, dict) else v for v in value]
        return value

    @field_serializer("proposal_methods")
    def _dump_proposals(self, value: list[TokenProposalConfig]) -> list[dict[str, Any]]:
        return [v.model_dump() for v in value]

    @model_validator(mode="after")
    def _default_method_is_listed(self) -> "SpeculatorsConfig":
        names = [m.proposal_type for m in self.proposal_methods]
        if self.default_proposal_method not in names:
            raise ValueError(
                f"default_proposal_method {self.default_proposal_method!r} is not one of the "
                f"configured proposal_methods {names}"
            )
        return self


class SpeculatorModelConfig(PydanticClassRegistryMixin):
    """Root of every algorithm's config; serialises to the checkpoint's config.json."""

    model_config = ConfigDict(arbitrary_types_allowed=True, extra="allow", validate_assignment=False)
    schema_discriminator: ClassVar[str] = "speculators_model_type"
    dispatch_on_construct: ClassVar[bool] = False  # only from_dict / from_pretrained / model_validate pick the algorithm's class
    model_type: ClassVar[str] = "speculator_model"

    speculators_model_type: str = ""
    speculators_version: str = __version__
    speculators_config: SpeculatorsConfig | None = None
    architectures: list[str] = Field(default_factory=list)
    torch_dtype: str | None = None
    tie_word_embeddings: bool = False

    # ---- nested decoder config shared by every algorithm -------------------------
    @classmethod
    def _coerce_layer_config(cls, value: Any) -> Any:
        return None if value is None else TransformerLayerConfig.from_any(value)

    # ---- dict / json -----------------------------------------------------------
    def to_dict(self) -> dict[str, Any]:
        out = self.model_dump()
        for key, value in list(out.items()):
            if isinstance(value, TransformerLayerConfig):
                out[key] = value.to_dict()
        if out.get("torch_dtype") is None:
            out.pop("torch_dtype", None)
        out["model_type"] = self.model_type
        return out

    to_diff_dict = to_dict

    def to_json_string(self) -> str:
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"

    def to_json_file(self, json_file_path: str | os.PathLike, **_: Any) -> None:
        with open(json_file_path, "w", encoding="utf-8") as fh:
            fh.write(self.to_json_string())

    @classmethod
    def from_dict(cls, config_dict: dict[str, Any], **kwargs: Any) -> "SpeculatorModelConfig":
        merged = {**config_dict, **kwargs}
        if "speculators_model_type" not in merged:
            raise ValueError(
                "The config dictionary must contain the 'speculators_model_type' field - without it "
                "this is not a speculators checkpoint (external checkpoints go through speculators_b200.convert)"
            )
        merged.pop("model_type", None)
        merged.pop("transformers_version", None)
        if "dtype" in merged and "torch_dtype" not in merged:
            merged["torch_dtype"] = merged.pop("dtype")
        return SpeculatorModelConfig.model_validate(merged) if cls is SpeculatorModelConfig else cls.model_validate(merged)

    @classmethod
    def get_config_dict(cls, pretrained_model_name_or_path: str | os.PathLike, cache_dir: str | None = None, force_download: bool = False,
                        local_files_only: bool = False, token: str | None = None, revision: str = "main",
                        **unused: Any) -> tuple[dict[str, Any], dict[str, Any]]:
        """``(config dict, unused kwargs)`` like ``transformers.PretrainedConfig.get_config_dict``: a local
        directory (or a path to a json file) is read directly; anything else is taken for a hub id and its
        ``config.json`` fetched through ``huggingface_hub`` when that package and a network are available."""
        path = os.fspath(pretrained_model_name_or_path)
        if os.path.isdir(path) or os.path.isfile(path):
            return read_config_json(path), dict(unused)
        try:
            from huggingface_hub import hf_hub_download
        except ImportError:
            return read_config_json(path), dict(unused)  # raises the FileNotFoundError that names what was looked for
        try:
            file = hf_hub_download(repo_id=path, filename="config.json", cache_dir=cache_dir, force_download=force_download,
                                   local_files_only=local_files_only, token=token, revision=revision)
        except Exception as err:  # noqa: BLE001 - the hub client raises several unrelated types when offline
            raise FileNotFoundError(f"no config.json at {path!r} and the hub could not provide one ({type(err).__name__})") from err
        return read_config_json(file), dict(unused)

    @classmethod
    def from_pretrained(cls, pretrained_model_name_or_path: str | os.PathLike, **kwargs: Any) -> "SpeculatorModelConfig":
        data, _ = cls.get_config_dict(
            pretrained_model_name_or_path, cache_dir=kwargs.pop("cache_dir", None), force_download=kwargs.pop("force_download", False),
            local_files_only=kwargs.pop("local_files_only", False), token=kwargs.pop("token", None), revision=kwargs.pop("revision", "main"),
        )
        if "speculators_model_type" not in data:
            raise NotImplementedError(
                "config.json has no 'speculators_model_type'. Loading a non-speculator model config "
                "is not supported yet; convert the checkpoint first"
            )
        kwargs = {k: v for k, v in kwargs.items() if k in cls.model_fields}
        return cls.from_dict(data, **kwargs)

    def save_pretrained(self, save_directory: str | os.PathLike, **_: Any) -> str:
        os.makedirs(save_directory, exist_ok=True)
        path = os.path.join(save_directory, "config.json")
        tmp = path + ".tmp"
        with open(tmp, "w") as fh:
            fh.write(self.to_json_string())
        os.replace(tmp, path)
        return path

    # ``name_or_path`` mirrors what HF sets after from_pretrained
    name_or_path: str | None = Field(default=None, exclude=True)


def reload_schemas() -> None:
    """Kept for API parity (src/speculators/config.py:379-387).  Dispatch on the
    discriminator is resolved at validation time here, so this only refreshes
    pydantic's cached schemas."""
    TokenProposalConfig.reload_schema()
    SpeculatorsConfig.reload_schema()
    SpeculatorModelConfig.reload_schema()
