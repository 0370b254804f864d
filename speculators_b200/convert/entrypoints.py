"""``convert_model`` (explicit conversion) and ``maybe_convert_external_checkpoint``
(auto-conversion used by ``SpeculatorModel.from_pretrained``; DFlash only, like
src/speculators/convert/entrypoints.py:29-164)."""

from __future__ import annotations

import logging
import os
import tempfile
from typing import Literal

from speculators_b200.layer_config import read_config_json

log = logging.getLogger("speculators")

__all__ = ["convert_model", "maybe_convert_external_checkpoint"]


def convert_model(model: str, verifier: str, algorithm: Literal["eagle3", "mtp", "dflash"], output_path: str = "converted",
                  validate_device: str | None = None, **kwargs) -> None:
    validate = validate_device is not None
    if algorithm == "eagle3":
        from speculators_b200.convert.eagle.eagle3_converter import Eagle3Converter

        Eagle3Converter().convert(model, output_path, verifier, validate=validate, **kwargs)
    elif algorithm == "mtp":
        from speculators_b200.convert.mtp.converter import MTPConverter

        MTPConverter().convert(model, output_path, verifier, validate=validate, **kwargs)
    elif algorithm == "dflash":
        from speculators_b200.convert.dflash.converter import DFlashConverter

        DFlashConverter().convert(model, output_path, verifier, validate=validate, **kwargs)
    else:
        raise ValueError(f"Unsupported algorithm: {algorithm}")


def maybe_convert_external_checkpoint(model: str | os.PathLike, verifier: str | None = None, cache_dir=None, output_path: str | None = None,
                                      config_dict: dict | None = None) -> str:
    config_dict = config_dict if config_dict is not None else read_config_json(model)
    if "speculators_model_type" in config_dict:
        return str(model)
    archs = config_dict.get("architectures") or []
    if not ("dflash_config" in config_dict or any("DFlash" in a for a in archs)):
        raise NotImplementedError(f"Cannot auto-convert checkpoint '{model}': unrecognized external format. Supported auto-conversion: DFlash.")
    if verifier is None:
        raise ValueError("Converting an external dflash checkpoint requires a verifier. Pass `verifier=<model id or path>`.")
    output_path = output_path or tempfile.mkdtemp(prefix="speculators_converted_")
    log.info("Auto-converting external dflash checkpoint to %s", output_path)
    convert_model(model=str(model), verifier=verifier, algorithm="dflash", output_path=output_path, cache_dir=cache_dir)
    return output_path
