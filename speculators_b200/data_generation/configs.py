"""Named dataset presets: where to fetch each one and how to turn its rows into the
``conversations`` schema (list of ``{"role"|"from", "content"|"value"}`` turns).

Reference surface: src/speculators/data_generation/configs.py:14 (DatasetConfig),
:92 (DATASET_CONFIGS).
"""

from __future__ import annotations

import os
from collections.abc import Callable
from dataclasses import dataclass

__all__ = ["DATASET_CONFIGS", "DatasetConfig", "get_coco_dir"]


@dataclass(kw_only=True)
class DatasetConfig:
    name: str
    hf_path: str
    split: str
    subset: str | None = None
    filter_fn: Callable[[dict], bool] | None = None
    normalize_fn: Callable[[dict], dict] | None = None
    # column holding a bare user prompt, for rows without a conversation
    prompt_field: str | None = None


def get_coco_dir() -> str:
    return os.getenv("COCO_DIR") or "coco/"


def _ultrachat(row: dict) -> dict:
    return {"conversations": row["messages"]} if "messages" in row else row


def _gsm8k(row: dict) -> dict:
    return {"conversations": [{"role": "user", "content": row["question"]}, {"role": "assistant", "content": row["answer"]}]}


def _nemotron(row: dict) -> dict:
    return {"conversations": [*row["input"], {"role": "assistant", "content": row["output"]}]}


def _is_coco(row: dict) -> bool:
    return row["image"].startswith("coco/")


def _sharegpt4v_coco(row: dict) -> dict:
    """User turns become part lists: ``<image>`` lines turn into image parts that
    point at the local COCO copy, other lines into text parts."""
    root = get_coco_dir()
    image = os.path.join(root, row["image"].removeprefix("coco/"))
    if not os.path.exists(image):
        how = "set to" if os.getenv("COCO_DIR") else "default"
        raise ValueError(
            f"No image found at <{image}>. Download the COCO 2017 train images "
            f"(http://images.cocodataset.org/zips/train2017.zip) and put the extracted folder "
            f"under COCO_DIR ({how}: {root})."
        )

    def user_parts(text: str) -> list[dict]:
        return [{"type": "image", "path": image} if line == "<image>" else {"type": "text", "text": line} for line in text.split("\n")]

    turns = []
    for turn in row["conversations"]:
        is_user = turn["from"] in ("human", "user")
        value = user_parts(turn["value"]) if is_user else [{"type": "text", "text": turn["value"]}]
        turns.append({**turn, "value": value})
    return {"conversations": turns}


def _preset(name: str, hf_path: str, split: str, **kw) -> tuple[str, DatasetConfig]:
    return name, DatasetConfig(name=name, hf_path=hf_path, split=split, **kw)


DATASET_CONFIGS: dict[str, DatasetConfig] = dict(
    [
        _preset("sharegpt", "Aeala/ShareGPT_Vicuna_unfiltered", "train"),
        _preset("ultrachat", "HuggingFaceH4/ultrachat_200k", "train_sft", normalize_fn=_ultrachat, prompt_field="prompt"),
        _preset("gsm8k", "openai/gsm8k", "train", subset="main", normalize_fn=_gsm8k, prompt_field="question"),
        _preset("magpie", "Magpie-Align/Magpie-Llama-3.1-Pro-300K-Filtered", "train", prompt_field="instruction"),
        _preset("nemotron", "nvidia/Llama-Nemotron-Post-Training-Dataset", "chat", subset="SFT", normalize_fn=_nemotron),
        # the vLLM server must be started with --allowed-local-media-path <COCO_DIR>
        _preset("sharegpt4v_coco", "Lin-Chen/ShareGPT4V", "train", subset="ShareGPT4V", filter_fn=_is_coco, normalize_fn=_sharegpt4v_coco),
        _preset("open-perfectblend", "mlabonne/open-perfectblend", "train"),
        _preset("hermes-fc", "NousResearch/hermes-function-calling-v1", "train", subset="func_calling"),
    ]
)
