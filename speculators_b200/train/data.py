"""Datasets and the packing collate function.

``ArrowDataset`` reads a preprocessed Hugging Face dataset (``input_ids``,
``loss_mask``, ``seq_len`` [, ``messages``]) and pairs each row with verifier
hidden states from a ``HiddenStatesTransfer``: cached, or generated on the fly by a
verifier server (``on_missing``: generate | skip | warn | raise; ``on_generate``:
cache | delete).  Stored hidden states are ``[seq, layers, H]``: the last layer slot
is the verifier's final hidden state, the others are concatenated into the aux
input (src/speculators/train/data.py:146-304).

``CollateFn`` packs the samples of a batch into one ``[1, max_len, ...]`` row
(zero padded, hidden states cast to the training dtype), clips lengths at
``max_len`` and emits ``document_ids`` (0, 1, ... per sample, -1 for padding);
a batch with no usable sample becomes one empty sample so every rank still steps
(:306-393).
"""

from __future__ import annotations

import warnings
from collections.abc import Callable, Sequence
from os import PathLike
from pathlib import Path
from typing import Any, Literal

import torch
from torch.utils.data import Dataset

from speculators_b200.data_generation.offline import check_hidden_states
from speculators_b200.data_generation.vllm_client import (
    DEFAULT_MAX_RETRIES, DEFAULT_REQUEST_TIMEOUT, ClientItem, generate_hidden_states,
)
from speculators_b200.hs_connectors import FileTransfer, HiddenStatesTransfer

BatchType = dict[str, Any]

__all__ = ["ArrowDataset", "BaseDataset", "BatchType", "CollateFn", "build_client_item", "create_empty_sample", "split_hidden_state_layers"]


def create_empty_sample(hidden_size: int, num_target_layers: int = 3, dtype: torch.dtype = torch.bfloat16) -> BatchType:
    return {
        "hidden_states": torch.empty(0, num_target_layers * hidden_size, dtype=dtype),
        "input_ids": torch.empty(0, dtype=torch.long),
        "verifier_last_hidden_states": torch.empty(0, hidden_size, dtype=dtype),
        "loss_mask": torch.empty(0, dtype=torch.bool),
        "lengths": torch.tensor([0], dtype=torch.long),
        "position_ids": torch.arange(0, dtype=torch.long),
    }


def build_client_item(dataset_item: dict) -> ClientItem:
    """Request payload for hidden-state extraction.  ``messages`` are forwarded only
    for multimodal conversations (content given as a list of typed parts): the
    chat endpoint re-tokenises the untruncated conversation, which is required
    for images but would overflow ``max_model_len`` for truncated text samples."""
    ids = dataset_item["input_ids"]
    item: dict = {"input_ids": ids.tolist() if hasattr(ids, "tolist") else [int(t) for t in ids]}
    messages = dataset_item.get("messages")
    if messages and any(isinstance(m.get("content"), list) for m in messages):
        item["messages"] = messages
    return item  # type: ignore[return-value]


def split_hidden_state_layers(stored: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``[seq, layers, H]`` -> (aux ``[seq, (layers-1)*H]``, last ``[seq, H]``)."""
    return stored[:, :-1].flatten(1), stored[:, -1]


class BaseDataset(Dataset):
    def __init__(self, max_len: int, transform=None, hidden_states_dtype=torch.bfloat16):
        self.max_len, self.transform, self.hidden_states_dtype = max_len, transform, hidden_states_dtype
        self.approx_lengths = self._compute_approx_lengths()

    def _compute_approx_lengths(self):
        raise NotImplementedError

    def _get_raw_data(self, index):
        raise NotImplementedError

    def __getitem__(self, index) -> BatchType | None:
        data = self._get_raw_data(index)
        if data is None:
            return None
        n = data["input_ids"].shape[0]
        data["lengths"] = torch.tensor([n], dtype=torch.long)
        data["position_ids"] = torch.arange(n, dtype=torch.long)
        return self.transform(data) if self.transform else data


class ArrowDataset(BaseDataset):
    def __init__(self, max_len: int, datapath: str | PathLike, transfer: HiddenStatesTransfer | None = None,
                 vllm_endpoint: str = "http://localhost:8000/v1", on_missing: Literal["generate", "skip", "warn", "raise"] = "generate",
                 on_generate: Literal["cache", "delete"] = "delete", train_ratio: float = 1.0, split: Literal["train", "val"] = "train",
                 transform=None, hidden_states_dtype=torch.bfloat16, model: str | None = None,
                 request_timeout: float | None = DEFAULT_REQUEST_TIMEOUT, max_retries: int = DEFAULT_MAX_RETRIES):
        from datasets import load_from_disk

        data = load_from_disk(str(datapath))
        if not 0.0 < train_ratio <= 1.0:
            raise ValueError(f"train_ratio must be in (0.0, 1.0], got {train_ratio}")
        if split == "val" and train_ratio == 1.0:
            raise ValueError("train_ratio=1.0 leaves no validation split")
        cut = int(len(data) * train_ratio)
        start, stop = (0, cut) if split == "train" else (cut, len(data))
        if start >= stop:
            raise ValueError(f"{split} split is empty (dataset has {len(data)} rows, train_ratio={train_ratio} gives split_idx={cut})")
        self.start_file_idx = start
        # rows are converted to tensors here rather than through the datasets "torch"
        # formatter, which drags in optional torchvision video readers
        self.data = data.select(range(start, stop)).with_format(None)
        self.transfer = transfer or FileTransfer(Path(datapath) / "hidden_states")
        self.vllm_endpoint, self.on_missing, self.on_generate = vllm_endpoint, on_missing, on_generate
        self.client = None
        self.model, self.request_timeout, self.max_retries = model, request_timeout, max_retries
        super().__init__(max_len, transform, hidden_states_dtype)

    def __len__(self) -> int:
        return len(self.data)

    def _map_to_file_idx(self, index: int) -> int:
        return index + self.start_file_idx

    def _compute_approx_lengths(self) -> list[int]:
        return [int(v) for v in self.data["seq_len"]]

    def _row(self, index: int) -> dict:
        row = dict(self.data[int(index)])
        row["input_ids"] = torch.as_tensor(row["input_ids"], dtype=torch.long)
        row["loss_mask"] = torch.as_tensor(row["loss_mask"])
        return row

    def _setup_client(self) -> None:
        import openai

        self.client = openai.OpenAI(base_url=self.vllm_endpoint, api_key="EMPTY", max_retries=0)
        served = self.client.models.list().data[0].id
        if self.model and self.model != served:
            raise ValueError(
                f"An explicit model name was passed ({self.model}) which doesn't match found model_id {served}. "
                "Please make sure --endpoint is set to the correct vllm instance."
            )
        self.model = served
        self.transfer.setup()

    def _maybe_generate_hs(self, index: int) -> dict[str, torch.Tensor] | None:
        if self.client is None:
            self._setup_client()
        row = self._row(index)
        try:
            handle = generate_hidden_states(self.client, self.model, build_client_item(row), timeout=self.request_timeout,
                                            max_retries=self.max_retries, kv_transfer_params=self.transfer.request_params())
            loaded = self.transfer.get_generated(handle)
            if loaded is None:
                raise ValueError(f"Failed to load hidden states for handle {handle}")
            check_hidden_states(loaded, row["input_ids"].tolist())
            if self.on_generate == "cache":
                self.transfer.cache(handle, self._map_to_file_idx(index))
            else:
                self.transfer.delete(handle)
        except Exception as err:  # noqa: BLE001 - a failed sample must not kill the epoch
            warnings.warn(f"Failed to load/cache hidden states for sample {index}: {err}", stacklevel=1)
            return None
        return loaded

    def _get_raw_data(self, index):
        loaded = self.transfer.get_cached(self._map_to_file_idx(index))
        if loaded is None:
            if self.on_missing == "generate":
                loaded = self._maybe_generate_hs(index)
            elif self.on_missing == "skip":
                return None
            elif self.on_missing == "warn":
                warnings.warn(f"Failed to load hidden states for sample {index}. Skipping...", stacklevel=1)
                return None
            else:
                raise RuntimeError(f"Failed to load hidden states for sample {index}.")
        if loaded is None:
            return None
        row = self._row(index)
        if not torch.equal(loaded["token_ids"].long(), row["input_ids"]):
            warnings.warn(f"Loaded token ids for index {index} don't match the dataset's input ids", stacklevel=1)
            return None
        aux, last = split_hidden_state_layers(loaded["hidden_states"])
        return {"hidden_states": aux, "input_ids": loaded["token_ids"], "verifier_last_hidden_states": last, "loss_mask": row["loss_mask"]}


class CollateFn:
    """Picklable (usable with spawned DataLoader workers)."""

    def __init__(self, max_len: int, hidden_size: int, num_target_layers: int = 3, dtype: torch.dtype = torch.bfloat16,
                 preprocess: Callable[[BatchType], BatchType] | None = None):
        self.max_len, self.hidden_size, self.num_target_layers = max_len, hidden_size, num_target_layers
        self.dtype, self.preprocess = dtype, preprocess

    def __call__(self, batch: Sequence[BatchType | None]) -> BatchType:
        pre = self.preprocess
        samples = [pre(b) if pre else b for b in batch if b is not None]
        if not samples:
            empty = create_empty_sample(self.hidden_size, self.num_target_layers, dtype=self.dtype)
            samples = [pre(empty) if pre else empty]
        max_len = self.max_len
        out: BatchType = {}
        for key, first in samples[0].items():
            if key == "lengths":
                continue
            dtype = self.dtype if "hidden_states" in key else first.dtype
            buf = torch.zeros((max_len, *first.shape[1:]), dtype=dtype)
            filled = 0
            for s in samples:
                take = min(s[key].shape[0], max_len - filled)
                buf[filled : filled + take] = s[key][:take]
                filled += take
                if filled == max_len:
                    break
            out[key] = buf.unsqueeze(0)
        lengths: list[int] = []
        used = 0
        for n in torch.cat([s["lengths"] for s in samples]).tolist():
            if used + n >= max_len:
                lengths.append(max_len - used)
                used = max_len
                break
            lengths.append(n)
            used += n
        doc = torch.full((max_len,), -1, dtype=torch.long)
        doc[:used] = torch.repeat_interleave(torch.arange(len(lengths)), torch.tensor(lengths, dtype=torch.long))
        out["document_ids"] = doc.unsqueeze(0)
        return out
