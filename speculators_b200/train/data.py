"""Datasets and the packing collate function.

Three pieces, each usable on its own:

* ``RowWindow``: which rows of the preprocessed dataset a split owns, and the file index a
  row's hidden states are stored under (the index in the whole dataset, so train and
  validation share one hidden-state directory).
* ``HiddenStateResolver``: where a row's verifier hidden states come from: the cache of a
  ``HiddenStatesTransfer``, or a verifier server asked on the fly, governed by two policies
  (``on_missing``: generate | skip | warn | raise; ``on_generate``: cache | delete).
* ``ArrowDataset``: a Hugging Face dataset on disk (``input_ids``, ``loss_mask``, ``seq_len``
  [, ``messages``]) joined with the resolver.  Stored hidden states are ``[seq, layers, H]``:
  the last layer slot is the verifier's final hidden state, the others are concatenated into
  the draft's auxiliary input.

``CollateFn`` packs the samples of a batch into one ``[1, max_len, ...]`` row: it first plans
how many positions each sample contributes (clipping at ``max_len``), then fills every key from
that plan (zero padded, hidden states cast to the training dtype) and derives ``document_ids``
(0, 1, ... per sample, -1 for padding) from the same plan.  A batch with no usable sample
becomes one empty sample so every rank still steps.

Behaviour follows src/speculators/train/data.py:146-393 of the reference (dataset row format,
policies, warning texts, collate output keys).
"""

from __future__ import annotations

import warnings
from collections.abc import Callable, Sequence
from dataclasses import dataclass
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

__all__ = ["ArrowDataset", "BaseDataset", "BatchType", "CollateFn", "HiddenStateResolver", "RowWindow", "build_client_item",
           "create_empty_sample", "split_hidden_state_layers"]


# ---------------------------------------------------------------------------------------------
# sample-level helpers
# ---------------------------------------------------------------------------------------------
def create_empty_sample(hidden_size: int, num_target_layers: int = 3, dtype: torch.dtype = torch.bfloat16) -> BatchType:
    """A sample of zero tokens with the key set and trailing shapes of a real one."""
    widths = {"hidden_states": num_target_layers * hidden_size, "verifier_last_hidden_states": hidden_size}
    sample: BatchType = {k: torch.empty(0, w, dtype=dtype) for k, w in widths.items()}
    sample.update(input_ids=torch.empty(0, dtype=torch.long), loss_mask=torch.empty(0, dtype=torch.bool),
                  lengths=torch.zeros(1, dtype=torch.long), position_ids=torch.empty(0, dtype=torch.long))
    return sample


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


# ---------------------------------------------------------------------------------------------
# which rows a split owns
# ---------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class RowWindow:
    """Rows ``[start, stop)`` of a dataset of ``total`` rows."""

    start: int
    stop: int
    total: int

    @classmethod
    def of(cls, total: int, train_ratio: float, split: str) -> "RowWindow":
        if not 0.0 < train_ratio <= 1.0:
            raise ValueError(f"train_ratio must be in (0.0, 1.0], got {train_ratio}")
        if split == "val" and train_ratio == 1.0:
            raise ValueError("train_ratio=1.0 leaves no validation split")
        cut = int(total * train_ratio)
        window = cls(0, cut, total) if split == "train" else cls(cut, total, total)
        if len(window) <= 0:
            raise ValueError(f"{split} split is empty (dataset has {total} rows, train_ratio={train_ratio} gives split_idx={cut})")
        return window

    def __len__(self) -> int:
        return self.stop - self.start

    def file_index(self, index: int) -> int:
        """Index in the whole dataset (the name the hidden-state cache stores the row under)."""
        return int(index) + self.start


# ---------------------------------------------------------------------------------------------
# where hidden states come from
# ---------------------------------------------------------------------------------------------
class HiddenStateResolver:
    """Cached hidden states of a row, or freshly generated ones, or ``None`` - by policy.

    The verifier server is contacted on first use only (a dataset that finds every row cached
    never opens a connection); the model name the server reports must equal an explicitly
    requested one."""

    def __init__(self, transfer: HiddenStatesTransfer, endpoint: str, on_missing: str, on_generate: str, model: str | None,
                 request_timeout: float | None, max_retries: int):
        if on_missing not in ("generate", "skip", "warn", "raise"):
            raise ValueError(f"on_missing must be generate, skip, warn or raise, got {on_missing!r}")
        if on_generate not in ("cache", "delete"):
            raise ValueError(f"on_generate must be cache or delete, got {on_generate!r}")
        self.transfer, self.endpoint, self.on_missing, self.on_generate = transfer, endpoint, on_missing, on_generate
        self.model, self.request_timeout, self.max_retries = model, request_timeout, max_retries
        self.client = None

    # -- server ---------------------------------------------------------------------------------
    def connect(self) -> None:
        import openai

        self.client = openai.OpenAI(base_url=self.endpoint, api_key="EMPTY", max_retries=0)
        served = self.client.models.list().data[0].id
        if self.model and self.model != served:
            raise ValueError(
                f"An explicit model name was passed ({self.model}) which doesn't match found model_id {served}. "
                "Please make sure --endpoint is set to the correct vllm instance."
            )
        self.model = served
        self.transfer.setup()

    def generate(self, index: int, file_index: int, row: dict) -> dict[str, torch.Tensor] | None:
        """Ask the server for ``row``'s hidden states, verify them against its token ids, then keep
        or drop the server-side copy.  Any failure costs the sample, not the epoch."""
        try:
            if self.client is None:
                self.connect()
            handle = generate_hidden_states(self.client, self.model, build_client_item(row), timeout=self.request_timeout,
                                            max_retries=self.max_retries, kv_transfer_params=self.transfer.request_params())
            loaded = self.transfer.get_generated(handle)
            if loaded is None:
                raise ValueError(f"Failed to load hidden states for handle {handle}")
            check_hidden_states(loaded, row["input_ids"].tolist())
            (self.transfer.cache(handle, file_index) if self.on_generate == "cache" else self.transfer.delete(handle))
            return loaded
        except Exception as err:  # noqa: BLE001 - a failed sample must not kill the epoch
            warnings.warn(f"Failed to load/cache hidden states for sample {index}: {err}", stacklevel=1)
            return None

    # -- policy ---------------------------------------------------------------------------------
    def resolve(self, index: int, file_index: int, row_of: Callable[[], dict]) -> dict[str, torch.Tensor] | None:
        loaded = self.transfer.get_cached(file_index)
        if loaded is not None:
            return loaded
        if self.on_missing == "generate":
            return self.generate(index, file_index, row_of())
        if self.on_missing == "raise":
            raise RuntimeError(f"Failed to load hidden states for sample {index}.")
        if self.on_missing == "warn":
            warnings.warn(f"Failed to load hidden states for sample {index}. Skipping...", stacklevel=1)
        return None


# ---------------------------------------------------------------------------------------------
# datasets
# ---------------------------------------------------------------------------------------------
class BaseDataset(Dataset):
    """Sample = raw tensors + ``lengths`` / ``position_ids`` (+ ``transform``).  Subclasses give
    ``sample_lengths()`` (token counts used by the packing sampler) and ``load(index)`` (the raw
    tensors of a row, or ``None`` to drop it)."""

    def __init__(self, max_len: int, transform=None, hidden_states_dtype=torch.bfloat16):
        self.max_len, self.transform, self.hidden_states_dtype = max_len, transform, hidden_states_dtype
        self.approx_lengths = self.sample_lengths()

    def sample_lengths(self) -> list[int]:
        hook = getattr(self, "_compute_approx_lengths", None)  # the hook name datasets written for the reference define
        if hook is None:
            raise NotImplementedError
        return hook()

    def load(self, index: int) -> BatchType | None:
        hook = getattr(self, "_get_raw_data", None)  # likewise
        if hook is None:
            raise NotImplementedError
        return hook(index)

    def __getitem__(self, index) -> BatchType | None:
        data = self.load(index)
        if data is None:
            return None
        n = data["input_ids"].shape[0]
        data.update(lengths=torch.tensor([n], dtype=torch.long), position_ids=torch.arange(n, dtype=torch.long))
        return self.transform(data) if self.transform else data


class ArrowDataset(BaseDataset):
    def __init__(self, max_len: int, datapath: str | PathLike, transfer: HiddenStatesTransfer | None = None,
                 vllm_endpoint: str = "http://localhost:8000/v1", on_missing: Literal["generate", "skip", "warn", "raise"] = "generate",
                 on_generate: Literal["cache", "delete"] = "delete", train_ratio: float = 1.0, split: Literal["train", "val"] = "train",
                 transform=None, hidden_states_dtype=torch.bfloat16, model: str | None = None,
                 request_timeout: float | None = DEFAULT_REQUEST_TIMEOUT, max_retries: int = DEFAULT_MAX_RETRIES):
        from datasets import load_from_disk

        table = load_from_disk(str(datapath))
        self.window = RowWindow.of(len(table), train_ratio, split)
        # plain python rows (tensors are made in ``row``): the datasets "torch" formatter
        # drags in optional torchvision video readers
        self.data = table.select(range(self.window.start, self.window.stop)).with_format(None)
        self.resolver = HiddenStateResolver(transfer or FileTransfer(Path(datapath) / "hidden_states"), vllm_endpoint, on_missing,
                                            on_generate, model, request_timeout, max_retries)
        super().__init__(max_len, transform, hidden_states_dtype)

    # names other parts of the package (and users' scripts) read
    start_file_idx = property(lambda self: self.window.start)
    transfer = property(lambda self: self.resolver.transfer)

    def _map_to_file_idx(self, index: int) -> int:  # the reference's name for ``window.file_index``
        return self.window.file_index(index)

    def __len__(self) -> int:
        return len(self.window)

    def sample_lengths(self) -> list[int]:
        return [int(v) for v in self.data["seq_len"]]

    def row(self, index: int) -> dict:
        r = dict(self.data[int(index)])
        r["input_ids"] = torch.as_tensor(r["input_ids"], dtype=torch.long)
        r["loss_mask"] = torch.as_tensor(r["loss_mask"])
        return r

    def load(self, index: int) -> BatchType | None:
        cached_row: list[dict] = []

        def row_of() -> dict:
            if not cached_row:
                cached_row.append(self.row(index))
            return cached_row[0]

        loaded = self.resolver.resolve(index, self.window.file_index(index), row_of)
        if loaded is None:
            return None
        if not torch.equal(loaded["token_ids"].long(), row_of()["input_ids"]):
            warnings.warn(f"Loaded token ids for index {index} don't match the dataset's input ids", stacklevel=1)
            return None
        aux, last = split_hidden_state_layers(loaded["hidden_states"])
        return {"hidden_states": aux, "input_ids": loaded["token_ids"], "verifier_last_hidden_states": last, "loss_mask": row_of()["loss_mask"]}


# ---------------------------------------------------------------------------------------------
# packing
# ---------------------------------------------------------------------------------------------
class CollateFn:
    """Picklable (usable with spawned DataLoader workers)."""

    def __init__(self, max_len: int, hidden_size: int, num_target_layers: int = 3, dtype: torch.dtype = torch.bfloat16,
                 preprocess: Callable[[BatchType], BatchType] | None = None):
        self.max_len, self.hidden_size, self.num_target_layers = max_len, hidden_size, num_target_layers
        self.dtype, self.preprocess = dtype, preprocess

    def plan(self, lengths: Sequence[int]) -> list[tuple[int, int, int]]:
        """``(sample, offset in the packed row, positions taken)`` for the samples that fit;
        the one that crosses ``max_len`` is clipped and ends the row."""
        placed, used = [], 0
        for i, n in enumerate(lengths):
            take = min(int(n), self.max_len - used)
            placed.append((i, used, take))
            used += take
            if used >= self.max_len:
                break
        return placed

    def __call__(self, batch: Sequence[BatchType | None]) -> BatchType:
        pre = self.preprocess if self.preprocess is not None else (lambda s: s)
        samples = [pre(b) for b in batch if b is not None] or [pre(create_empty_sample(self.hidden_size, self.num_target_layers, dtype=self.dtype))]
        placed = self.plan([int(s["lengths"].sum()) for s in samples])
        out: BatchType = {}
        for key, first in samples[0].items():
            if key == "lengths":
                continue
            packed = torch.zeros((self.max_len, *first.shape[1:]), dtype=self.dtype if "hidden_states" in key else first.dtype)
            for i, at, take in placed:
                packed[at : at + take] = samples[i][key][:take]
            out[key] = packed.unsqueeze(0)
        doc = torch.full((self.max_len,), -1, dtype=torch.long)
        for i, at, take in placed:
            doc[at : at + take] = i
        out["document_ids"] = doc.unsqueeze(0)
        return out
