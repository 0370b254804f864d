"""Turn raw conversation datasets into training rows ``(input_ids, loss_mask)``.

A conversation fans out to one row per assistant turn.  For assistant turn *j* the
row's ids are the render of ``conv[:j+1]``; the supervised region starts where that
render stops agreeing with the generation-prompt render of ``conv[:j]`` (what the
server would have been given before producing the turn).  When the generation prompt
itself differs from the recorded turn (a pre-filled reasoning scaffold), the common
prefix is used, provided the plain history render is still a prefix of both.

Rendering goes through a ``Renderer`` callable so the same code runs against the
verifier server's ``/render`` endpoint (production) or a local chat template
(``LocalTemplateRenderer``: offline runs and tests).  Rows that already carry
``input_ids``/``loss_mask`` skip rendering.

Reference surface: src/speculators/data_generation/preprocessing.py:71
(_normalize_conversation), :208 (_render_boundary_rows), :441 (_preprocess_batch),
:523 (build_speculator_training_dataset), :643 (load_raw_dataset), :726
(load_and_preprocess_dataset).
"""

from __future__ import annotations

import json
from collections.abc import Callable
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Any, Protocol

import torch

from speculators_b200.data_generation.configs import DATASET_CONFIGS
from speculators_b200.data_generation.logging_utils import PipelineLogger
from speculators_b200.data_generation.render_client import render_conversation
from speculators_b200.train.vocab_mapping import save_token_frequency_distribution

__all__ = [
    "BoundaryUnstableError", "EndpointRenderer", "LocalTemplateRenderer", "Renderer", "adapt_conversation_for_server",
    "boundary_rows", "build_speculator_training_dataset", "get_tokenizer", "load_and_preprocess_dataset", "load_processor",
    "load_raw_dataset", "normalize_conversation", "preprocess_batch",
]

log = PipelineLogger(__name__)
_ROLE_ALIASES = {"human": "user", "user": "user", "gpt": "assistant", "assistant": "assistant", "system": "system", "tool": "tool"}
_unknown_roles_seen: set[str] = set()


class BoundaryUnstableError(ValueError):
    """The chat template re-renders earlier turns differently once a turn is appended."""


# ----------------------------------------------------------------------------- renderers
class Renderer(Protocol):
    def __call__(self, messages: list[dict], *, add_generation_prompt: bool, tools: list | None) -> list[int]: ...


class EndpointRenderer:
    """Renders through a running verifier server."""

    def __init__(self, endpoint: str):
        self.endpoint = endpoint

    def __call__(self, messages, *, add_generation_prompt, tools=None):
        return render_conversation(
            self.endpoint, adapt_conversation_for_server(messages), add_generation_prompt=add_generation_prompt, tools=tools
        )


class LocalTemplateRenderer:
    """Renders with a tokenizer/processor's own ``apply_chat_template`` (text only)."""

    def __init__(self, processor):
        self.tokenizer = get_tokenizer(processor)

    def __call__(self, messages, *, add_generation_prompt, tools=None):
        out = self.tokenizer.apply_chat_template(messages, tools=tools, add_generation_prompt=add_generation_prompt, tokenize=True)
        if isinstance(out, dict) or hasattr(out, "input_ids"):
            out = out["input_ids"]
        return list(out)


# ----------------------------------------------------------------------------- conversation shape
def normalize_conversation(conv: list[dict]) -> list[dict]:
    """Map ``from/value`` or ``role/content`` turns onto ``role/content`` with roles in
    {user, assistant, system, tool}; unknown roles (model names in on-policy dumps) count
    as assistant.  Tool-call fields and reasoning text are carried along."""
    out = []
    for turn in conv:
        raw = turn.get("from", turn.get("role", ""))
        role = _ROLE_ALIASES.get(raw)
        if role is None:
            if raw not in _unknown_roles_seen:
                _unknown_roles_seen.add(raw)
                log.warning(f"Mapping unknown role '{raw}' -> 'assistant'")
            role = "assistant"
        item: dict[str, Any] = {"role": role, "content": turn.get("value") or turn.get("content") or ""}
        for key in ("tool_calls", "tool_call_id"):
            if turn.get(key):
                item[key] = turn[key]
        thinking = turn.get("thinking") or turn.get("reasoning_content")
        if thinking:
            item["thinking"] = item["reasoning_content"] = thinking
        out.append(item)
    return out


def _part_for_server(part: str | dict) -> dict:
    if isinstance(part, str):
        return {"type": "text", "text": part}
    kind = part["type"]
    if kind == "text":
        return {"type": "text", "text": part["text"]}
    if kind in ("image", "video", "audio"):
        if part.get("path"):
            url = f"file://{Path(part['path']).absolute()}"
        elif part.get("url"):
            url = part["url"]
        else:
            raise ValueError(f"{kind} part needs a 'path' or 'url': {part}")
        return {"type": f"{kind}_url", f"{kind}_url": {"url": url}}
    if kind.endswith("_url"):
        return part
    raise ValueError(f"Unsupported content part type: {kind}")


def adapt_conversation_for_server(conv: list[dict]) -> list[dict]:
    """OpenAI chat-completions wire format: media parts become ``*_url`` parts with
    ``file://`` URLs, string content stays a string."""
    out = []
    for turn in conv:
        content = turn["content"]
        if isinstance(content, list):
            content = [_part_for_server(p) for p in content]
        out.append({**turn, "content": content})
    return out


# ----------------------------------------------------------------------------- boundaries
def _shared_prefix(a: list[int], b: list[int]) -> int:
    n = 0
    for x, y in zip(a, b):
        if x != y:
            break
        n += 1
    return n


def boundary_rows(conv: list[dict], render: Renderer, max_length: int, *, tools: list | None = None) -> list[dict]:
    """One ``{"input_ids", "loss_mask", "conv"}`` row per assistant turn that has a
    context.  A turn whose context alone reaches ``max_length`` is skipped (a later
    turn may fit again when the template drops earlier reasoning)."""
    rows = []
    for j, turn in enumerate(conv):
        if j == 0 or turn["role"] != "assistant":
            continue
        prompt = render(conv[:j], add_generation_prompt=True, tools=tools)
        if len(prompt) >= max_length:
            continue
        full = render(conv[: j + 1], add_generation_prompt=False, tools=tools)
        if full[: len(prompt)] == prompt:
            start = len(prompt)
        else:
            start = _shared_prefix(prompt, full)
            history = render(conv[:j], add_generation_prompt=False, tools=tools)
            if full[: len(history)] != history or start < len(history):
                raise BoundaryUnstableError(f"prompt and full renders diverge inside the history at assistant turn {j}")
        rows.append({"input_ids": full, "loss_mask": [0] * start + [1] * (len(full) - start), "conv": conv[: j + 1]})
    return rows


def _parse_tools(value: object, idx: int) -> list | None:
    if not value:
        return None
    if isinstance(value, list):
        return value
    if not isinstance(value, str):
        log.warning(f"Non-string value in tools column for conversation {idx}: {type(value).__name__}, proceeding without tools")
        return None
    try:
        return json.loads(value)
    except json.JSONDecodeError as err:
        log.warning(f"Invalid JSON in tools column for conversation {idx}: {err}, proceeding without tools")
        return None


class _RowSink:
    """Clips, filters and tensorises rows; counts why rows were lost."""

    def __init__(self, max_length: int, minimum_valid_tokens: int | None, keep_messages: bool = False):
        self.max_length = max_length
        self.min_valid = minimum_valid_tokens
        self.out: dict[str, list] = {"input_ids": [], "loss_mask": [], "seq_len": []}
        if keep_messages:
            self.out["messages"] = []
        self.unsupervised = 0  # nothing supervised inside the window
        self.clipped = 0  # kept, but the response was cut

    def add(self, ids: list[int], mask: list[int], conv: list[dict] | None = None) -> bool:
        too_long = len(ids) > self.max_length
        ids, mask = ids[: self.max_length], mask[: self.max_length]
        valid = sum(mask)
        if valid == 0:
            self.unsupervised += 1
            return False
        if self.min_valid is not None and valid < self.min_valid:
            return False
        self.out["input_ids"].append(torch.tensor(ids, dtype=torch.long))
        self.out["loss_mask"].append(torch.tensor(mask, dtype=torch.long))
        self.out["seq_len"].append(len(ids))
        if "messages" in self.out and conv is not None:
            self.out["messages"].append(adapt_conversation_for_server(conv))
        self.clipped += too_long
        return True

    def report(self) -> None:
        if self.unsupervised:
            log.warning(
                f"Dropped {self.unsupervised} rows with no supervised tokens. If unexpected, raise --seq-length so "
                f"assistant responses are not truncated away."
            )
        if self.clipped:
            log.warning(
                f"Clipped {self.clipped} rows at --seq-length: their responses are cut, so the tail and closing tokens "
                f"are never supervised. Raise --seq-length to supervise whole responses."
            )


def preprocess_batch(
    examples: dict,
    is_multimodal: bool,
    render: Renderer | None,
    max_length: int,
    minimum_valid_tokens: int | None = None,
    render_threads: int = 8,
) -> dict[str, list]:
    """Columnar batch in, columnar rows out (``datasets.map(batched=True)`` shape)."""
    if "input_ids" in examples and "loss_mask" in examples:
        sink = _RowSink(max_length, minimum_valid_tokens)
        for ids, mask in zip(examples["input_ids"], examples["loss_mask"], strict=True):
            if len(ids) != len(mask):
                raise ValueError(f"Speculator-format row shape mismatch: input_ids={len(ids)}, loss_mask={len(mask)}")
            sink.add(list(ids), list(mask))
        sink.report()
        return sink.out
    if render is None:
        raise ValueError("a renderer (render endpoint) is required to convert conversations to training rows")
    sink = _RowSink(max_length, minimum_valid_tokens, keep_messages=is_multimodal)
    conversations = examples.get("conversations") or []
    if not conversations:
        log.warning(f"No conversations key found. Keys: {list(examples.keys())}")
        return sink.out
    tools_col = examples.get("tools")
    if tools_col is not None and len(tools_col) != len(conversations):
        log.warning(f"Tools column length ({len(tools_col)}) != conversations length ({len(conversations)}), proceeding without tools")
        tools_col = None

    def one(idx: int) -> list[dict] | None:
        conv = conversations[idx]
        if not conv or not isinstance(conv, list):
            return None
        norm = normalize_conversation(conv)
        if not norm:
            return None
        tools = _parse_tools(tools_col[idx], idx) if tools_col is not None else None
        try:
            return boundary_rows(norm, render, max_length, tools=tools)
        except Exception as err:  # noqa: BLE001 - templates raise arbitrary types; one bad row must not end the run
            log.error(f"Failed to process conversation {idx}: {type(err).__name__}: {err}")
            return []

    # renders are network round-trips: overlap them, keep the output order
    if render_threads > 1 and len(conversations) > 1:
        with ThreadPoolExecutor(max_workers=render_threads) as pool:
            rendered = list(pool.map(one, range(len(conversations))))
    else:
        rendered = [one(i) for i in range(len(conversations))]

    n_in = n_empty = 0
    for rows in rendered:
        if rows is None:
            continue
        n_in += 1
        kept = sum(sink.add(r["input_ids"], r["loss_mask"], r["conv"]) for r in rows)
        n_empty += kept == 0
    sink.report()
    if n_empty:
        log.warning(f"{n_empty}/{n_in} conversations produced no training rows (no assistant turn with context, unstable template, or fully truncated)")
    if len(sink.out["input_ids"]) > n_in:
        log.info(f"Per-turn fan-out: {n_in} conversations -> {len(sink.out['input_ids'])} rows")
    return sink.out


def _preprocess_batch(examples: dict, is_multimodal: bool, render_endpoint: str | None, max_length: int,
                      minimum_valid_tokens: int | None = None) -> dict[str, list]:
    """``preprocess_batch`` with the renderer given as a server URL
    (src/speculators/data_generation/preprocessing.py:441-447 takes the endpoint)."""
    render = EndpointRenderer(render_endpoint) if render_endpoint is not None else None
    return preprocess_batch(examples, is_multimodal, render, max_length, minimum_valid_tokens)


# ----------------------------------------------------------------------------- datasets
def _is_multimodal_processor(processor) -> bool:
    try:
        from transformers import ProcessorMixin
    except ImportError:  # pragma: no cover
        return False
    return isinstance(processor, ProcessorMixin)


def get_tokenizer(processor):
    return processor.tokenizer if _is_multimodal_processor(processor) else processor


def load_processor(target_model_path: str, *, trust_remote_code: bool = False):
    from transformers import AutoProcessor

    processor = AutoProcessor.from_pretrained(target_model_path, trust_remote_code=trust_remote_code)
    tok = get_tokenizer(processor)
    if tok.pad_token is None:
        tok.pad_token = tok.eos_token
    return processor


def build_speculator_training_dataset(
    dataset,
    processor,
    max_length: int = 2048,
    num_proc: int = 8,
    *,
    render_endpoint: str | None = None,
    renderer: Renderer | None = None,
    minimum_valid_tokens: int | None = None,
):
    """``datasets.Dataset`` of conversations (or pre-tokenised rows) -> dataset with ``input_ids``, ``loss_mask``, ``seq_len`` (and ``messages`` for
    multimodal processors).  Rows are stored as plain integer lists; readers
    convert to tensors themselves."""
    cols = dataset.column_names
    pretokenized = {"input_ids", "loss_mask"} <= set(cols)
    multimodal = _is_multimodal_processor(processor)
    if renderer is None and render_endpoint is not None:
        renderer = EndpointRenderer(render_endpoint)
    if pretokenized:
        log.info("Speculator-format rows: using their loss mask, skipping render")
    elif renderer is None:
        raise ValueError(
            "render_endpoint is required to convert natural-language conversations to training rows. "
            "Pass --render-endpoint pointing at the target model's server."
        )
    else:
        log.info("Deriving loss masks from render boundaries")

    def fn(examples):
        return preprocess_batch(examples, multimodal, renderer, max_length, minimum_valid_tokens)

    if len(dataset) == 0:
        from datasets import Dataset

        empty = {"input_ids": [], "loss_mask": [], "seq_len": []}
        out = Dataset.from_dict(empty)
    else:
        out = dataset.map(fn, batched=True, batch_size=1000, num_proc=num_proc if num_proc and num_proc > 1 else None,
                          remove_columns=cols, keep_in_memory=True)
    return out


def _load_hf_spec(spec: str):
    from datasets import load_dataset

    parts = spec.removeprefix("hf:").split(":")
    if len(parts) == 1:
        hf_id, subset, split = parts[0], None, "train"
    elif len(parts) == 2:
        hf_id, subset, split = parts[0], None, parts[1]
    elif len(parts) == 3:
        hf_id, subset, split = parts
    else:
        raise ValueError(f"Invalid hf: spec '{spec}'. Expected hf:<dataset_id>[:<subset>:<split>].")
    if not hf_id:
        raise ValueError(f"Invalid hf: spec '{spec}': missing dataset id.")
    if subset == "":
        raise ValueError(f"Invalid hf: spec '{spec}': empty subset.")
    if not split:
        raise ValueError(f"Invalid hf: spec '{spec}': empty split.")
    raw = load_dataset(hf_id, name=subset, split=split)
    if "conversations" not in raw.column_names:
        raise ValueError(
            f"HuggingFace dataset '{hf_id}' (split '{split}') is not in conversations format: expected a "
            f"'conversations' column but found {raw.column_names}."
        )
    return raw, None


def load_raw_dataset(train_data_path: str) -> tuple[Any, Callable[[dict], dict] | None]:
    """Resolve a data source: a ``.json``/``.jsonl`` file, a directory of them
    (recursive), a preset name, or ``hf:<id>[:<subset>:<split>]``.  Returns the raw
    dataset and the preset's row normaliser (``None`` when rows already hold
    ``conversations``)."""
    from datasets import load_dataset

    if train_data_path.endswith((".jsonl", ".json")):
        return load_dataset("json", data_files=train_data_path, split="train"), None
    path = Path(train_data_path)
    if path.is_dir():
        files = sorted(str(p) for p in (*path.rglob("*.json"), *path.rglob("*.jsonl")))
        if not files:
            raise ValueError(f"No .json/.jsonl files found in directory: {train_data_path}")
        return load_dataset("json", data_files=files, split="train"), None
    if train_data_path in DATASET_CONFIGS:
        cfg = DATASET_CONFIGS[train_data_path]
        raw = load_dataset(cfg.hf_path, name=cfg.subset, split=cfg.split)
        if cfg.filter_fn is not None:
            raw = raw.filter(cfg.filter_fn)
        return raw, cfg.normalize_fn
    if train_data_path.startswith("hf:"):
        return _load_hf_spec(train_data_path)
    raise ValueError(
        f"Unsupported dataset: {train_data_path}. Supported: local .json/.jsonl file, local directory of such files, "
        f"hf:<id>[:<subset>:<split>], or a preset {list(DATASET_CONFIGS)}."
    )


def visualize_sample(dataset, processor, idx: int = 0) -> str:
    """Decoded sample with supervised tokens in blue and context in grey."""
    row = dataset[idx]
    tok = get_tokenizer(processor)
    pieces, state = [], None
    for tid, flag in zip(torch.as_tensor(row["input_ids"]).tolist(), torch.as_tensor(row["loss_mask"]).tolist()):
        flag = bool(flag)
        if flag != state:
            pieces.append("\033[94m" if flag else "\033[90m")
            state = flag
        pieces.append(tok.decode([tid]))
    pieces.append("\033[0m")
    text = "".join(pieces)
    log.info(text)
    return text


def load_and_preprocess_dataset(
    target_model_path: str,
    train_data_paths: list[str],
    *,
    seq_length: int,
    build_dataset_num_proc: int = 8,
    seed: int = 0,
    max_samples: int | None = None,
    token_freq_path: Path | str = "./token_freq.pt",  # noqa: S107
    render_endpoint: str | None = None,
    renderer: Renderer | None = None,
    minimum_valid_tokens: int | None = None,
    allow_empty_output: bool = False,
    trust_remote_code: bool = False,
):
    """Load every source, render/mask it, concatenate, shuffle, cap at ``max_samples``,
    and write the token-frequency table used for draft-vocabulary selection.
    Returns ``(dataset, processor)``."""
    from datasets import concatenate_datasets

    if minimum_valid_tokens is not None and minimum_valid_tokens < 0:
        raise ValueError("minimum_valid_tokens must be >= 0")
    log.section("Starting dataset preprocessing")
    processor = load_processor(target_model_path, trust_remote_code=trust_remote_code)
    has_template = hasattr(processor, "apply_chat_template") and getattr(processor, "chat_template", None) is not None
    parts = []
    for src in train_data_paths:
        log.subsection(f"Processing {src}")
        raw, normalize = load_raw_dataset(src)
        raw = raw.shuffle(seed=seed)
        if max_samples is not None and len(raw) > 3 * max_samples:
            raw = raw.select(range(3 * max_samples))  # enough head-room for rows lost to filtering
        if normalize is not None:
            raw = raw.map(normalize, num_proc=build_dataset_num_proc, keep_in_memory=True)
        pretokenized = {"input_ids", "loss_mask"} <= set(raw.column_names)
        if not pretokenized and not has_template:
            raise ValueError(
                f"Processor for {target_model_path} does not support chat templates. Use a model with a chat "
                f"template or provide pre-tokenized input_ids and loss_mask columns."
            )
        log.info(f"Loaded {len(raw)} samples")
        built = build_speculator_training_dataset(
            raw, processor, seq_length, build_dataset_num_proc, render_endpoint=render_endpoint, renderer=renderer,
            minimum_valid_tokens=minimum_valid_tokens,
        )
        if minimum_valid_tokens is not None:
            log.info(f"Kept {len(built)} samples after filtering")
        parts.append(built)
    combined = concatenate_datasets(parts).shuffle(seed=seed)
    if max_samples is not None and len(combined) > max_samples:
        combined = combined.select(range(max_samples))
    if len(combined) == 0 and not allow_empty_output:
        raise ValueError(
            "No samples remain after preprocessing. Check the dataset schema, assistant masking, and "
            "--minimum-valid-tokens. Pass --allow-empty-output if an empty dataset is intentional."
        )
    log.subsection("Computing token frequency distribution")
    save_token_frequency_distribution(combined, str(token_freq_path))
    if len(combined):
        visualize_sample(combined, processor, 0)
    else:
        log.warning("No samples remain after preprocessing; skipping visualization")
    log.section("Dataset preprocessing complete")
    return combined, processor
