"""On-policy response regeneration: replay the user/system turns of a dataset against
the target model's chat endpoint and record, for every generation of the target (a tool
call or a final answer), one training row ``(input_ids, loss_mask)`` whose mask is the
generation boundary reported by the server (prompt token ids -> 0, completion token
ids -> 1; the endpoint must honour ``return_token_ids``).

Tool calls are not executed: the i-th regenerated call of a conversation is answered with
the i-th tool result cached in the source row, provided there is exactly one call and it
names the tool that result belongs to; otherwise the conversation is cut after the call
(rows written so far are kept).

Reference surface: scripts/response_regeneration/script.py (extract_conversation:191,
extract_tools:260, load_seen:327, _sample_from_response:469, regenerate_conversation:538,
worker:658).
"""

from __future__ import annotations

import asyncio
import hashlib
import json
import os
import re
import time
from collections import deque
from collections.abc import Awaitable, Callable, Iterable
from dataclasses import dataclass, field
from typing import Any

from speculators_b200.data_generation.configs import DATASET_CONFIGS, DatasetConfig

__all__ = [
    "MULTIMODAL_DATASETS", "REGEN_DATASETS", "RegenStats", "boundary_sample", "extract_conversation", "extract_tools", "prepare_row",
    "load_seen", "prepare_item", "primary_identifier", "regenerate_conversation", "run_regeneration", "sanitize_filename",
    "tool_result_names",
]

# regeneration is text-only; multimodal responses are produced elsewhere and converted by prepare_data.py
MULTIMODAL_DATASETS = frozenset({"sharegpt4v_coco"})
REGEN_DATASETS = [name for name in DATASET_CONFIGS if name not in MULTIMODAL_DATASETS]
_TOOL_RESPONSE = re.compile(r"<tool_response>\s*(.*?)\s*</tool_response>", re.DOTALL)


def sanitize_filename(name: str) -> str:
    return re.sub(r'[/\\:*?"<>|]', "_", name).replace(" ", "_").strip("._")


# ----------------------------------------------------------------------------- row ingestion
def _json_or_none(value: Any):
    try:
        return json.loads(value)
    except (TypeError, json.JSONDecodeError):
        return None


def tool_result_names(content: Any) -> list[str]:
    """Names inside the ``<tool_response>{"name": ...}</tool_response>`` blocks of a cached
    tool result; empty when none can be read (which disables the name check)."""
    if not isinstance(content, str):
        return []
    names = []
    for block in _TOOL_RESPONSE.findall(content):
        obj = _json_or_none(block)
        if isinstance(obj, dict) and isinstance(obj.get("name"), str):
            names.append(obj["name"])
    return names


def extract_conversation(row: dict, prompt_field: str | None) -> tuple[list[dict], list[tuple[Any, list[str]]]]:
    """``(turns, tool_results)``: the system/user turns to replay (assistant turns are
    dropped: they get regenerated) and the cached ``(content, tool names)`` of every tool
    turn.  Rows without a user turn fall back to a single turn from ``prompt_field``."""
    msgs = row.get("messages")
    if not (isinstance(msgs, list) and msgs):
        msgs = row.get("conversations")
    turns, results = [], []
    for m in msgs if isinstance(msgs, list) else []:
        if not isinstance(m, dict):
            continue
        role = m.get("role") or m.get("from")
        role = "user" if role in ("user", "human") else role
        content = m.get("content") if m.get("content") is not None else m.get("value")
        if role in ("system", "user") and content:
            turns.append({"role": role, "content": content})
        elif role == "tool" and content is not None:
            results.append((content, tool_result_names(content)))
    if any(t["role"] == "user" for t in turns):
        return turns, results
    prompt = row.get(prompt_field) if prompt_field else None
    return ([{"role": "user", "content": prompt}], []) if prompt else ([], [])


def extract_tools(row: dict) -> list | None:
    """OpenAI-style tool schema of a row (a list, or its JSON string); ``None`` for a
    tool-free row; ``ValueError`` for a tools field that cannot be read as a list."""
    value = row.get("tools")
    if isinstance(value, str):
        value = _json_or_none(value)
    if isinstance(value, list) and value:
        return value
    if row.get("tools") not in (None, "", [], {}):
        raise ValueError("a tools field is present but not a usable list")
    return None


def primary_identifier(row: dict) -> str:
    """``id`` / ``uuid`` when present, else a content hash: stable under reordering,
    ``--limit`` and filters, so resuming skips exactly the finished conversations."""
    for key in ("id", "uuid"):
        if row.get(key) not in (None, ""):
            return str(row[key])
    blob = json.dumps(row, sort_keys=True, ensure_ascii=False, default=str)
    return "hash_" + hashlib.sha256(blob.encode("utf-8")).hexdigest()


def prepare_row(row: dict, config: DatasetConfig) -> tuple[dict, list[dict], list] | None:
    """``(normalised row, turns to replay, cached tool results)`` of one dataset row, or ``None``
    when the preset's filter drops it.  The preset's ``normalize_fn`` output is laid over the
    raw row (as ``datasets.map`` merges columns), so raw fall-back fields stay readable."""
    if config.filter_fn is not None and not config.filter_fn(row):
        return None
    norm = {**row, **config.normalize_fn(row)} if config.normalize_fn else row
    turns, results = extract_conversation(norm, config.prompt_field)
    return norm, turns, results


def prepare_item(row: dict, config: DatasetConfig, idx: int) -> dict | None:
    """Work item for one dataset row, or ``None`` to skip it (filtered / nothing to ask)."""
    prepared = prepare_row(row, config)
    if prepared is None or not prepared[1]:
        return None
    norm, turns, results = prepared
    return {"idx": idx, "primary_id": primary_identifier(row), "turns": turns, "tools": extract_tools(norm), "tool_results": results}


def load_seen(path: str) -> set[str]:
    """Conversation ids already present in an output file (``primary_id``, or ``id`` for
    files written before rows were fanned out per generation)."""
    seen: set[str] = set()
    if not os.path.isfile(path):
        return seen
    with open(path, encoding="utf-8") as fh:
        for line in fh:
            try:
                obj = json.loads(line)
            except json.JSONDecodeError:
                continue
            key = obj.get("primary_id")
            if key in (None, ""):
                key = obj.get("id")
            if key not in (None, ""):
                seen.add(str(key))
    return seen


# ----------------------------------------------------------------------------- regeneration
def boundary_sample(prompt_token_ids: list[int], completion_token_ids: list[int]) -> tuple[list[int], list[int]]:
    return [*prompt_token_ids, *completion_token_ids], [0] * len(prompt_token_ids) + [1] * len(completion_token_ids)


def _row_from_response(data: dict, *, conv_id: str, n: int, idx: int, endpoint: str, sampling_params: dict,
                       detokenize: Callable[[list[int]], str] | None) -> tuple[dict, dict, list | None]:
    choice = data["choices"][0]
    msg = choice["message"]
    content, calls = msg.get("content"), msg.get("tool_calls")
    if not content and not calls:
        raise ValueError(f"empty assistant generation (sample {n})")
    prompt_ids, completion_ids = data.get("prompt_token_ids"), choice.get("token_ids")
    if not prompt_ids or not completion_ids:
        raise ValueError("endpoint returned no token ids; it must support return_token_ids")
    ids, mask = boundary_sample(prompt_ids, completion_ids)
    reply: dict[str, Any] = {"role": "assistant", "content": content or ""}
    if calls:
        reply["tool_calls"] = calls
    row = {
        "id": f"{conv_id}_gen{n}", "primary_id": conv_id, "input_ids": ids, "loss_mask": mask,
        "text": detokenize(ids) if detokenize else None,  # for review only, training ignores it
        "metadata": {"idx": idx, "finish_reason": choice.get("finish_reason"), "is_tool_call": bool(calls),
                     "usage": data.get("usage") or {}, "endpoint": endpoint, "sampling_params": sampling_params},
    }
    return row, reply, calls


async def regenerate_conversation(post: Callable[[dict], Awaitable[dict]], item: dict, *, model: str, max_tokens: int, endpoint: str = "",
                                  sampling_params: dict | None = None, samples: list[dict],
                                  detokenize: Callable[[list[int]], str] | None = None) -> bool:
    """Append one row per generation to ``samples`` (kept even if a later request
    raises); returns whether the conversation was cut at an unpairable tool call."""
    sampling_params = sampling_params or {}
    cached = deque(item.get("tool_results") or [])
    history: list[dict] = []
    for turn in item["turns"]:
        history.append({"role": turn["role"], "content": turn["content"]})
        if turn["role"] == "system":
            continue
        while True:  # a tool call splices its cached result and asks again; an answer ends the turn
            payload = {**sampling_params, "model": model, "messages": history, "max_tokens": max_tokens, "return_token_ids": True}
            if item.get("tools"):
                payload["tools"], payload["tool_choice"] = item["tools"], "auto"
            row, reply, calls = _row_from_response(
                await post(payload), conv_id=item["primary_id"], n=len(samples), idx=item["idx"], endpoint=endpoint,
                sampling_params=sampling_params, detokenize=detokenize,
            )
            samples.append(row)
            history.append(reply)
            if not calls:
                break
            if len(calls) != 1 or not cached:
                return True
            content, names = cached.popleft()
            if names and (calls[0].get("function") or {}).get("name") not in names:
                return True
            result = {"role": "tool", "content": content}
            if calls[0].get("id"):
                result["tool_call_id"] = calls[0]["id"]
            history.append(result)
    return False


# ----------------------------------------------------------------------------- driver
@dataclass
class RegenStats:
    ok: int = 0
    errors: int = 0
    truncated: int = 0
    requests: int = 0
    completion_tokens: int = 0
    request_s: float = 0.0
    started: float = field(default_factory=time.perf_counter)

    def summary(self) -> str:
        elapsed = time.perf_counter() - self.started
        text = (f"Pipeline complete in {elapsed:.1f}s: {self.ok + self.errors} conversations "
                f"({self.ok} ok, {self.errors} errors, {self.truncated} truncated)")
        if self.requests:
            text += (f"\nThroughput: {self.requests / max(elapsed, 1e-9):.1f} req/s, "
                     f"{int(self.completion_tokens / max(elapsed, 1e-9))} tok/s | "
                     f"Avg request latency: {self.request_s / self.requests * 1e3:.0f} ms")
        return text


async def run_regeneration(items: Iterable[dict], post: Callable[[dict], Awaitable[dict]], write: Callable[[dict], None], *,
                           model: str, max_tokens: int, concurrency: int = 64, endpoint: str = "", sampling_params: dict | None = None,
                           detokenize: Callable[[list[int]], str] | None = None, on_done: Callable[[RegenStats], None] | None = None) -> RegenStats:
    """Regenerate ``items`` with at most ``concurrency`` conversations in flight.  Rows of a
    conversation are written together when it ends (also the partial rows of one that
    failed midway are written, followed by an ``error`` record)."""
    stats = RegenStats()

    async def timed_post(payload: dict) -> dict:
        t0 = time.perf_counter()
        data = await post(payload)
        stats.requests += 1
        stats.request_s += time.perf_counter() - t0
        stats.completion_tokens += int((data.get("usage") or {}).get("completion_tokens") or 0)
        return data

    async def one(item: dict) -> None:
        rows: list[dict] = []
        try:
            cut = await regenerate_conversation(timed_post, item, model=model, max_tokens=max_tokens, endpoint=endpoint,
                                                sampling_params=sampling_params, samples=rows, detokenize=detokenize)
            stats.ok += 1
            stats.truncated += bool(cut)
        except Exception as err:  # noqa: BLE001 - one bad conversation must not stop the run
            stats.errors += 1
            rows.append({"id": f"{item['primary_id']}_error", "error": f"{type(err).__name__}: {err}", "metadata": {"idx": item["idx"]}})
        for row in rows:
            write(row)
        if on_done is not None:
            on_done(stats)

    pending: set[asyncio.Task] = set()
    for item in items:
        if len(pending) >= max(1, concurrency):
            _, pending = await asyncio.wait(pending, return_when=asyncio.FIRST_COMPLETED)
        pending.add(asyncio.create_task(one(item)))
    if pending:
        await asyncio.wait(pending)
    return stats
