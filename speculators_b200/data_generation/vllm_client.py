"""Client side of hidden-state generation against an OpenAI-compatible verifier
server: one ``max_tokens=1`` request per sample; the response carries the handle
(file path or store key) under ``kv_transfer_params``.

Retry policy (src/speculators/data_generation/vllm_client.py:28-91): up to
``max_retries`` extra attempts with ``2**attempt`` seconds of back-off; an
``InvalidResponseError`` (the server answered, but wrongly: token mismatch, no
handle) is deterministic and never retried.
"""

from __future__ import annotations

import asyncio
import functools
import logging
import time
from typing import Any, TypedDict

log = logging.getLogger(__name__)

DEFAULT_REQUEST_TIMEOUT = 120  # seconds
DEFAULT_MAX_RETRIES = 3
RETRY_BACKOFF_BASE = 2  # seconds

__all__ = [
    "DEFAULT_MAX_RETRIES", "DEFAULT_REQUEST_TIMEOUT", "ClientItem", "InvalidResponseError", "extract_output",
    "generate_hidden_states", "generate_hidden_states_async", "with_retries",
]


class InvalidResponseError(Exception):
    pass


class ClientItem(TypedDict, total=False):
    input_ids: list[int]
    messages: list[dict]  # only for multimodal conversations (chat completions re-tokenises)
from speculators_b200.hs_connectors.transfer import wait_for_lock, wait_for_lock_async  # noqa: E402,F401 - reference exposes them here too


def _backoff_or_raise(err: Exception, attempt: int, total: int) -> float | None:
    if isinstance(err, InvalidResponseError):
        raise err
    if attempt < total:
        delay = RETRY_BACKOFF_BASE**attempt
        log.warning("Request aborted (attempt %d/%d): %s. Retrying in %ds...", attempt, total, err, delay)
        return delay
    log.error("Request timed out after %d attempts: %s", total, err)
    return None


def with_retries(fn):
    """Adds a ``max_retries`` keyword (default 3) to a sync or async callable."""
    if asyncio.iscoroutinefunction(fn):
        @functools.wraps(fn)
        async def awrapper(*args, max_retries=DEFAULT_MAX_RETRIES, **kwargs):
            total = max_retries + 1
            last: Exception | None = None
            for attempt in range(1, total + 1):
                try:
                    return await fn(*args, **kwargs)
                except Exception as err:  # noqa: BLE001
                    last = err
                    delay = _backoff_or_raise(err, attempt, total)
                    if delay is not None:
                        await asyncio.sleep(delay)
            raise last  # type: ignore[misc]

        return awrapper

    @functools.wraps(fn)
    def wrapper(*args, max_retries=DEFAULT_MAX_RETRIES, **kwargs):
        total = max_retries + 1
        last: Exception | None = None
        for attempt in range(1, total + 1):
            try:
                return fn(*args, **kwargs)
            except Exception as err:  # noqa: BLE001
                last = err
                delay = _backoff_or_raise(err, attempt, total)
                if delay is not None:
                    time.sleep(delay)
        raise last  # type: ignore[misc]

    return wrapper


def extract_output(response: Any, token_ids: list[int]) -> str:
    """Validate the echo of the prompt and return the hidden-state handle."""
    choices = getattr(response, "choices", None)
    prompt_ids = getattr(choices[0], "prompt_token_ids", None) if choices else None
    if prompt_ids is None:
        prompt_ids = getattr(response, "prompt_token_ids", None)
    if prompt_ids is None:
        raise InvalidResponseError("Response missing prompt_token_ids")
    if list(prompt_ids) != list(token_ids):
        raise InvalidResponseError(f"Prompt token IDs mismatch: expected {token_ids}, got {prompt_ids}")
    params = getattr(response, "kv_transfer_params", None)
    if params is None:
        raise InvalidResponseError("Response missing kv_transfer_params")
    handle = params.get("hidden_states_path") or params.get("handle")
    if handle is None:
        raise InvalidResponseError("Response kv_transfer_params missing both 'hidden_states_path' and 'handle'")
    return handle


def _leave_final_turn_open(model: str) -> bool:
    # Mistral templates append a spurious EOS when the last assistant turn is closed
    return "mistral" in model.rsplit("/", 1)[-1].lower()


def _request(model: str, item: ClientItem, timeout: float | None, kv_transfer_params: dict | None = None) -> tuple[str, dict]:
    extra: dict[str, Any] = {"return_token_ids": True}
    if kv_transfer_params:
        extra["kv_transfer_params"] = dict(kv_transfer_params)
    if item.get("messages") is None:
        return "completions", dict(model=model, prompt=item["input_ids"], max_tokens=1, extra_body=extra, timeout=timeout)
    extra.update({"add_generation_prompt": False, "continue_final_message": _leave_final_turn_open(model)})
    return "chat", dict(model=model, messages=item["messages"], max_tokens=1, extra_body=extra, timeout=timeout)


@with_retries
def generate_hidden_states(client, model: str, client_item: ClientItem, *, timeout: float | None = DEFAULT_REQUEST_TIMEOUT,
                           kv_transfer_params: dict | None = None) -> str:
    kind, kwargs = _request(model, client_item, timeout, kv_transfer_params)
    res = client.completions.create(**kwargs) if kind == "completions" else client.chat.completions.create(**kwargs)
    return extract_output(res, client_item["input_ids"])


@with_retries
async def generate_hidden_states_async(client, model: str, client_item: ClientItem, *, timeout: float | None = DEFAULT_REQUEST_TIMEOUT,
                                       kv_transfer_params: dict | None = None) -> str:
    kind, kwargs = _request(model, client_item, timeout, kv_transfer_params)
    coro = client.completions.create(**kwargs) if kind == "completions" else client.chat.completions.create(**kwargs)
    res = await (asyncio.wait_for(coro, timeout=timeout) if timeout is not None else coro)
    return extract_output(res, client_item["input_ids"])
