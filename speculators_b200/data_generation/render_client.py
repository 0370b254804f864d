"""Tokenise a conversation with the verifier server's own chat template
(``POST <endpoint>/v1/chat/completions/render``), so the ids used for training are
the ids the server would produce at inference time.

Error policy: 4xx other than the transient ones (408, 425, 429) is a deterministic
client error -> ``InvalidResponseError`` (never retried); any other non-200 or a body
without ``token_ids`` -> ``RenderError`` (retried with back-off by ``with_retries``).

Reference surface: src/speculators/data_generation/render_client.py:23,28.
"""

from __future__ import annotations

import json
import urllib.error
import urllib.request

from speculators_b200.data_generation.vllm_client import InvalidResponseError, with_retries

__all__ = ["DEFAULT_RENDER_TIMEOUT", "TRANSIENT_STATUSES", "RenderError", "render_conversation"]

DEFAULT_RENDER_TIMEOUT = 60.0
TRANSIENT_STATUSES = frozenset({408, 425, 429})


class RenderError(Exception):
    """Retry-eligible failure of the render endpoint."""


def _post_json(url: str, body: dict, timeout: float) -> tuple[int, str]:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"}, method="POST")
    try:
        with urllib.request.urlopen(req, timeout=timeout) as resp:  # noqa: S310
            return resp.status, resp.read().decode("utf-8", "replace")
    except urllib.error.HTTPError as err:
        return err.code, err.read().decode("utf-8", "replace")


@with_retries
def render_conversation(
    endpoint: str,
    messages: list[dict],
    *,
    add_generation_prompt: bool,
    tools: list[dict] | None = None,
    chat_template_kwargs: dict | None = None,
    timeout: float = DEFAULT_RENDER_TIMEOUT,
) -> list[int]:
    """Token ids of ``messages`` under the server's chat template.  Never truncates:
    boundary detection needs the full lengths."""
    body: dict = {"messages": messages, "add_generation_prompt": add_generation_prompt}
    if tools is not None:
        body["tools"] = tools
    if chat_template_kwargs is not None:
        body["chat_template_kwargs"] = chat_template_kwargs
    status, text = _post_json(f"{endpoint.rstrip('/')}/v1/chat/completions/render", body, timeout)
    if 400 <= status < 500 and status not in TRANSIENT_STATUSES:
        raise InvalidResponseError(f"Render endpoint returned {status}: {text}")
    if status != 200:
        raise RenderError(f"Render endpoint returned {status}: {text}")
    try:
        data = json.loads(text)
    except json.JSONDecodeError as err:
        raise RenderError(f"Render endpoint returned a non-JSON body: {text[:200]}") from err
    if "token_ids" not in data:
        raise RenderError(f"Render endpoint response missing 'token_ids': {data}")
    return data["token_ids"]
