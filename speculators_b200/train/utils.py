"""Trainer-side helpers (parity: src/speculators/train/utils.py:71-150)."""

from __future__ import annotations

import datetime
import os
import shlex
import sys

from speculators_b200 import provenance

__all__ = ["normalize_counted_metrics", "resolve_mask_token_id", "save_train_command"]


def normalize_counted_metrics(metrics: dict[str, float], world_size: int = 1) -> dict[str, float]:
    """``x_sum`` / ``x_total`` pairs (already summed over ranks) become ``x``; keys
    without a partner were summed over ranks too, so they are averaged."""
    out: dict[str, float] = {}
    for key, value in metrics.items():
        if key.endswith("_sum"):
            base = key[: -len("_sum")]
            total = metrics.get(base + "_total")
            if total is not None:
                out[base] = value / total if total else 0.0
                continue
        if key.endswith("_total") and key[: -len("_total")] + "_sum" in metrics:
            continue
        out[key] = value / world_size
    return out


def save_train_command(save_dir: str | os.PathLike, argv: list[str] | None = None) -> str:
    """Write ``train_command.txt``: a provenance header (``# Timestamp:``, ``# Git SHA:``,
    ``# World size:``, one ``# <package>: <version>`` line per tracked package) followed by
    the shell-quoted command line.  ``argv`` is the command the run was resolved from;
    without it the live ``sys.argv`` is recorded.  The file is replaced atomically
    (src/speculators/train/utils.py:103-150)."""
    argv = list(argv or sys.argv)
    os.makedirs(save_dir, exist_ok=True)
    lines = [
        f"# Timestamp: {datetime.datetime.now(datetime.timezone.utc).isoformat()}",
        f"# Git SHA: {provenance.git_sha()}",
        f"# World size: {os.environ.get('WORLD_SIZE', '1')}",
    ]
    lines += provenance.package_versions()
    lines.append(shlex.join(argv))
    path = os.path.join(save_dir, "train_command.txt")
    provenance.atomic_write(path, "\n".join(lines) + "\n")
    return path


def resolve_mask_token_id(verifier_name_or_path: str, vocab_size: int, mask_token_id: int | None = None, *, trust_remote_code: bool = False) -> int:
    """Mask token for P-EAGLE / DFlash / DSpark.  Order: the explicit value; the
    tokenizer's own mask token; a new ``<|MASK|>`` token if the embedding table has
    unused rows; else pad / eos / unk (with a warning).  Passing ``--mask-token-id``
    avoids loading a tokenizer altogether (src/speculators/train/utils.py:17-68)."""
    import logging
    import warnings

    log = logging.getLogger("speculators")
    if mask_token_id is not None:
        log.info("Using explicit mask_token_id=%d", mask_token_id)
        return mask_token_id
    from transformers import AutoTokenizer

    tokenizer = AutoTokenizer.from_pretrained(verifier_name_or_path, trust_remote_code=trust_remote_code)
    if tokenizer.mask_token_id is not None:
        log.info("Using tokenizer mask_token_id=%d", tokenizer.mask_token_id)
        return tokenizer.mask_token_id
    if len(tokenizer) < vocab_size:
        tokenizer.add_special_tokens({"mask_token": "<|MASK|>"})
        log.warning("Added <|MASK|> to tokenizer, mask_token_id=%d (tokenizer len=%d, vocab_size=%d)", tokenizer.mask_token_id, len(tokenizer), vocab_size)
        return tokenizer.mask_token_id
    for name in ("pad_token_id", "eos_token_id", "unk_token_id"):
        token_id = getattr(tokenizer, name, None)
        if token_id is not None:
            warnings.warn(f"Tokenizer does not have mask_token and no unused embedding slots. Using {name}={token_id} as fallback.", stacklevel=2)
            return token_id
    raise ValueError(
        "Could not resolve mask_token_id: no --mask-token-id provided, tokenizer has no mask_token, no unused "
        "embedding slots, and no pad/eos/unk fallback tokens."
    )
