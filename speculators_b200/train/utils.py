"""Trainer-side helpers (parity: src/speculators/train/utils.py:71-150)."""

from __future__ import annotations

import datetime
import os
import shlex
import sys

from speculators_b200 import provenance

__all__ = ["normalize_counted_metrics", "save_train_command"]


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
    """Write ``train_command.txt``: timestamp, git revision, world size, package
    versions and the exact command line."""
    argv = list(sys.argv if argv is None else argv)
    os.makedirs(save_dir, exist_ok=True)
    lines = [
        f"# {datetime.datetime.now(datetime.timezone.utc).isoformat()}",
        f"# git: {provenance.git_sha() or 'unknown'}",
        f"# world_size: {os.environ.get('WORLD_SIZE', '1')}",
    ]
    lines += [f"# {pkg}=={ver}" for pkg, ver in provenance.package_versions().items()]
    lines.append(" ".join(shlex.quote(a) for a in [sys.executable, *argv]))
    path = os.path.join(save_dir, "train_command.txt")
    provenance.atomic_write(path, "\n".join(lines) + "\n")
    return path
