"""Run provenance: atomic file writes, git revision / diff, package versions
(parity: src/speculators/provenance.py)."""

from __future__ import annotations

import importlib.metadata
import os
import subprocess
import tempfile
from pathlib import Path

TRACKED_PACKAGES = ("torch", "transformers", "safetensors", "numpy", "pydantic", "datasets")

__all__ = ["TRACKED_PACKAGES", "atomic_write", "find_repo_root", "git_diff", "git_sha", "package_versions", "pkg_version"]


def atomic_write(path: str | os.PathLike, text: str) -> None:
    """Write ``text`` so that readers see either the old or the new file, never a torn one."""
    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    fd, tmp = tempfile.mkstemp(dir=target.parent, prefix=target.name, suffix=".tmp")
    try:
        with os.fdopen(fd, "w") as fh:
            fh.write(text)
            fh.flush()
            os.fsync(fh.fileno())
        os.replace(tmp, target)
    except BaseException:
        if os.path.exists(tmp):
            os.unlink(tmp)
        raise


def pkg_version(name: str) -> str:
    try:
        return importlib.metadata.version(name)
    except importlib.metadata.PackageNotFoundError:
        return "unknown"


def package_versions() -> dict[str, str]:
    from speculators_b200.version import __version__

    out = {"speculators_b200": __version__}
    out.update({name: pkg_version(name) for name in TRACKED_PACKAGES})
    return out


def find_repo_root(start: str | os.PathLike | None = None) -> Path | None:
    here = Path(start or __file__).resolve()
    for cand in (here, *here.parents):
        if (cand / ".git").exists():
            return cand
    return None


def _git(*args: str) -> str | None:
    root = find_repo_root()
    if root is None:
        return None
    try:
        res = subprocess.run(["git", *args], cwd=root, capture_output=True, text=True, timeout=5, check=False)
    except (OSError, subprocess.TimeoutExpired):
        return None
    return res.stdout.strip() if res.returncode == 0 else None


def git_sha() -> str | None:
    return _git("rev-parse", "HEAD")


def git_diff() -> str | None:
    return _git("diff", "HEAD")
