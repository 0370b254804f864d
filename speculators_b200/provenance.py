"""Run provenance: atomic file writes, git revision / diff of a checkout, package versions
(parity: src/speculators/provenance.py; same function signatures)."""

from __future__ import annotations

import importlib.metadata
import importlib.util
import os
import subprocess
import tempfile
from pathlib import Path

TRACKED_PACKAGES = ("speculators_b200", "vllm", "transformers", "torch", "safetensors", "datasets")

__all__ = ["TRACKED_PACKAGES", "atomic_write", "find_package_repo", "find_repo_root", "git_diff", "git_sha", "package_versions",
           "pkg_version", "run_git"]


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
    """Installed version of a distribution; this package answers from its own version module
    when it runs from a checkout; ``"not installed"`` otherwise."""
    if name == "speculators_b200":
        from speculators_b200.version import __version__

        return __version__
    try:
        return importlib.metadata.version(name)
    except importlib.metadata.PackageNotFoundError:
        return "not installed"


def package_versions(packages: tuple[str, ...] = TRACKED_PACKAGES) -> list[str]:
    """``["# pkg: version", ...]`` header lines."""
    return [f"# {p}: {pkg_version(p)}" for p in packages]


def find_repo_root(start: str | os.PathLike | None = None) -> Path | None:
    """The closest directory at or above ``start`` (default: this file) that holds ``.git``."""
    here = Path(start or __file__).resolve()
    for cand in (here, *here.parents):
        if (cand / ".git").exists():
            return cand
    return None


def find_package_repo(package_name: str) -> Path | None:
    """Git checkout an importable package lives in (editable installs), if any."""
    try:
        spec = importlib.util.find_spec(package_name)
    except (ModuleNotFoundError, ValueError):
        return None
    return find_repo_root(spec.origin) if spec is not None and spec.origin else None


def run_git(args: list[str], cwd: str | os.PathLike, *, timeout: int = 5) -> str:
    """stdout of a git command line (``args`` starts with ``"git"``), ``""`` on any failure."""
    try:
        res = subprocess.run(args, cwd=str(cwd), capture_output=True, text=True, timeout=timeout, check=False)
    except (OSError, subprocess.TimeoutExpired):
        return ""
    return res.stdout.strip() if res.returncode == 0 else ""


_OWN_CHECKOUT = object()


def git_sha(repo_root: str | os.PathLike | None = _OWN_CHECKOUT) -> str:  # type: ignore[assignment]
    """HEAD revision of ``repo_root`` (default: the checkout this package runs from);
    ``"unknown"`` when there is none or git fails."""
    root = find_repo_root() if repo_root is _OWN_CHECKOUT else repo_root
    if root is None:
        return "unknown"
    return run_git(["git", "rev-parse", "HEAD"], root) or "unknown"


def git_diff(repo_root: str | os.PathLike | None = _OWN_CHECKOUT, *, timeout: int = 30) -> str:  # type: ignore[assignment]
    """Uncommitted changes of ``repo_root`` against HEAD, ``""`` when clean or unavailable."""
    root = find_repo_root() if repo_root is _OWN_CHECKOUT else repo_root
    if root is None:
        return ""
    return run_git(["git", "diff", "HEAD"], root, timeout=timeout)
