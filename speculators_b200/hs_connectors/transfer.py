"""Hidden-state transfer between the verifier (producer) and the trainer (consumer).

``HiddenStatesTransfer`` is what a dataset worker talks to: fetch a cached sample
by index, fetch a freshly generated sample by the handle the producer returned,
then keep (``cache``) or drop (``delete``) it.  ``HiddenStatesBackend`` is the
plugin point the CLIs use: each backend contributes its own ``train.py`` /
``launch_vllm.py`` flags, builds its transfer object from parsed args and renders
the ``kv_transfer_config`` handed to ``vllm serve``.  Interface parity:
hs_connectors/src/hs_connectors/transfer.py:46-117; the ``file`` backend mirrors
:136-203 (``hs_<idx>.safetensors`` plus ``.lock`` files on a shared filesystem).
"""

from __future__ import annotations

import argparse
import fcntl
import os
import shutil
import time
from abc import ABC, abstractmethod
from collections.abc import Callable
from pathlib import Path
from typing import Any, ClassVar

import torch
from safetensors.torch import load_file

__all__ = ["FileBackend", "FileTransfer", "HiddenStatesBackend", "HiddenStatesTransfer", "wait_for_lock", "wait_for_lock_async"]


def wait_for_lock(lock_path: str, timeout: float = 10.0, poll_interval: float = 0.1) -> None:
    """Block until the producer has released ``lock_path`` (it holds an exclusive
    ``flock`` while writing), then remove the lock file.  ``TimeoutError`` after
    ``timeout`` seconds."""
    fd = os.open(lock_path, os.O_RDWR)
    try:
        deadline = time.monotonic() + timeout
        while True:
            try:
                fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
                break
            except BlockingIOError:
                if time.monotonic() >= deadline:
                    raise TimeoutError(f"Timed out waiting for lock: {lock_path}") from None
                time.sleep(poll_interval)
    finally:
        os.close(fd)
    try:
        os.remove(lock_path)
    except FileNotFoundError:
        pass


async def wait_for_lock_async(lock_path: str, timeout: float = 10.0, poll_interval: float = 0.1) -> None:
    """``wait_for_lock`` for event-loop callers: polls the producer's ``flock`` without
    blocking the loop; ``TimeoutError`` (``asyncio.TimeoutError``) after ``timeout`` seconds."""
    import asyncio

    fd = os.open(lock_path, os.O_RDWR)

    async def poll() -> None:
        while True:
            try:
                fcntl.flock(fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
                return
            except BlockingIOError:
                await asyncio.sleep(poll_interval)

    try:
        await asyncio.wait_for(poll(), timeout=timeout)
    finally:
        os.close(fd)
    try:
        os.remove(lock_path)
    except FileNotFoundError:
        pass


class HiddenStatesTransfer(ABC):
    def setup(self) -> None:  # noqa: B027
        """Lazy initialisation; safe to call inside a dataloader worker."""

    @abstractmethod
    def get_cached(self, file_idx: int) -> dict[str, torch.Tensor] | None: ...

    @abstractmethod
    def get_generated(self, handle: str) -> dict[str, torch.Tensor] | None: ...

    def cache(self, handle: str, file_idx: int) -> None:  # noqa: B027
        """Persist a generated sample under its dataset index."""

    def delete(self, handle: str) -> None:  # noqa: B027
        """Drop a generated sample."""

    def request_params(self) -> dict | None:
        """``kv_transfer_params`` to send with a generation request (what the server-side
        connector needs to know about this consumer); ``None``: nothing to send."""
        return None


class HiddenStatesBackend(ABC):
    registry: ClassVar[dict[str, type["HiddenStatesBackend"]]] = {}

    @classmethod
    def register(cls, name: str) -> Callable[[type["HiddenStatesBackend"]], type["HiddenStatesBackend"]]:
        def decorator(subclass: type["HiddenStatesBackend"]) -> type["HiddenStatesBackend"]:
            if name in cls.registry:
                raise ValueError(f"Backend '{name}' is already registered.")
            cls.registry[name] = subclass
            return subclass

        return decorator

    @staticmethod
    @abstractmethod
    def add_train_args(parser: argparse.ArgumentParser) -> None: ...

    @staticmethod
    @abstractmethod
    def add_launch_args(parser: argparse.ArgumentParser) -> None: ...

    @staticmethod
    @abstractmethod
    def from_train_args(args: argparse.Namespace, data_path: str) -> HiddenStatesTransfer: ...

    @staticmethod
    @abstractmethod
    def build_kv_transfer_config(args: argparse.Namespace) -> dict[str, Any]: ...


def _load_when_unlocked(path: Path) -> dict[str, torch.Tensor] | None:
    lock = str(path) + ".lock"
    if os.path.exists(lock):
        wait_for_lock(lock)
    return load_file(path) if path.exists() else None


class FileTransfer(HiddenStatesTransfer):
    def __init__(self, hidden_states_path: Path | str):
        self.hidden_states_path = Path(hidden_states_path)

    def _cached_path(self, file_idx: int) -> Path:
        return self.hidden_states_path / f"hs_{file_idx}.safetensors"

    def get_cached(self, file_idx: int) -> dict[str, torch.Tensor] | None:
        return _load_when_unlocked(self._cached_path(file_idx))

    def get_generated(self, handle: str) -> dict[str, torch.Tensor] | None:
        return _load_when_unlocked(Path(handle))

    def cache(self, handle: str, file_idx: int) -> None:
        self.hidden_states_path.mkdir(parents=True, exist_ok=True)
        shutil.move(handle, self._cached_path(file_idx))

    def delete(self, handle: str) -> None:
        Path(handle).unlink()


@HiddenStatesBackend.register("file")
class FileBackend(HiddenStatesBackend):
    @staticmethod
    def add_train_args(parser: argparse.ArgumentParser) -> None:
        parser.add_argument("--hidden-states-path", type=str, default=None,
                            help="Directory of cached hidden-state files (default: <data_path>/hidden_states).")

    @staticmethod
    def add_launch_args(parser: argparse.ArgumentParser) -> None:
        parser.add_argument("--hidden-states-path", type=str, default="/tmp/hidden_states",  # noqa: S108
                            help="Directory the verifier writes hidden states to. Default '/tmp/hidden_states'.")

    @staticmethod
    def from_train_args(args: argparse.Namespace, data_path: str) -> FileTransfer:
        explicit = getattr(args, "hidden_states_path", None)
        return FileTransfer(Path(explicit) if explicit else Path(data_path) / "hidden_states")

    @staticmethod
    def build_kv_transfer_config(args: argparse.Namespace) -> dict[str, Any]:
        return {
            "kv_connector": "ExampleHiddenStatesConnector",
            "kv_role": "kv_producer",
            "kv_connector_extra_config": {"shared_storage_path": args.hidden_states_path},
        }
