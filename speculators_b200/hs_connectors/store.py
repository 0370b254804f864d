"""Integrity-checked sample store on top of any key/value client.

A sample is a dict of tensors published under ``<key>:<name>`` plus a JSON manifest
under ``<key>:meta`` that is written *last*: a reader that sees the manifest may
assume every tensor is complete.  The manifest carries shape, dtype and a CRC32 of
every tensor; readers verify all three.  A producer that fails publishes an error
manifest so consumers fail fast instead of timing out.  A failed write removes
whatever it had written.  Wire format and error taxonomy follow
hs_connectors/src/hs_connectors/mooncake_store.py:99-310, so a Mooncake cluster
can be shared with the reference.

The client is duck-typed (``put``, ``get``, ``put_tensor``, ``get_tensor``,
``batch_remove``); negative integer return codes are failures.  ``DictStoreClient``
is the in-process implementation used for tests and single-node runs.
"""

from __future__ import annotations

import json
import logging
import threading
import time
import zlib
from dataclasses import dataclass, fields
from typing import Any

import torch

log = logging.getLogger(__name__)

__all__ = [
    "DictStoreClient", "HiddenStatesStore", "MooncakeHiddenStatesStore", "MooncakeIntegrityError",
    "MooncakeStoreConfig", "NonFiniteTensorError", "assert_finite",
]

_MANIFEST_VERSION = 1


class MooncakeIntegrityError(RuntimeError):
    """An object was present in the store but failed an integrity check."""


class NonFiniteTensorError(MooncakeIntegrityError):
    """A producer tried to publish NaN or infinity."""


def _host(t: torch.Tensor) -> torch.Tensor:
    return t.detach().to("cpu").contiguous()


def _crc(t: torch.Tensor) -> str:
    raw = t.reshape(-1).view(torch.uint8).numpy()
    return f"{zlib.crc32(memoryview(raw)) & 0xFFFFFFFF:08x}"


def assert_finite(name: str, tensor: torch.Tensor) -> None:
    """Two reductions (``amin`` / ``amax`` propagate NaN and expose either
    infinity) instead of a full-size boolean temporary; call it while the data
    is still on the device."""
    if not tensor.is_floating_point() or tensor.numel() == 0:
        return
    if bool(torch.isfinite(torch.stack((tensor.amin(), tensor.amax()))).all()):
        return
    raise NonFiniteTensorError(
        f"Non-finite producer tensor {name!r}: shape={tuple(tensor.shape)}, dtype={tensor.dtype}, "
        f"nan_count={int(torch.isnan(tensor).sum())}, inf_count={int(torch.isinf(tensor).sum())}"
    )


def _check(op: str, key: str, result: Any) -> None:
    if isinstance(result, int) and not isinstance(result, bool) and result != 0:
        raise RuntimeError(f"Mooncake {op} failed for key={key} with status={result}")


@dataclass
class MooncakeStoreConfig:
    local_hostname: str = "localhost"
    metadata_server: str = "P2PHANDSHAKE"
    master_server_address: str = "127.0.0.1:50051"
    global_segment_size: int = 4 * 1024**3
    local_buffer_size: int = 2 * 1024**3
    protocol: str = "tcp"
    device_name: str = ""
    num_writer_threads: int = 4

    @classmethod
    def from_dict(cls, d: dict | None) -> "MooncakeStoreConfig":
        d = d or {}
        known = {f.name for f in fields(cls)}
        extra = set(d) - known
        if extra:
            log.warning("Unknown MooncakeStoreConfig keys ignored: %s", extra)
        return cls(**{k: v for k, v in d.items() if k in known})


class DictStoreClient:
    """Thread-safe in-process key/value client with the Mooncake call shapes."""

    def __init__(self) -> None:
        self._data: dict[str, Any] = {}
        self._lock = threading.Lock()

    def put(self, key: str, value: bytes) -> int:
        with self._lock:
            self._data[key] = bytes(value)
        return 0

    def get(self, key: str) -> bytes:
        with self._lock:
            return self._data.get(key, b"")

    def put_tensor(self, key: str, tensor: torch.Tensor) -> int:
        with self._lock:
            self._data[key] = tensor.clone()
        return 0

    def get_tensor(self, key: str):
        with self._lock:
            value = self._data.get(key)
        return value.clone() if isinstance(value, torch.Tensor) else None

    def batch_remove(self, keys: list[str], force: bool = False) -> list[int]:  # noqa: ARG002
        with self._lock:
            for k in keys:
                self._data.pop(k, None)
        return [0] * len(keys)


class HiddenStatesStore:
    def __init__(self, config: MooncakeStoreConfig | None = None, client: Any = None):
        self.config = config or MooncakeStoreConfig()
        self._store = client

    @property
    def is_setup(self) -> bool:
        return self._store is not None

    def setup(self) -> "HiddenStatesStore":
        if self._store is not None:
            return self
        try:
            from mooncake.store import MooncakeDistributedStore  # type: ignore[import-not-found]
        except ImportError as err:
            raise ImportError(
                "Mooncake is required for the Mooncake hidden-states backend. Install it with "
                "`pip install mooncake-transfer-engine` or `pip install mooncake-transfer-engine-cuda13`."
            ) from err
        c = self.config
        client = MooncakeDistributedStore()
        _check("setup", c.local_hostname, client.setup(
            c.local_hostname, c.metadata_server, c.global_segment_size, c.local_buffer_size, c.protocol, c.device_name,
            c.master_server_address,
        ))
        self._store = client
        return self

    def _client(self):
        if self._store is None:
            raise RuntimeError("call setup() first")
        return self._store

    # ---- producer -----------------------------------------------------------------
    def put_sample(self, key: str, tensors: dict[str, torch.Tensor]) -> None:
        client = self._client()
        staged = {name: _host(t) for name, t in tensors.items()}
        manifest = {
            "version": _MANIFEST_VERSION, "status": "ok",
            "tensors": {n: {"shape": list(t.shape), "dtype": str(t.dtype), "checksum": _crc(t)} for n, t in staged.items()},
        }
        meta_key = f"{key}:meta"
        written: list[str] = []
        try:
            for name, t in staged.items():
                tkey = f"{key}:{name}"
                result = client.put_tensor(tkey, t)
                written.append(tkey)
                _check("put_tensor", tkey, result)
            _check("put", meta_key, client.put(meta_key, json.dumps(manifest).encode()))
        except Exception:
            try:
                client.batch_remove([*written, meta_key], force=True)
            except Exception:  # noqa: BLE001
                log.exception("Failed to clean partial sample %s", key)
            raise

    def put_error(self, key: str, error: str) -> None:
        manifest = {"version": _MANIFEST_VERSION, "status": "error", "error": error[:4096], "tensors": {}}
        _check("put", f"{key}:meta", self._client().put(f"{key}:meta", json.dumps(manifest).encode()))

    # ---- consumer -----------------------------------------------------------------
    def get_sample(self, key: str, timeout: float = 120.0, poll_interval: float = 0.05) -> dict[str, torch.Tensor]:
        client = self._client()
        specs = self._parse_manifest(key, self._wait_for(f"{key}:meta", timeout, poll_interval))
        out = {}
        for name, spec in specs.items():
            t = client.get_tensor(f"{key}:{name}")
            if t is None:
                raise MooncakeIntegrityError(f"Mooncake tensor unavailable for key={key}:{name}")
            self._validate(key, name, t, spec)
            out[name] = t
        return out

    def delete_sample(self, key: str) -> None:
        client = self._client()
        raw = client.get(f"{key}:meta")
        if not raw:
            return
        try:
            names = list(json.loads(raw).get("tensors", {}))
        except (UnicodeDecodeError, json.JSONDecodeError, AttributeError, TypeError):
            log.warning("Corrupt manifest for key=%s; falling back to default tensor names", key)
            names = ["hidden_states", "token_ids"]
        keys = [f"{key}:{n}" for n in names] + [f"{key}:meta"]
        for k, status in zip(keys, client.batch_remove(keys, force=True), strict=True):
            _check("batch_remove", k, status)

    def _wait_for(self, key: str, timeout: float, poll_interval: float) -> bytes:
        client = self._client()
        deadline = time.monotonic() + timeout
        while True:
            raw = client.get(key)
            if raw:
                return raw
            if time.monotonic() >= deadline:
                raise TimeoutError(f"Timed out waiting for Mooncake key: {key}")
            time.sleep(poll_interval)

    @staticmethod
    def _parse_manifest(key: str, raw: bytes) -> dict[str, dict[str, Any]]:
        try:
            manifest = json.loads(raw)
        except (UnicodeDecodeError, json.JSONDecodeError) as err:
            raise MooncakeIntegrityError(f"Corrupt Mooncake manifest for key={key}: {err}") from err
        if not isinstance(manifest, dict):
            raise MooncakeIntegrityError(f"Invalid Mooncake manifest type for key={key}: {type(manifest).__name__}")
        if manifest.get("status") == "error":
            raise MooncakeIntegrityError(f"Mooncake producer rejected key={key}: {manifest.get('error', 'unknown producer error')}")
        if manifest.get("version") != _MANIFEST_VERSION:
            raise MooncakeIntegrityError(f"Unsupported Mooncake manifest version for key={key}: {manifest.get('version')!r}")
        specs = manifest.get("tensors")
        if not isinstance(specs, dict) or not specs:
            raise MooncakeIntegrityError(f"Mooncake manifest has no tensors for key={key}")
        return specs

    @staticmethod
    def _validate(key: str, name: str, tensor: torch.Tensor, spec: Any) -> None:
        if not isinstance(spec, dict):
            raise MooncakeIntegrityError(f"Invalid tensor manifest for key={key}:{name}: expected object, got {type(spec).__name__}")
        want_shape = tuple(spec.get("shape", ()))
        if tuple(tensor.shape) != want_shape:
            raise MooncakeIntegrityError(f"Mooncake shape mismatch for key={key}:{name}: expected={want_shape}, actual={tuple(tensor.shape)}")
        if str(tensor.dtype) != spec.get("dtype"):
            raise MooncakeIntegrityError(f"Mooncake dtype mismatch for key={key}:{name}: expected={spec.get('dtype')}, actual={tensor.dtype}")
        got = _crc(_host(tensor))
        if got != spec.get("checksum"):
            raise MooncakeIntegrityError(f"Mooncake checksum mismatch for key={key}:{name}: expected={spec.get('checksum')}, actual={got}")


MooncakeHiddenStatesStore = HiddenStatesStore
