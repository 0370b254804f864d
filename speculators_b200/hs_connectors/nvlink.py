"""Hidden states handed from the verifier's GPU to a trainer's GPU over NVLink peer
memory: no file system, no host staging.

The consumer (trainer rank) owns a ring of fixed-size slots in peer-visible device memory
(``HiddenStateRing``) and publishes its CUDA IPC handles (``describe`` -> a small dict; the
``nvlink`` backend writes it to a rendezvous file).  The producer maps the ring
(``HiddenStateRingWriter``) and pushes sample ``seq`` (1, 2, ...) into slot
``(seq - 1) % n_slots`` with a copy kernel that ends in a release-store of ``seq``; the
consumer pops with a kernel that waits for that value, copies the payload out and
acknowledges, which frees the slot for sample ``seq + n_slots``.  Both waits are bounded
(``timeout_s``): on expiry the status word is set and the host raises ``TimeoutError``;
nothing hangs.

Payload of a slot: ``hidden_states`` ``[rows, width]`` (bf16) followed by ``token_ids``
``[rows]`` (int32), both at fixed offsets for ``max_rows`` rows.

There is no counterpart of this transport in the reference (its transports are files and
a Mooncake store: hs_connectors/src/hs_connectors/transfer.py:136-334); it plugs into the
same ``HiddenStatesBackend`` / ``HiddenStatesTransfer`` interface.
"""

from __future__ import annotations

import argparse
import json
import os
import threading
import time
from pathlib import Path
from typing import Any

import torch

from speculators_b200.hs_connectors.transfer import HiddenStatesBackend, HiddenStatesTransfer

__all__ = ["HiddenStateRing", "HiddenStateRingWriter", "NvlinkBackend", "NvlinkTransfer"]

_SPIN_NS = 256  # one poll of the wait kernel sleeps this long


def _native():
    from speculators_b200 import ops

    return ops.native()


def _spin_limit(timeout_s: float) -> int:
    return max(1, min(int(timeout_s * 1e9 / _SPIN_NS), 2**31 - 1))


def _layout(max_rows: int, width: int) -> tuple[int, int, int]:
    """(offset of token ids, used bytes, slot bytes) for bf16 hidden states + int32 ids."""
    hs_bytes = max_rows * width * 2
    ids_off = (hs_bytes + 255) // 256 * 256
    used = ids_off + max_rows * 4
    return ids_off, (used + 15) // 16 * 16, (used + 255) // 256 * 256


class _RingBase:
    def __init__(self, n_slots: int, max_rows: int, width: int, device: torch.device):
        self.n_slots, self.max_rows, self.width, self.device = int(n_slots), int(max_rows), int(width), torch.device(device)
        self.ids_off, self.used_bytes, self.slot_bytes = _layout(self.max_rows, self.width)
        self.ctl_words = int(_native().hs_ring_ctl_words())
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.scratch = torch.zeros(4, dtype=torch.int32, device=self.device)  # go flag, block ticket, popped rows, popped width
        self._data = self._ctl = 0

    def _slot(self, seq: int) -> tuple[int, int]:
        i = (seq - 1) % self.n_slots
        return self._data + i * self.slot_bytes, self._ctl + i * self.ctl_words * 4

    def _check(self, what: str) -> None:
        code = int(self.status.item())
        if code:
            self.status.zero_()
            reason = {21: "the slot was not freed by the consumer", 22: "the sample never arrived"}.get(code, f"code {code}")
            raise TimeoutError(f"hidden-state ring {what}: {reason}")


class HiddenStateRing(_RingBase):
    """Consumer side: owns the slots."""

    def __init__(self, n_slots: int, max_rows: int, width: int, device: torch.device | str = "cuda"):
        super().__init__(n_slots, max_rows, width, torch.device(device))
        nat = _native()
        with torch.cuda.device(self.device):
            self._data = int(nat.peer_alloc(self.n_slots * self.slot_bytes))
            self._ctl = int(nat.peer_alloc(self.n_slots * self.ctl_words * 4))
        self._staging = torch.empty(self.used_bytes, dtype=torch.uint8, device=self.device)

    def describe(self) -> dict[str, Any]:
        """What a producer needs to map the ring (JSON-serialisable)."""
        nat = _native()
        return {
            "data": nat.peer_handle(self._data).tolist(), "ctl": nat.peer_handle(self._ctl).tolist(), "n_slots": self.n_slots,
            "max_rows": self.max_rows, "width": self.width, "pid": os.getpid(),
        }

    def pop(self, seq: int, timeout_s: float = 1.0) -> dict[str, torch.Tensor]:
        """Sample ``seq`` as ``{"hidden_states": [rows, width] bf16, "token_ids": [rows] int64}``
        (fresh tensors).  ``TimeoutError`` if it does not arrive within ``timeout_s``."""
        data, ctl = self._slot(seq)
        _native().hs_pop(self._staging, data, ctl, seq, _spin_limit(timeout_s), self.scratch, self.status)
        rows = int(self.scratch[2].item())  # taken out by the pop kernel before it freed the slot; synchronises with the copy
        self._check(f"pop of sample {seq}")
        hs = self._staging[: self.max_rows * self.width * 2].view(torch.bfloat16).view(self.max_rows, self.width)[:rows].clone()
        ids = self._staging[self.ids_off : self.ids_off + self.max_rows * 4].view(torch.int32)[:rows].long()
        return {"hidden_states": hs, "token_ids": ids}

    def close(self) -> None:
        if self._data:
            torch.cuda.synchronize(self.device)
            nat = _native()
            nat.peer_release(self._data)
            nat.peer_release(self._ctl)
            self._data = self._ctl = 0


class HiddenStateRingWriter(_RingBase):
    """Producer side: maps a consumer's ring and pushes samples into it."""

    def __init__(self, description: dict[str, Any], device: torch.device | str = "cuda"):
        super().__init__(description["n_slots"], description["max_rows"], description["width"], torch.device(device))
        nat = _native()
        self._same_process = description.get("pid") == os.getpid()
        with torch.cuda.device(self.device):
            if self._same_process:  # IPC handles cannot be opened by the exporting process: use the addresses directly
                self._data, self._ctl = int(description["_data_ptr"]), int(description["_ctl_ptr"])
            else:
                self._data = int(nat.peer_open(torch.tensor(description["data"], dtype=torch.uint8)))
                self._ctl = int(nat.peer_open(torch.tensor(description["ctl"], dtype=torch.uint8)))
        self._staging = torch.zeros(self.used_bytes, dtype=torch.uint8, device=self.device)

    def push(self, seq: int, hidden_states: torch.Tensor, token_ids: torch.Tensor | None = None, timeout_s: float = 1.0,
             check: bool = True) -> None:
        """Send sample ``seq`` (>= 1, consecutive).  ``check=False`` skips the host read of the
        status word (call ``check_status`` later) so pushes can be queued back to back."""
        rows = hidden_states.shape[0]
        if rows > self.max_rows or hidden_states.reshape(rows, -1).shape[1] != self.width:
            raise ValueError(f"sample of shape {tuple(hidden_states.shape)} does not fit slots of [{self.max_rows}, {self.width}]")
        hs_view = self._staging[: self.max_rows * self.width * 2].view(torch.bfloat16).view(self.max_rows, self.width)
        hs_view[:rows].copy_(hidden_states.reshape(rows, -1))
        if token_ids is not None:
            self._staging[self.ids_off : self.ids_off + self.max_rows * 4].view(torch.int32)[:rows].copy_(token_ids.reshape(-1))
        data, ctl = self._slot(seq)
        _native().hs_push(self._staging, data, ctl, seq, self.n_slots, rows, self.width, _spin_limit(timeout_s), self.scratch, self.status)
        if check:
            self.check_status(seq)

    def check_status(self, seq: int | None = None) -> None:
        self._check("push" if seq is None else f"push of sample {seq}")

    def close(self) -> None:
        if self._data and not self._same_process:
            torch.cuda.synchronize(self.device)
            nat = _native()
            nat.peer_close(self._data)
            nat.peer_close(self._ctl)
        self._data = self._ctl = 0


def describe_for_same_process(ring: HiddenStateRing) -> dict[str, Any]:
    """Description that also works inside the exporting process (tests, single-process
    pipelines with verifier and trainer on different GPUs): carries the raw addresses."""
    d = ring.describe()
    d["_data_ptr"], d["_ctl_ptr"] = ring._data, ring._ctl  # noqa: SLF001
    return d


class NvlinkTransfer(HiddenStatesTransfer):
    """Trainer-side transport: ``get_generated(handle)`` pops sample ``handle`` (its
    sequence number as a string) from this rank's ring.  The ring is created lazily in the
    process that consumes it and announced through ``rendezvous_path/ring_<rank>.json``."""

    def __init__(self, rendezvous_path: str | Path, n_slots: int = 8, max_rows: int = 8192, width: int = 0, rank: int = 0,
                 device: str | None = None, timeout_s: float = 30.0):
        self.rendezvous_path, self.n_slots, self.max_rows, self.width = Path(rendezvous_path), n_slots, max_rows, width
        self.rank, self.device, self.timeout_s = rank, device, timeout_s
        self.ring: HiddenStateRing | None = None

    def setup(self) -> None:
        if self.ring is not None:
            return
        if self.width <= 0:
            raise ValueError("NvlinkTransfer needs the payload width (num_target_layers * hidden_size)")
        self.ring = HiddenStateRing(self.n_slots, self.max_rows, self.width, self.device or f"cuda:{torch.cuda.current_device()}")
        self.rendezvous_path.mkdir(parents=True, exist_ok=True)
        tmp = self.rendezvous_path / f".ring_{self.rank}.json.tmp"
        tmp.write_text(json.dumps(self.ring.describe()))
        os.replace(tmp, self.rendezvous_path / f"ring_{self.rank}.json")

    def get_cached(self, file_idx: int) -> dict[str, torch.Tensor] | None:  # nothing persists in a ring
        return None

    def get_generated(self, handle: str) -> dict[str, torch.Tensor] | None:
        self.setup()
        return self.ring.pop(int(handle), self.timeout_s)

    def request_params(self) -> dict:
        """Tells the server-side connector which trainer rank's ring the sample goes to; the
        connector answers with the sample's sequence number in that ring as the handle."""
        self.setup()  # the ring must be announced before the server looks for it
        return {"ring_rank": self.rank}

    @staticmethod
    def wait_for_ring(rendezvous_path: str | Path, rank: int = 0, timeout_s: float = 60.0) -> dict[str, Any]:
        """Producer side: block until trainer ``rank`` has announced its ring."""
        path = Path(rendezvous_path) / f"ring_{rank}.json"
        deadline = time.monotonic() + timeout_s
        while not path.exists():
            if time.monotonic() > deadline:
                raise TimeoutError(f"no ring announced at {path} after {timeout_s}s")
            time.sleep(0.05)
        return json.loads(path.read_text())


def ring_key(rank: int, seq: int) -> str:
    return f"ring{rank}-{seq}"


def parse_ring_key(key: str) -> tuple[int, int]:
    rank, _, seq = key.removeprefix("ring").partition("-")
    if not key.startswith("ring") or not rank.isdigit() or not seq.isdigit():
        raise ValueError(f"not a ring key: {key!r}")
    return int(rank), int(seq)


class NvlinkRingSink:
    """Store-shaped end of the server-side connector (``put_sample`` / ``put_error``): samples
    keyed ``ring<rank>-<seq>`` are pushed into trainer ``rank``'s ring straight from device
    memory.  A ring takes its samples in sequence order, requests finish in any order, so a
    sample that arrives early is held until its predecessors have been pushed."""

    accepts_device_tensors = True
    is_setup = True

    def __init__(self, rendezvous_path: str | Path, device: torch.device | str | None = None, timeout_s: float = 60.0, writer_factory=None):
        self.rendezvous_path, self.device, self.timeout_s = Path(rendezvous_path), device, timeout_s
        self._writer_factory = writer_factory or self._open_writer
        self._writers: dict[int, Any] = {}
        self._next: dict[int, int] = {}
        self._held: dict[int, dict[int, tuple[torch.Tensor, torch.Tensor | None]]] = {}
        self._lock = threading.Lock()

    def setup(self) -> None:
        """Rings are opened per trainer rank when its first sample arrives."""

    def _open_writer(self, rank: int):
        description = NvlinkTransfer.wait_for_ring(self.rendezvous_path, rank, self.timeout_s)
        return HiddenStateRingWriter(description, self.device or f"cuda:{torch.cuda.current_device()}")

    def _offer(self, rank: int, seq: int, hidden_states: torch.Tensor, token_ids: torch.Tensor | None) -> None:
        with self._lock:
            self._held.setdefault(rank, {})[seq] = (hidden_states, token_ids)
            writer = self._writers.get(rank)
            if writer is None:
                writer = self._writers[rank] = self._writer_factory(rank)
            nxt = self._next.get(rank, 1)
            while nxt in self._held[rank]:
                hs, ids = self._held[rank].pop(nxt)
                writer.push(nxt, hs, ids, timeout_s=self.timeout_s)
                nxt += 1
            self._next[rank] = nxt

    def put_sample(self, key: str, sample: dict[str, torch.Tensor]) -> None:
        rank, seq = parse_ring_key(key)
        self._offer(rank, seq, sample["hidden_states"], sample.get("token_ids"))

    def put_error(self, key: str, message: str) -> None:
        """A failed request still takes its place in the sequence: an empty sample (zero rows)
        reaches the consumer, whose length check rejects it."""
        rank, seq = parse_ring_key(key)
        writer = self._writers.get(rank) or self._writer_factory(rank)
        self._writers[rank] = writer
        empty = torch.zeros(0, writer.width, dtype=torch.bfloat16, device=getattr(writer, "device", "cpu"))
        self._offer(rank, seq, empty, None)

    def close(self) -> None:
        for writer in self._writers.values():
            writer.close()
        self._writers = {}


@HiddenStatesBackend.register("nvlink")
class NvlinkBackend(HiddenStatesBackend):
    @staticmethod
    def add_train_args(parser: argparse.ArgumentParser) -> None:
        parser.add_argument("--nvlink-rendezvous-path", type=str, default=None,
                            help="Directory where trainer ranks announce their hidden-state rings (default: <data_path>/nvlink).")
        parser.add_argument("--nvlink-slots", type=int, default=8, help="Ring depth per trainer rank.")

    @staticmethod
    def add_launch_args(parser: argparse.ArgumentParser) -> None:
        parser.add_argument("--nvlink-rendezvous-path", type=str, default="/tmp/hidden_states_nvlink",  # noqa: S108
                            help="Directory where trainer ranks announce their hidden-state rings.")

    @staticmethod
    def from_train_args(args: argparse.Namespace, data_path: str) -> NvlinkTransfer:
        where = getattr(args, "nvlink_rendezvous_path", None) or str(Path(data_path) / "nvlink")
        return NvlinkTransfer(where, n_slots=getattr(args, "nvlink_slots", 8), max_rows=getattr(args, "total_seq_len", 8192),
                              rank=int(os.environ.get("RANK", "0")))

    @staticmethod
    def build_kv_transfer_config(args: argparse.Namespace) -> dict[str, Any]:
        return {
            "kv_connector": "NvlinkHiddenStatesConnector", "kv_role": "kv_producer",
            "kv_connector_module_path": "speculators_b200.hs_connectors.vllm_connector",
            "kv_connector_extra_config": {"rendezvous_path": args.nvlink_rendezvous_path},
        }
