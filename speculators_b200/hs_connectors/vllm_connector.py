"""vLLM-side plugin: publish extracted hidden states to a store instead of files.

Used with vLLM's ``extract_hidden_states`` speculative method: the auxiliary hidden states
of a request sit in a cache-only attention layer's paged KV cache; when the request
finishes they are gathered, checked, moved to pinned host memory on a side stream and
written to the store under the request's key, which the client receives as
``kv_transfer_params["handle"]``.

The logic lives in two vLLM-independent halves so it can run (and be tested) without a
server: ``SchedulerSide`` (request bookkeeping, hand-off of pending saves) and
``WorkerSide`` (gather + check + D2H + store write on a thread pool, completion polling).
``MooncakeHiddenStatesConnector`` adapts them to vLLM's ``KVConnectorBase_V1`` interface
and exists only where vLLM imports.

Reference surface: hs_connectors/src/hs_connectors/mooncake_hidden_states_connector.py
(extract_from_kv_cache:44, request_finished:337, get_finished:271, _write_sample:218).
"""

from __future__ import annotations

import logging
import re
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any

import torch

from speculators_b200.hs_connectors.store import HiddenStatesStore, MooncakeStoreConfig, assert_finite

log = logging.getLogger(__name__)

__all__ = ["PendingSave", "SchedulerSide", "WorkerSide", "extract_from_kv_cache", "sanitize_key", "slot_mapping_for_blocks"]


def sanitize_key(key: str) -> str:
    """Request id -> store key (``[A-Za-z0-9_-]``, not starting with a digit)."""
    safe = re.sub(r"[^a-zA-Z0-9_-]", "_", key)
    return "k" + safe if safe[:1].isdigit() else safe


def slot_mapping_for_blocks(block_ids: list[int], block_size: int) -> torch.Tensor:
    """Flat slot indices of the given blocks in order (``block * block_size + offset``)."""
    blocks = torch.as_tensor(block_ids, dtype=torch.long).reshape(-1, 1)
    return (blocks * block_size + torch.arange(block_size, dtype=torch.long).reshape(1, -1)).flatten()


def extract_from_kv_cache(kv_cache: torch.Tensor, slot_mapping: torch.Tensor, num_tokens: int) -> torch.Tensor:
    """Rows of a paged cache ``[num_blocks, block_size, ...]`` for the first ``num_tokens`` slots."""
    block_size = kv_cache.shape[1]
    return kv_cache[slot_mapping // block_size, slot_mapping % block_size][:num_tokens]


@dataclass
class PendingSave:
    req_id: str
    key: str
    token_ids: torch.Tensor
    block_ids: list[int]


class SchedulerSide:
    """Runs in the scheduler process: names requests, and when one finishes keeps its
    blocks alive (returns ``True``) until the worker has copied the hidden states out."""

    def __init__(self, ring_mode: bool = False) -> None:
        """``ring_mode``: samples go to per-trainer-rank rings (NVLink transport).  A finished
        request is then named by the ring of the rank that asked (``ring_rank`` in its
        ``kv_transfer_params``) and the next sequence number of that ring, which is also the
        handle the client gets back."""
        self._keys: dict[str, str] = {}
        self._pending: dict[str, PendingSave] = {}
        self._ring_mode = ring_mode
        self._ring_seq: dict[int, int] = {}

    def on_new_request(self, req_id: str) -> None:
        self._keys[req_id] = sanitize_key(req_id)

    def request_finished(self, req_id: str, prompt_token_ids: list[int] | None, all_token_ids: list[int], block_ids: list[int],
                         kv_params: dict | None = None) -> tuple[bool, dict[str, Any]]:
        key = self._keys.pop(req_id, sanitize_key(req_id))
        handle = key
        if self._ring_mode:
            from speculators_b200.hs_connectors.nvlink import ring_key

            rank = int((kv_params or {}).get("ring_rank", 0))
            seq = self._ring_seq.get(rank, 0) + 1
            self._ring_seq[rank] = seq
            key, handle = ring_key(rank, seq), str(seq)
        if (kv_params or {}).get("include_output_tokens", False):
            # the last token was sampled but never fed through the model: no hidden state for it
            ids = torch.tensor(list(all_token_ids)[:-1])
        elif prompt_token_ids is not None:
            ids = torch.tensor(prompt_token_ids)
        else:
            ids = torch.tensor([], dtype=torch.long)
        self._pending[req_id] = PendingSave(req_id, key, ids, list(block_ids))
        return True, {"handle": handle}

    def drain(self) -> list[PendingSave]:
        out = list(self._pending.values())
        self._pending.clear()
        return out


class WorkerSide:
    """Runs in the model worker (tensor-parallel rank 0 writes, the others only report)."""

    def __init__(self, store: HiddenStatesStore, block_size: int, num_writer_threads: int = 4, is_writer: bool = True):
        self.store, self.block_size, self.is_writer = store, block_size, is_writer
        self._threads = num_writer_threads
        self._pool: ThreadPoolExecutor | None = None
        self._futures: dict[str, Future] = {}
        self._waiting: set[str] = set()
        self._kv_cache: torch.Tensor | None = None
        self._copy_stream = None

    def register(self, kv_cache: torch.Tensor) -> None:
        self._kv_cache = kv_cache
        if kv_cache.is_cuda:
            self._copy_stream = torch.cuda.Stream(device=kv_cache.device)

    def _write(self, pending: PendingSave, ready) -> None:
        cache = self._kv_cache
        n = pending.token_ids.shape[0]
        try:
            slots = slot_mapping_for_blocks(pending.block_ids, self.block_size)
            if cache.is_cuda:
                stream = self._copy_stream
                stream.wait_event(ready)  # the forward pass that filled the cache has finished
                with torch.cuda.stream(stream):
                    hs = extract_from_kv_cache(cache, slots.to(cache.device, non_blocking=True), n)
                    assert_finite("hidden_states", hs)
                    if getattr(self.store, "accepts_device_tensors", False):
                        # device-to-device transports take the rows where they are
                        self.store.put_sample(pending.key, {"hidden_states": hs, "token_ids": pending.token_ids.to(cache.device)})
                        stream.synchronize()
                        return
                    host = torch.empty_like(hs, device="cpu", pin_memory=True)
                    host.copy_(hs, non_blocking=True)
                stream.synchronize()
            else:
                host = extract_from_kv_cache(cache, slots, n).clone()
                assert_finite("hidden_states", host)
            self.store.put_sample(pending.key, {"hidden_states": host, "token_ids": pending.token_ids})
        except Exception as err:
            try:  # leave an error marker so the consumer fails fast and can re-request
                self.store.put_error(pending.key, str(err))
            except Exception:  # noqa: BLE001
                log.exception("Failed to publish error marker for %s", pending.req_id)
            raise

    def submit(self, pending_saves: list[PendingSave]) -> None:
        if not self.is_writer:
            return
        for pending in pending_saves:
            if pending.req_id in self._futures:
                continue
            if not self.store.is_setup:
                self.store.setup()
            ready = None
            if self._kv_cache is not None and self._kv_cache.is_cuda:
                ready = torch.cuda.Event()
                ready.record()
            if self._pool is None:
                self._pool = ThreadPoolExecutor(max_workers=self._threads, thread_name_prefix="hs-writer")
            self._futures[pending.req_id] = self._pool.submit(self._write, pending, ready)

    def poll(self, finished_req_ids: set[str]) -> set[str]:
        """Requests whose sample is in the store (or that this rank does not write): their
        blocks may be freed and the client may be answered."""
        self._waiting.update(finished_req_ids)
        done = set()
        for req_id in list(self._waiting):
            fut = self._futures.get(req_id)
            if fut is None or fut.done():
                if fut is not None:
                    if fut.exception() is not None:
                        log.error("Hidden-state write failed for %s: %r", req_id, fut.exception())
                    del self._futures[req_id]
                done.add(req_id)
                self._waiting.discard(req_id)
        return done

    def shutdown(self) -> None:
        if self._pool is not None:
            self._pool.shutdown(wait=True)
            self._pool = None


try:  # the adapter needs vLLM's connector base classes
    from vllm.distributed.kv_transfer.kv_connector.v1.base import KVConnectorBase_V1, KVConnectorMetadata
except Exception:  # noqa: BLE001 - any import problem means "no vLLM here"
    KVConnectorBase_V1 = None  # type: ignore[assignment,misc]

if KVConnectorBase_V1 is not None:

    @dataclass
    class MooncakeConnectorMetadata(KVConnectorMetadata):  # type: ignore[misc,valid-type]
        pending_saves: list[PendingSave] = field(default_factory=list)

    class MooncakeHiddenStatesConnector(KVConnectorBase_V1):  # type: ignore[misc,valid-type]
        """Load with ``--kv_transfer_config '{"kv_connector": "MooncakeHiddenStatesConnector",
        "kv_connector_module_path": "speculators_b200.hs_connectors.vllm_connector", ...}'``."""

        @property
        def prefer_cross_layer_blocks(self) -> bool:
            return False  # the cache-only layer must keep its own blocks

        def __init__(self, vllm_config, role, kv_cache_config=None):
            super().__init__(vllm_config=vllm_config, role=role, kv_cache_config=kv_cache_config)
            spec = vllm_config.speculative_config
            if spec is None or spec.method != "extract_hidden_states":
                raise ValueError("MooncakeHiddenStatesConnector requires the 'extract_hidden_states' speculative method")
            self._group = self._hidden_state_group(kv_cache_config)
            block_size = (kv_cache_config.kv_cache_groups[self._group].kv_cache_spec.block_size
                          if kv_cache_config is not None else vllm_config.cache_config.block_size)
            self._scheduler, self._worker = self._build_sides(block_size)

        def _build_sides(self, block_size: int):
            cfg = MooncakeStoreConfig.from_dict(self._kv_transfer_config.get_from_extra_config("mooncake", {}))
            return SchedulerSide(), WorkerSide(HiddenStatesStore(cfg), block_size, getattr(cfg, "num_writer_threads", 4))

        @staticmethod
        def _hidden_state_group(kv_cache_config) -> int:
            if kv_cache_config is None:
                return 0
            from vllm.v1.kv_cache_interface import HiddenStateCacheSpec

            groups = kv_cache_config.kv_cache_groups
            ids = [i for i, g in enumerate(groups) if isinstance(g.kv_cache_spec, HiddenStateCacheSpec)]
            if len(ids) == 1:
                return ids[0]
            if not ids and len(groups) == 1:
                return 0
            raise ValueError(f"Could not uniquely identify the hidden-states KV cache group among {len(groups)} groups")

        # ---- worker side
        def start_load_kv(self, *args, **kwargs) -> None: ...
        def wait_for_layer_load(self, layer_name: str) -> None: ...
        def save_kv_layer(self, *args, **kwargs) -> None: ...
        def wait_for_save(self) -> None: ...

        def register_kv_caches(self, kv_caches: dict[str, torch.Tensor]) -> None:
            from vllm.config import get_layers_from_vllm_config
            from vllm.distributed.parallel_state import get_tensor_model_parallel_rank
            from vllm.model_executor.models.extract_hidden_states import CacheOnlyAttentionLayer

            names = list(get_layers_from_vllm_config(self._vllm_config, CacheOnlyAttentionLayer, list(kv_caches)))
            if len(names) != 1:
                raise ValueError(f"Expected 1 cache-only attention layer, got {len(names)}")
            self._worker.is_writer = get_tensor_model_parallel_rank() == 0
            self._worker.register(kv_caches[names[0]])

        def get_finished(self, finished_req_ids: set[str]):
            if self.has_connector_metadata():
                meta = self._get_connector_metadata()
                if isinstance(meta, MooncakeConnectorMetadata):
                    self._worker.submit(meta.pending_saves)
            return self._worker.poll(finished_req_ids) or None, None

        # ---- scheduler side
        def get_num_new_matched_tokens(self, request, num_computed_tokens):
            return 0, False  # this connector only stores

        def update_state_after_alloc(self, request, blocks, num_external_tokens) -> None:
            assert num_external_tokens == 0, "This connector is store-only"

        def build_connector_meta(self, scheduler_output):
            meta = MooncakeConnectorMetadata()
            meta.pending_saves = self._scheduler.drain()
            for req in scheduler_output.scheduled_new_reqs:
                self._scheduler.on_new_request(req.req_id)
            return meta

        def request_finished(self, request, block_ids):
            return self._scheduler.request_finished(request.request_id, request.prompt_token_ids, list(request.all_token_ids), block_ids,
                                                    request.kv_transfer_params)

        def request_finished_all_groups(self, request, block_ids):
            return self.request_finished(request, block_ids[self._group])

        @classmethod
        def get_required_kvcache_layout(cls, vllm_config):
            return "NHD"  # keeps one token's hidden states contiguous

    class NvlinkHiddenStatesConnector(MooncakeHiddenStatesConnector):
        """Same capture path, different sink: finished requests' hidden states are pushed from
        the verifier GPU into the asking trainer rank's NVLink ring
        (``hs_connectors/nvlink.py``).  Load with ``--kv_transfer_config '{"kv_connector":
        "NvlinkHiddenStatesConnector", "kv_connector_module_path":
        "speculators_b200.hs_connectors.vllm_connector", "kv_connector_extra_config":
        {"rendezvous_path": ...}}'``."""

        def _build_sides(self, block_size: int):
            from speculators_b200.hs_connectors.nvlink import NvlinkRingSink

            where = self._kv_transfer_config.get_from_extra_config("rendezvous_path", "/tmp/hidden_states_nvlink")  # noqa: S108
            # one writer thread: pushes into a ring are ordered anyway
            return SchedulerSide(ring_mode=True), WorkerSide(NvlinkRingSink(where), block_size, num_writer_threads=1)

    __all__ += ["MooncakeConnectorMetadata", "MooncakeHiddenStatesConnector", "NvlinkHiddenStatesConnector"]
