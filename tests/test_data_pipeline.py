import os
import sys
import warnings

import numpy as np
import pytest
import torch
from safetensors.torch import save_file

from speculators_b200.data_generation.offline import check_hidden_states, get_existing_hidden_state_indices, get_indices_to_process
from speculators_b200.data_generation.vllm_client import InvalidResponseError, extract_output, with_retries
from speculators_b200.hs_connectors import (
    DictStoreClient, FileBackend, FileTransfer, HiddenStatesBackend, HiddenStatesStore, MooncakeIntegrityError, wait_for_lock,
)
from speculators_b200.models.eagle3.data import shift_batch
from speculators_b200.train.data import ArrowDataset, CollateFn, create_empty_sample
from speculators_b200.train.distributed_batch_sampler import MultipackDistributedBatchSamplerV2, lpt_bins
from speculators_b200.train.noise_transforms import AddGaussianNoise, AddUniformNoise
from speculators_b200.train.vocab_mapping import build_vocab_mappings_from_distribution, token_frequency_from_ids

from conftest import ROOT


# ---- sampler -------------------------------------------------------------------------------
def test_sampler_balance_partition_and_budget():
    rng = np.random.default_rng(0)
    lengths = rng.integers(16, 2000, size=400)
    R = 4
    per_rank = []
    for rank in range(R):
        s = MultipackDistributedBatchSamplerV2(4096, lengths, R, rank, seed=1)
        per_rank.append([list(map(int, b)) for b in s])
    counts = {len(b) for b in per_rank}
    assert len(counts) == 1  # every rank gets the same number of batches
    seen = [i for batches in per_rank for b in batches for i in b]
    assert len(seen) == len(set(seen))  # no sample on two ranks / in two batches
    for batches in per_rank:
        assert all(lengths[b].sum() <= 4096 for b in batches)
    s = MultipackDistributedBatchSamplerV2(4096, lengths, R, 0, seed=1)
    first = [list(map(int, b)) for b in s]
    s.set_epoch(1)
    assert [list(map(int, b)) for b in s] != first  # reshuffled per epoch
    assert s._generate_batches(1) is s._cached_generated_batches[1]


def test_sampler_truncates_or_drops_long_samples():
    lengths = [10, 5000, 20, 30]
    with warnings.catch_warnings(record=True) as w:
        warnings.simplefilter("always")
        s = MultipackDistributedBatchSamplerV2(100, lengths, 1, 0)
        assert s.lengths.max() == 100 and len(s.valid_indices) == 4 and "truncated" in str(w[0].message)
        s2 = MultipackDistributedBatchSamplerV2(100, lengths, 1, 0, truncate_long_samples=False)
        assert 1 not in s2.valid_indices
    assert lpt_bins(np.array([60, 60]), 100, 1) is None
    assert lpt_bins(np.array([60, 50, 40]), 100, 2) == [[0], [1, 2]]


@pytest.mark.skipif(not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "speculators")), reason="reference not installed")
def test_sampler_assignment_identical_to_reference():
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    try:
        from speculators.train.distributed_batch_sampler import MultipackDistributedBatchSamplerV2 as Ref
    finally:
        sys.path.pop(0)
    lengths = np.random.default_rng(5).integers(10, 3000, size=300)
    for R in (1, 3):
        for rank in range(R):
            a, b = Ref(4096, lengths, R, rank, seed=2), MultipackDistributedBatchSamplerV2(4096, lengths, R, rank, seed=2)
            assert [list(map(int, x)) for x in a] == [list(map(int, x)) for x in b]


# ---- collate ---------------------------------------------------------------------------------
def _sample(n, H=4, layers=3):
    return {"hidden_states": torch.randn(n, layers * H), "input_ids": torch.arange(n), "verifier_last_hidden_states": torch.randn(n, H),
            "loss_mask": torch.ones(n, dtype=torch.bool), "lengths": torch.tensor([n]), "position_ids": torch.arange(n)}


def test_collate_packs_pads_and_builds_document_ids():
    col = CollateFn(max_len=16, hidden_size=4, num_target_layers=3, dtype=torch.bfloat16, preprocess=shift_batch)
    out = col([_sample(6), None, _sample(5)])
    assert out["hidden_states"].shape == (1, 16, 12) and out["hidden_states"].dtype == torch.bfloat16
    assert out["document_ids"][0].tolist() == [0] * 5 + [1] * 4 + [-1] * 7
    assert out["position_ids"][0, :5].tolist() == [1, 2, 3, 4, 5] and out["input_ids"][0, 5:9].tolist() == [1, 2, 3, 4]
    assert "lengths" not in out


def test_collate_truncates_at_max_len_and_handles_empty_batches():
    col = CollateFn(max_len=8, hidden_size=4)
    out = col([_sample(6), _sample(6)])
    assert out["document_ids"][0].tolist() == [0] * 6 + [1] * 2
    empty = CollateFn(max_len=8, hidden_size=4, preprocess=shift_batch)([None, None])
    assert (empty["document_ids"] == -1).all() and empty["hidden_states"].shape == (1, 8, 12)
    assert create_empty_sample(4)["lengths"].item() == 0


def test_noise_transforms():
    x = {"hidden_states": torch.zeros(1000, 4), "other": torch.zeros(3)}
    y = AddUniformNoise(std=0.1)(dict(x))
    assert y["hidden_states"].abs().max() <= 0.1 and y["hidden_states"].abs().mean() > 0.02 and (y["other"] == 0).all()
    z = AddGaussianNoise(std=0.1)(dict(x))
    assert 0.05 < z["hidden_states"].std() < 0.15


# ---- dataset over the file backend ---------------------------------------------------------------
def test_arrow_dataset_cached_hidden_states(tmp_path):
    from datasets import Dataset

    rows = [{"input_ids": list(range(i, i + 5 + i)), "loss_mask": [1] * (5 + i), "seq_len": 5 + i} for i in range(6)]
    Dataset.from_list(rows).save_to_disk(str(tmp_path / "ds"))
    hs_dir = tmp_path / "ds" / "hidden_states"
    hs_dir.mkdir()
    for i, r in enumerate(rows):
        if i == 3:
            continue  # missing sample
        save_file({"hidden_states": torch.randn(r["seq_len"], 4, 8).to(torch.bfloat16), "token_ids": torch.tensor(r["input_ids"])}, str(hs_dir / f"hs_{i}.safetensors"))
    train = ArrowDataset(32, tmp_path / "ds", on_missing="skip", train_ratio=0.67, split="train")
    val = ArrowDataset(32, tmp_path / "ds", on_missing="skip", train_ratio=0.67, split="val")
    assert len(train) == 4 and len(val) == 2 and val.start_file_idx == 4 and train.approx_lengths == [5, 6, 7, 8]
    item = train[1]
    assert item["hidden_states"].shape == (6, 24) and item["verifier_last_hidden_states"].shape == (6, 8) and item["lengths"].item() == 6
    assert train[3] is None
    with pytest.raises(RuntimeError):
        ArrowDataset(32, tmp_path / "ds", on_missing="raise")[3]
    assert val[0]["input_ids"].tolist() == rows[4]["input_ids"]
    with pytest.raises(ValueError):
        ArrowDataset(32, tmp_path / "ds", train_ratio=1.0, split="val")


# ---- transports -------------------------------------------------------------------------------------
def test_file_transfer_and_lock(tmp_path):
    t = FileTransfer(tmp_path / "hs")
    assert t.get_cached(0) is None
    gen = tmp_path / "gen.safetensors"
    save_file({"hidden_states": torch.zeros(2, 2, 2), "token_ids": torch.arange(2)}, str(gen))
    assert t.get_generated(str(gen))["token_ids"].tolist() == [0, 1]
    t.cache(str(gen), 7)
    assert not gen.exists() and t.get_cached(7) is not None
    lock = tmp_path / "x.lock"
    lock.write_text("")
    wait_for_lock(str(lock))
    assert not lock.exists()
    assert set(HiddenStatesBackend.registry) >= {"file", "mooncake"}
    with pytest.raises(ValueError):
        HiddenStatesBackend.register("file")(FileBackend)


class _FailingClient(DictStoreClient):
    def __init__(self, fail_on):
        super().__init__()
        self.fail_on = fail_on

    def put_tensor(self, key, tensor):
        if key.endswith(self.fail_on):
            return -5
        return super().put_tensor(key, tensor)


def test_store_manifest_last_integrity_and_cleanup():
    client = DictStoreClient()
    store = HiddenStatesStore(client=client)
    sample = {"hidden_states": torch.randn(3, 4).to(torch.bfloat16), "token_ids": torch.arange(3)}
    store.put_sample("k", sample)
    got = store.get_sample("k")
    assert torch.equal(got["hidden_states"], sample["hidden_states"])
    client._data["k:hidden_states"][0, 0] += 1  # corrupt payload
    with pytest.raises(MooncakeIntegrityError, match="checksum"):
        store.get_sample("k")
    store.delete_sample("k")
    assert not client._data
    with pytest.raises(TimeoutError):
        store.get_sample("missing", timeout=0.05, poll_interval=0.01)
    store.put_error("bad", "producer failed")
    with pytest.raises(MooncakeIntegrityError, match="producer failed"):
        store.get_sample("bad")
    failing = _FailingClient(":token_ids")
    with pytest.raises(RuntimeError, match="status=-5"):
        HiddenStatesStore(client=failing).put_sample("p", sample)
    assert not failing._data  # partial write removed
    with pytest.raises(RuntimeError, match="setup"):
        HiddenStatesStore().put_sample("x", sample)


# ---- client / offline helpers ----------------------------------------------------------------------------
def test_retries_and_response_validation(monkeypatch):
    monkeypatch.setattr("time.sleep", lambda s: None)
    calls = {"n": 0}

    @with_retries
    def flaky():
        calls["n"] += 1
        if calls["n"] < 3:
            raise TimeoutError("slow")
        return "ok"

    assert flaky(max_retries=3) == "ok" and calls["n"] == 3

    @with_retries
    def invalid():
        calls["n"] += 1
        raise InvalidResponseError("bad")

    calls["n"] = 0
    with pytest.raises(InvalidResponseError):
        invalid(max_retries=5)
    assert calls["n"] == 1  # deterministic errors are not retried

    class R:
        prompt_token_ids = [1, 2]
        kv_transfer_params = {"handle": "h"}
        choices = None

    assert extract_output(R(), [1, 2]) == "h"
    with pytest.raises(InvalidResponseError):
        extract_output(R(), [1, 3])


def test_check_hidden_states_and_index_split(tmp_path):
    good = {"token_ids": torch.arange(4), "hidden_states": torch.zeros(4, 3, 2)}
    check_hidden_states(good, [0, 1, 2, 3])
    bad = {"token_ids": torch.arange(4), "hidden_states": torch.zeros(4, 3, 2)}
    bad["hidden_states"][2, 1, 0] = float("nan")
    with pytest.raises(ValueError, match=r"affected layer slots=\[1\]"):
        check_hidden_states(bad, [0, 1, 2, 3])
    with pytest.raises(ValueError):
        check_hidden_states(good, [0, 1, 2])
    (tmp_path / "hs_3.safetensors").write_text("")
    (tmp_path / "hs_x.safetensors").write_text("")
    assert get_existing_hidden_state_indices(tmp_path) == [3]
    assert get_indices_to_process(10, None, [], 3, 0) == [0, 1, 2, 3]
    assert get_indices_to_process(10, None, [4, 5], 3, 1) == [6]
    assert get_indices_to_process(10, 5, [], 2, 1) == [3, 4]


def test_vocab_mapping_offsets_and_ties():
    freq = token_frequency_from_ids(torch.tensor([5, 5, 5, 2, 2, 9, 7]), torch.tensor([1, 1, 1, 1, 1, 1, 0]))
    assert freq == {2: 2, 5: 3, 9: 1}
    d2t, t2d = build_vocab_mappings_from_distribution(freq, 4, 12)
    kept = torch.nonzero(t2d).squeeze(1)
    assert kept.tolist() == [0, 2, 5, 9]  # top-3 by count, then the lowest unseen id
    assert (torch.arange(4) + d2t).tolist() == kept.tolist()  # d2t stores offsets


def test_vllm_connector_halves_with_dict_store():
    """Scheduler/worker halves of the server-side plugin against an in-memory store:
    paged-cache gather, key naming, delayed completion, error marker on non-finite data."""
    import time as _time

    from speculators_b200.hs_connectors import DictStoreClient, HiddenStatesStore
    from speculators_b200.hs_connectors.vllm_connector import (
        SchedulerSide, WorkerSide, extract_from_kv_cache, sanitize_key, slot_mapping_for_blocks,
    )

    assert sanitize_key("cmpl-12/ab") == "cmpl-12_ab" and sanitize_key("9x") == "k9x"
    block_size, width = 4, 6
    cache = torch.arange(8 * block_size * width, dtype=torch.float32).reshape(8, block_size, width)
    slots = slot_mapping_for_blocks([5, 2], block_size)
    assert slots.tolist() == [20, 21, 22, 23, 8, 9, 10, 11]
    got = extract_from_kv_cache(cache, slots, 6)
    assert torch.equal(got, torch.cat([cache[5], cache[2][:2]]))

    store = HiddenStatesStore(client=DictStoreClient())
    sched, worker = SchedulerSide(), WorkerSide(store, block_size, num_writer_threads=2)
    worker.register(cache)
    sched.on_new_request("req/1")
    delay_free, params = sched.request_finished("req/1", [7, 8, 9, 10, 11, 12], [7, 8, 9, 10, 11, 12, 13], [5, 2])
    assert delay_free is True and params == {"handle": "req_1"}
    # with include_output_tokens the sampled last token is dropped
    _, p2 = sched.request_finished("r2", None, [1, 2, 3], [0], {"include_output_tokens": True})
    pending = sched.drain()
    assert [p.key for p in pending] == ["req_1", "r2"] and pending[1].token_ids.tolist() == [1, 2] and sched.drain() == []
    worker.submit(pending)
    done: set = set()
    for _ in range(200):
        done |= worker.poll({"req/1", "r2", "other-rank-only"})
        if {"req/1", "r2"} <= done:
            break
        _time.sleep(0.01)
    assert done == {"req/1", "r2", "other-rank-only"}
    sample = store.get_sample("req_1", timeout=1.0)
    assert torch.equal(sample["hidden_states"], got) and sample["token_ids"].tolist() == [7, 8, 9, 10, 11, 12]
    # non-finite hidden states: the write fails and leaves an error marker the consumer sees
    cache[1, 0, 0] = float("nan")
    _, _ = sched.request_finished("bad", [1, 2], [1, 2], [1])
    worker.submit(sched.drain())
    for _ in range(200):
        if worker.poll({"bad"}):
            break
        _time.sleep(0.01)
    with pytest.raises(Exception, match="(?i)non-finite|nan|error"):
        store.get_sample("bad", timeout=0.5)
    worker.shutdown()


def test_ring_mode_names_requests_by_rank_and_sequence_and_sink_pushes_in_order():
    """NVLink transport, server side: the scheduler half numbers finished requests per trainer
    rank and hands the number back as the handle; the sink holds samples that finish early
    until their predecessors are in the ring; a failed request still takes its place."""
    import time as _time

    from speculators_b200.hs_connectors.nvlink import NvlinkRingSink, parse_ring_key, ring_key
    from speculators_b200.hs_connectors.vllm_connector import SchedulerSide, WorkerSide

    assert parse_ring_key(ring_key(3, 17)) == (3, 17)
    with pytest.raises(ValueError):
        parse_ring_key("req_1")

    sched = SchedulerSide(ring_mode=True)
    handles = [sched.request_finished(f"r{i}", [1, 2, 3], [1, 2, 3], [i], {"ring_rank": rank})[1]["handle"]
               for i, rank in enumerate([0, 1, 0, 0, 1])]
    assert handles == ["1", "1", "2", "3", "2"]
    pending = sched.drain()
    assert [p.key for p in pending] == ["ring0-1", "ring1-1", "ring0-2", "ring0-3", "ring1-2"]

    pushed: dict[int, list] = {}

    class _Writer:
        width = 6

        def __init__(self, rank):
            self.rank = rank

        def push(self, seq, hs, ids, timeout_s=1.0):
            pushed.setdefault(self.rank, []).append((seq, hs.shape[0]))

        def close(self):
            pass

    sink = NvlinkRingSink("/nonexistent", writer_factory=_Writer)
    rows = lambda n: {"hidden_states": torch.zeros(n, 6), "token_ids": torch.arange(n)}  # noqa: E731
    sink.put_sample("ring0-3", rows(3))  # early: held
    sink.put_sample("ring0-2", rows(2))  # still waiting for 1
    assert pushed == {}
    sink.put_sample("ring0-1", rows(1))
    assert pushed[0] == [(1, 1), (2, 2), (3, 3)]
    sink.put_error("ring1-1", "boom")  # empty sample keeps ring 1's sequence going
    sink.put_sample("ring1-2", rows(5))
    assert pushed[1] == [(1, 0), (2, 5)]

    # through the worker half (CPU cache): device-capable sinks are only used on CUDA caches,
    # a CPU cache goes through the same put_sample with host rows
    cache = torch.arange(4 * 2 * 6, dtype=torch.float32).reshape(4, 2, 6)
    worker = WorkerSide(NvlinkRingSink("/nonexistent", writer_factory=_Writer), block_size=2, num_writer_threads=1)
    worker.register(cache)
    sched2 = SchedulerSide(ring_mode=True)
    sched2.request_finished("a", [5, 6, 7], [5, 6, 7], [2, 0], {"ring_rank": 2})
    worker.submit(sched2.drain())
    for _ in range(200):
        if worker.poll({"a"}):
            break
        _time.sleep(0.01)
    assert pushed[2] == [(1, 3)]


def test_generation_request_carries_the_transfer_parameters():
    from speculators_b200.data_generation.vllm_client import _request

    kind, kwargs = _request("m", {"input_ids": [1, 2]}, 5.0, {"ring_rank": 3})
    assert kind == "completions" and kwargs["extra_body"]["kv_transfer_params"] == {"ring_rank": 3}
    kind, kwargs = _request("m", {"input_ids": [1], "messages": [{"role": "user", "content": "hi"}]}, None)
    assert kind == "chat" and "kv_transfer_params" not in kwargs["extra_body"] and kwargs["extra_body"]["return_token_ids"] is True


def test_top_level_hs_connectors_import_paths():
    """The stand-alone package name of the transports resolves to the same objects (checked in a
    fresh interpreter: other tests import the reference's own ``hs_connectors`` for comparisons)."""
    import subprocess

    code = """
import hs_connectors
from hs_connectors import FileTransfer, HiddenStatesBackend
from hs_connectors.mooncake_store import MooncakeHiddenStatesStore
import hs_connectors.mooncake_hidden_states_connector as connector
import speculators_b200.hs_connectors as own
assert HiddenStatesBackend is own.HiddenStatesBackend and FileTransfer is own.FileTransfer
assert MooncakeHiddenStatesStore is own.store.MooncakeHiddenStatesStore
assert connector is own.mooncake_hidden_states_connector
assert {"file", "mooncake", "nvlink"} <= set(hs_connectors.HiddenStatesBackend.registry)
print("ok")
"""
    proc = subprocess.run([sys.executable, "-c", code], cwd=ROOT, capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and proc.stdout.strip().endswith("ok"), proc.stderr[-2000:]


def test_datasets_written_against_the_reference_hooks_still_work():
    """A ``BaseDataset`` subclass that defines the reference's hook names (``_compute_approx_lengths``,
    ``_get_raw_data``) runs unchanged."""
    from speculators_b200.train.data import BaseDataset

    class Theirs(BaseDataset):
        def __len__(self):
            return 2

        def _compute_approx_lengths(self):
            return [3, 4]

        def _get_raw_data(self, index):
            n = 3 + index
            return {"hidden_states": torch.zeros(n, 12), "input_ids": torch.arange(n), "verifier_last_hidden_states": torch.zeros(n, 4),
                    "loss_mask": torch.ones(n, dtype=torch.bool)}

    ds = Theirs(max_len=8)
    assert ds.approx_lengths == [3, 4] and ds[1]["lengths"].item() == 4 and ds[0]["position_ids"].tolist() == [0, 1, 2]
