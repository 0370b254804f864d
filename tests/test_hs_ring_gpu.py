"""Hidden-state ring on one GPU: producer and consumer ends in one process, used strictly
one after the other (no kernel ever waits for a later launch), plus the bounded waits."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _pair(n_slots, max_rows=64, width=128):
    from speculators_b200.hs_connectors import HiddenStateRing, HiddenStateRingWriter
    from speculators_b200.hs_connectors.nvlink import describe_for_same_process

    ring = HiddenStateRing(n_slots, max_rows, width, "cuda:0")
    return ring, HiddenStateRingWriter(describe_for_same_process(ring), "cuda:0")


def test_push_pop_roundtrip_reuses_slots():
    ring, writer = _pair(n_slots=2)
    for seq in range(1, 7):
        rows = 10 + seq
        hs = torch.randn(rows, 128, device="cuda").to(torch.bfloat16)
        ids = torch.randint(0, 1000, (rows,), device="cuda", dtype=torch.int32)
        writer.push(seq, hs, ids)
        got = ring.pop(seq)
        assert got["hidden_states"].shape == (rows, 128) and torch.equal(got["hidden_states"], hs)
        assert got["token_ids"].dtype == torch.int64 and torch.equal(got["token_ids"], ids.long())
    with pytest.raises(ValueError):
        writer.push(7, torch.zeros(65, 128, device="cuda", dtype=torch.bfloat16))
    writer.close()
    ring.close()


def test_waits_run_out_and_leave_the_context_usable():
    ring, writer = _pair(n_slots=1)
    with pytest.raises(TimeoutError, match="never arrived"):
        ring.pop(1, timeout_s=0.05)  # nothing was pushed: the wait gives up and reports it
    hs = torch.ones(4, 128, device="cuda", dtype=torch.bfloat16)
    writer.push(1, hs)
    with pytest.raises(TimeoutError, match="not freed"):
        writer.push(2, hs, timeout_s=0.05)  # the only slot still holds sample 1
    assert torch.equal(ring.pop(1)["hidden_states"], hs)
    writer.push(2, hs * 2)  # freed now
    assert torch.equal(ring.pop(2)["hidden_states"], hs * 2)
    assert float((torch.ones(8, device="cuda") * 3).sum()) == 24.0  # the context still works
    writer.close()
    ring.close()
