"""Expert-parallel exchange kernels on one GPU: several virtual ranks of one process, driven
one phase at a time (push / signal of every rank first, then the waits, then the pulls), so
no kernel ever waits for a launch that has not been issued."""

import pytest
import torch

from speculators_b200.parallel.ep_comm import EpComm, build_plan

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _world(R, H, cap):
    comms = [EpComm(None, H, cap, DEV, rank=r, world=R, spin_limit=1 << 16) for r in range(R)]
    EpComm.connect_local(comms)
    return comms


def test_dispatch_and_weighted_combine_match_dense_indexing():
    R, E, k, H = 4, 8, 2, 64
    nl = E // R
    tokens = [33, 0, 57, 8]
    torch.manual_seed(0)
    tops = [torch.stack([torch.randperm(E)[:k] for _ in range(t)]).to(DEV) if t else torch.zeros(0, k, dtype=torch.long, device=DEV)
            for t in tokens]
    xs = [torch.randn(t, H, device=DEV).to(torch.bfloat16) for t in tokens]
    ws = [torch.rand(t * k, device=DEV) for t in tokens]
    counts_all = torch.stack([torch.bincount(t.reshape(-1), minlength=E) for t in tops])
    plans = [build_plan(tops[r], counts_all, r, nl) for r in range(R)]
    comms = _world(R, H, sum(tokens) * k)
    try:
        # dispatch: all pushes, then all waits
        seqs = [comms[r].push("x", 0, xs[r], plans[r]) for r in range(R)]
        for r in range(R):
            comms[r].wait(seqs[r])
        torch.cuda.synchronize()
        for d in range(R):
            comms[d].check_status()
            recv = comms[d].buf[("x", 0)][: plans[d].n_recv].float()
            # reference: rows in (local expert, source rank, appearance) order
            ref = []
            for el in range(nl):
                for r in range(R):
                    flat_e = tops[r].reshape(-1)
                    slots = torch.nonzero(flat_e == d * nl + el).squeeze(-1)
                    ref.append(xs[r][slots // k].float())
            ref = torch.cat(ref) if ref else torch.zeros(0, H, device=DEV)
            assert torch.equal(recv, ref)
        # "experts": y = 2 * x + expert index, then combine with the routing weights
        for d in range(R):
            el_of_row = torch.repeat_interleave(torch.arange(nl, device=DEV), plans[d].local_counts)
            y = (2 * comms[d].buf[("x", 0)][: plans[d].n_recv].float() + el_of_row.unsqueeze(-1)).to(torch.bfloat16)
            comms[d].buf[("y", 0)][: plans[d].n_recv].copy_(y)
        seqs = [comms[r].signal() for r in range(R)]
        for r in range(R):
            comms[r].wait(seqs[r])
        for r in range(R):
            out, rows = comms[r].pull("y", 0, plans[r], ws[r], tokens[r], keep_rows=True)
            el = (tops[r] % nl).reshape(-1).float().unsqueeze(-1)
            y_ref = (2 * xs[r].float().repeat_interleave(k, 0) + el).to(torch.bfloat16).float()
            assert torch.equal(rows.float(), y_ref)
            ref = (y_ref * ws[r].unsqueeze(-1)).view(tokens[r], k, H).sum(1)
            torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
            comms[r].check_status()
    finally:
        for c in comms:
            c.close()


def test_wait_for_a_rank_that_never_publishes_reports_status():
    comms = _world(2, 64, 8)
    try:
        comms[0].wait(5)  # nothing has published sequence 5: the bounded poll runs out
        torch.cuda.synchronize()
        with pytest.raises(RuntimeError, match="did not arrive"):
            comms[0].check_status()
        # the context is still usable
        assert float(torch.ones(4, device=DEV).sum()) == 4.0
    finally:
        for c in comms:
            c.close()
