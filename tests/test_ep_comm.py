"""Placement plan of the expert-parallel exchange (pure tensor arithmetic, CPU)."""

import torch

from speculators_b200.parallel.ep_comm import build_plan


def _plans(R, E, k, tokens, seed=0):
    g = torch.Generator().manual_seed(seed)
    tops = [torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(t)]) if t else torch.zeros(0, k, dtype=torch.long)
            for t in tokens]
    counts_all = torch.stack([torch.bincount(t.reshape(-1), minlength=E) for t in tops])
    nl = E // R
    return tops, counts_all, [build_plan(tops[r], counts_all, r, nl) for r in range(R)]


def test_every_slot_gets_its_own_row_in_expert_then_source_order():
    R, E, k = 4, 8, 2
    tokens = [5, 0, 9, 3]
    tops, counts_all, plans = _plans(R, E, k, tokens)
    nl = E // R
    for d in range(R):  # receive side of rank d
        n_recv = plans[d].n_recv
        assert n_recv == int(counts_all[:, d * nl : (d + 1) * nl].sum())
        assert plans[d].max_recv == max(p.n_recv for p in plans)
        owner = torch.full((n_recv, 3), -1)  # (local expert, source rank, order at the source)
        for r in range(R):
            p = plans[r]
            flat_e = tops[r].reshape(-1)
            seen = {}
            for s in range(flat_e.numel()):
                e = int(flat_e[s])
                nth = seen.get(e, 0)
                seen[e] = nth + 1
                if int(p.dst_rank[s]) != d:
                    continue
                pos = int(p.dst_pos[s])
                assert 0 <= pos < n_recv and owner[pos, 0] == -1  # in range, no collision
                owner[pos] = torch.tensor([e - d * nl, r, nth])
                assert int(p.src_row[s]) == s // k
        assert (owner[:, 0] >= 0).all()  # every row filled
        keys = [tuple(row.tolist()) for row in owner]
        assert keys == sorted(keys)  # grouped by local expert, then source rank, then appearance
        assert plans[d].local_counts.tolist() == [sum(1 for key in keys if key[0] == el) for el in range(nl)]


def test_single_rank_plan_is_a_stable_sort_by_expert():
    tops, counts_all, plans = _plans(1, 4, 2, [7], seed=3)
    flat_e = tops[0].reshape(-1)
    order = torch.argsort(flat_e, stable=True)
    assert torch.equal(plans[0].dst_pos[order].long(), torch.arange(flat_e.numel()))
    assert plans[0].dst_rank.eq(0).all() and plans[0].n_recv == flat_e.numel()
