"""Muon in the training engine: against ``torch.optim.Muon`` + ``torch.optim.AdamW`` on one
process, and two gloo ranks (replicated and sharded, matrices owned by ranks) against one."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from speculators_b200.parallel.engine import EngineConfig, TrainEngine, split_named_params_for_muon


def _model(seed=0):
    torch.manual_seed(seed)
    return nn.Sequential(nn.Linear(24, 40, bias=False), nn.LayerNorm(40), nn.Linear(40, 16, bias=True), nn.Linear(16, 56, bias=False))


def _data(step, rank=0):
    g = torch.Generator().manual_seed(100 * step + rank)
    return torch.randn(12, 24, generator=g), torch.randn(12, 56, generator=g)


CFG = dict(lr=1e-2, weight_decay=0.01, max_grad_norm=0.0, optimizer="muon", muon_lr=0.02, muon_momentum=0.95, muon_weight_decay=0.1,
           muon_ns_steps=5, compute_dtype=torch.float32)


def test_engine_muon_matches_torch_optim():
    ours, ref = _model(), _model()
    eng = TrainEngine(ours, EngineConfig(**CFG), device="cpu")
    muon_named, adamw_named = split_named_params_for_muon(ref)
    opt_m = torch.optim.Muon([p for _, p in muon_named], lr=0.02, weight_decay=0.1, momentum=0.95, nesterov=True, ns_steps=5,
                             adjust_lr_fn="match_rms_adamw")
    opt_a = torch.optim.AdamW([p for _, p in adamw_named], lr=1e-2, weight_decay=0.01)
    for step in range(4):
        x, y = _data(step)
        eng.zero_grad()
        ((ours(x) - y) ** 2).mean().backward()
        eng.step()
        opt_m.zero_grad(); opt_a.zero_grad()
        ((ref(x) - y) ** 2).mean().backward()
        opt_m.step(); opt_a.step()
    for (name, a), (_, b) in zip(ours.named_parameters(), ref.named_parameters()):
        # torch.optim.Muon iterates in bf16 on any device; the engine iterates in fp32 on CPU
        assert torch.allclose(a, b, rtol=2e-2, atol=2e-3), (name, (a - b).abs().max())


def test_muon_state_dict_round_trip():
    m1 = _model()
    e1 = TrainEngine(m1, EngineConfig(**CFG), device="cpu")
    for step in range(2):
        x, y = _data(step)
        e1.zero_grad()
        ((m1(x) - y) ** 2).mean().backward()
        e1.step()
    sd, weights = e1.optimizer_state_dict(), e1.master_state_dict()
    m2 = _model(seed=5)
    e2 = TrainEngine(m2, EngineConfig(**CFG), device="cpu")
    e2.load_optimizer_state_dict(sd)
    for name, w in e2.master_state_dict().items():
        assert torch.equal(w, weights[name]), name
    x, y = _data(7)
    for m, e in ((m1, e1), (m2, e2)):
        e.zero_grad()
        ((m(x) - y) ** 2).mean().backward()
        e.step()
    for (name, a), (_, b) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.allclose(a, b, atol=1e-6), name


def _worker(rank, world, port, out_path, shard):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    model = _model()
    eng = TrainEngine(model, EngineConfig(**CFG, shard=shard), device="cpu")
    owners = sorted(set(eng.muon_owner.values()))
    for step in range(3):
        x, y = _data(step, rank)
        eng.zero_grad()
        ((model(x) - y) ** 2).mean().backward()
        eng.step()
    full = eng.master_state_dict()
    sd = eng.optimizer_state_dict(first_rank_only=True)
    if rank == 0:
        torch.save({"master": full, "momentum": {k: v["exp_avg"] for k, v in sd["state"].items()}, "owners": owners,
                    "weights": {k: v.detach().clone() for k, v in model.state_dict().items()}}, out_path)
    dist.barrier()  # nobody tears its connections down while a peer still talks
    dist.barrier()
    dist.destroy_process_group()
    os._exit(0)  # skip interpreter teardown: gloo aborts there now and then


@pytest.mark.parametrize("shard", [False, True])
def test_two_gloo_ranks_with_owned_matrices_equal_one_rank(tmp_path, shard):
    out = tmp_path / "muon.pt"
    mp.spawn(_worker, args=(2, 29651 + int(shard), str(out), shard), nprocs=2, join=True)
    got = torch.load(out)
    assert got["owners"] == [0, 1]  # the three matrices are spread over both ranks
    model = _model()
    eng = TrainEngine(model, EngineConfig(**CFG), device="cpu")
    for step in range(3):
        eng.zero_grad()
        total = 0
        for rank in range(2):
            x, y = _data(step, rank)
            total = total + ((model(x) - y) ** 2).mean() / 2
        total.backward()
        eng.step()
    want = eng.master_state_dict()
    want_m = {k: v["exp_avg"] for k, v in eng.optimizer_state_dict()["state"].items()}
    for name, w in want.items():
        assert torch.allclose(got["master"][name], w, rtol=1e-4, atol=1e-6), name
        assert torch.allclose(got["momentum"][name], want_m[name], rtol=1e-4, atol=1e-7), name
    for name, w in model.state_dict().items():  # the non-owner's compute weights were refreshed too
        assert torch.allclose(got["weights"][name], w, rtol=1e-4, atol=1e-6), name
