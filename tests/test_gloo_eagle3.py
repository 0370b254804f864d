"""EAGLE-3 data parallelism on CPU: two gloo ranks (sharded optimizer state, one batch
each) must take the same optimizer steps as one process that sees both batches, and the
benchmark's plumbing configuration must run end to end on two ranks."""

import json
import os
import subprocess
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import speculators_b200 as sb
from speculators_b200.parallel.engine import EngineConfig, TrainEngine

from conftest import TINY_VERIFIER, make_tiny_batch, make_tiny_eagle3

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STEPS = 3


def _maps():
    g = torch.Generator().manual_seed(1)
    t2d = torch.zeros(128, dtype=torch.bool)
    t2d[torch.randperm(128, generator=g)[:32]] = True
    kept = torch.nonzero(t2d).squeeze(1)
    return t2d, kept - torch.arange(32)


def _kwargs():
    return sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=2, ttt_step_loss_decay=1.0)[0]


def _worker(rank, world, port, vdir, out_path, shard):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    model = make_tiny_eagle3(vdir, _maps())
    eng = TrainEngine(model, EngineConfig(lr=1e-2, compute_dtype=torch.float32, shard=shard), device="cpu")
    for step in range(STEPS):
        eng.zero_grad()
        _, loss, _ = model(**make_tiny_batch(T=40, seed=10 * step + rank), **_kwargs())
        loss.backward()
        eng.step()
    full = eng.master_state_dict()  # collective
    state = eng.optimizer_state_dict(first_rank_only=True)
    if rank == 0:
        torch.save({"master": full, "moments": {k: v["exp_avg"] for k, v in state["state"].items()}}, out_path)
    else:
        assert state["state"] == {}  # the full state is assembled on the writer only
    dist.barrier()  # nobody tears its connections down while a peer still talks
    dist.barrier()
    dist.destroy_process_group()
    os._exit(0)  # skip interpreter teardown: gloo aborts there now and then


def _single(vdir):
    model = make_tiny_eagle3(vdir, _maps())
    eng = TrainEngine(model, EngineConfig(lr=1e-2, compute_dtype=torch.float32), device="cpu")
    for step in range(STEPS):
        eng.zero_grad()
        total = 0
        for rank in range(2):
            _, loss, _ = model(**make_tiny_batch(T=40, seed=10 * step + rank), **_kwargs())
            total = total + loss / 2
        total.backward()
        eng.step()
    return eng.master_state_dict(), {k: v["exp_avg"] for k, v in eng.optimizer_state_dict()["state"].items()}


def _check(tmp_path, tiny_verifier_dir, shard, port):
    out = tmp_path / f"ranks_{shard}.pt"
    mp.spawn(_worker, args=(2, port, tiny_verifier_dir, str(out), shard), nprocs=2, join=True)
    got = torch.load(out)
    want_master, want_m = _single(tiny_verifier_dir)
    assert set(got["master"]) == set(want_master)
    for name, w in want_master.items():
        assert torch.allclose(got["master"][name], w, rtol=1e-4, atol=1e-6), name
        assert torch.allclose(got["moments"][name], want_m[name], rtol=1e-4, atol=1e-7), name


def test_two_sharded_gloo_ranks_equal_one_rank(tmp_path, tiny_verifier_dir):
    _check(tmp_path, tiny_verifier_dir, True, 29641)


def test_two_replicated_gloo_ranks_equal_one_rank(tmp_path, tiny_verifier_dir):
    _check(tmp_path, tiny_verifier_dir, False, 29642)


def test_bench_plumbing_config_two_gloo_ranks():
    """The benchmark's CPU plumbing configuration: tiny 4-layer Llama verifier run in plain
    PyTorch for the hidden states, draft vocab 512, TTT 3, two gloo ranks, fp32."""
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29643", "bench.py", "--gpus", "2", "--model", "tiny", "--device", "cpu", "--seq-len", "128",
           "--steps", "2", "--warmup", "3", "--regions", "1"]
    out = subprocess.run(cmd, cwd=REPO, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stderr[-3000:]
    rec = json.loads([ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1])
    assert rec["n_gpus"] == 2 and rec["config"]["parallelism"] == "dp2-sharded" and rec["impl_detail"]["optimizer_comm"] == "gloo"
    assert rec["dtype"] == "fp32" and len(rec["loss_trace"]) == 6 and all(x == x and x > 0 for x in rec["loss_trace"])
    assert rec["loss_trace"][-1] < rec["loss_trace"][0]
    assert TINY_VERIFIER["hidden_size"] == 64
