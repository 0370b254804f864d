"""Expert parallelism end to end on CPU: two gloo ranks, each holding half of the experts of a
sparse MoE block (tokens exchanged with all-to-all), trained by the engine with the experts as
rank-local parameters, must take the same optimizer steps as one process that holds all experts
and sees both ranks' batches; state dicts present the experts as the stack of all ranks."""

import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from torch import nn

from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.models.layers import Linear
from speculators_b200.models.moe import SparseMoeBlock
from speculators_b200.parallel.engine import EngineConfig, TrainEngine

CFG = dict(model_type="qwen3_next", hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
           head_dim=16, vocab_size=64, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=24, shared_expert_intermediate_size=16,
           norm_topk_prob=True)
STEPS = 3


class Net(nn.Module):
    def __init__(self, ep_group=None):
        super().__init__()
        torch.manual_seed(0)
        self.inp = Linear(32, 32)
        self.moe = SparseMoeBlock(TransformerLayerConfig(**CFG), ep_group=ep_group)
        self.gain = nn.Parameter(torch.ones(32))

    def forward(self, x):
        return self.moe(torch.tanh(self.inp(x))) * self.gain


def _data(step, rank):
    g = torch.Generator().manual_seed(31 * step + rank)
    return torch.randn(40, 32, generator=g), torch.randn(40, 32, generator=g)


def _engine(model, shard, optimizer):
    return TrainEngine(model, EngineConfig(lr=1e-2, compute_dtype=torch.float32, shard=shard, optimizer=optimizer, max_grad_norm=0.5), device="cpu")


def _worker(rank, world, port, out_path, shard, optimizer):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = Net()  # all experts, the common initialisation
    model = Net(ep_group=dist.group.WORLD)
    model.load_state_dict(full.state_dict())  # the block keeps its own half of the experts
    assert model.moe.experts.gate_up_proj.shape[0] == 4
    assert torch.equal(model.moe.experts.down_proj, full.moe.experts.down_proj[rank * 4 : rank * 4 + 4])
    eng = _engine(model, shard, optimizer)
    assert eng.local_names == {"moe.experts.gate_up_proj", "moe.experts.down_proj"} and eng.total > eng.shared_end
    for step in range(STEPS):
        x, y = _data(step, rank)
        eng.zero_grad()
        ((model(x) - y) ** 2).mean().backward()
        eng.step()
    master = eng.master_state_dict()
    sd = eng.optimizer_state_dict(first_rank_only=True)
    if rank == 0:
        torch.save({"master": master, "exp_avg": {k: v["exp_avg"] for k, v in sd["state"].items()}}, out_path)
    dist.barrier()  # nobody tears its connections down while a peer still talks
    dist.destroy_process_group()
    os._exit(0)  # skip interpreter teardown: gloo's worker threads occasionally abort there (no Python frame on the stack)


@pytest.mark.parametrize("shard,optimizer", [(False, "adamw"), (True, "adamw"), (True, "muon")])
def test_expert_parallel_training_equals_replicated_experts(tmp_path, shard, optimizer):
    out = tmp_path / "ep.pt"
    port = 29661 + 2 * int(shard) + (optimizer == "muon")
    mp.spawn(_worker, args=(2, port, str(out), shard, optimizer), nprocs=2, join=True)
    got = torch.load(out)
    model = Net()
    eng = _engine(model, False, optimizer)
    for step in range(STEPS):
        eng.zero_grad()
        total = 0
        for rank in range(2):
            x, y = _data(step, rank)
            total = total + ((model(x) - y) ** 2).mean() / 2
        total.backward()
        eng.step()
    want = eng.master_state_dict()
    want_m = {k: v["exp_avg"] for k, v in eng.optimizer_state_dict()["state"].items()}
    assert set(got["master"]) == set(want)
    for name, w in want.items():
        assert got["master"][name].shape == w.shape, name  # experts come back as the full stack
        assert torch.allclose(got["master"][name], w, rtol=2e-4, atol=2e-6), (name, float((got["master"][name] - w).abs().max()))
        assert torch.allclose(got["exp_avg"][name], want_m[name], rtol=2e-4, atol=1e-7), name
