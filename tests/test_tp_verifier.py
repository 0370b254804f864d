"""Tensor-parallel verifier forward: two gloo ranks (column / row parallel layers, partial sums
all-reduced) must reproduce the single-device forward of the same seeded random verifier."""

import os

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from speculators_b200.verifier import RandomVerifier, TensorParallelVerifier

CFG = dict(architectures=["Qwen3ForCausalLM"], model_type="qwen3", hidden_size=64, intermediate_size=96, num_hidden_layers=3,
           num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=128, max_position_embeddings=256, rms_norm_eps=1e-6,
           rope_theta=10000.0, hidden_act="silu")


def _inputs():
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 128, (50,), generator=g)
    doc = torch.cat([torch.zeros(20), torch.ones(25), torch.full((5,), -1)]).long()
    pos = torch.cat([torch.arange(20), torch.arange(25), torch.arange(5)])
    return ids, doc, pos


def _worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ids, doc, pos = _inputs()
    tp = TensorParallelVerifier(CFG, seed=3)
    assert tp.local_cfg.num_attention_heads == 2 and tp.local_cfg.num_key_value_heads == 1 and tp.local_cfg.intermediate_size == 48
    out = tp.forward(ids, [0, 2], document_ids=doc, position_ids=pos)
    torch.save(out, f"{out_path}.{rank}")
    dist.barrier()
    dist.destroy_process_group()
    os._exit(0)


def test_two_rank_tensor_parallel_forward_equals_single_device(tmp_path):
    out = tmp_path / "tp"
    mp.spawn(_worker, args=(2, 29681, str(out)), nprocs=2, join=True)
    ids, doc, pos = _inputs()
    want = RandomVerifier(CFG, seed=3).forward(ids, [0, 2], document_ids=doc, position_ids=pos)
    for rank in range(2):
        got = torch.load(f"{out}.{rank}")
        for key in ("hidden_states", "verifier_last_hidden_states"):
            assert got[key].shape == want[key].shape
            assert torch.allclose(got[key], want[key], atol=2e-5, rtol=1e-4), (rank, key, float((got[key] - want[key]).abs().max()))
