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


# ---- weights from a Hugging Face style checkpoint -----------------------------------------------------
def _write_checkpoint(path):
    """Three full layers and the embedding, saved under Hugging Face names in two shards with an index."""
    import json

    from safetensors.torch import save_file

    from speculators_b200.layer_config import TransformerLayerConfig
    from speculators_b200.models.layers import DecoderLayer

    torch.manual_seed(11)
    cfg = TransformerLayerConfig(**CFG)
    tensors = {"model.embed_tokens.weight": torch.randn(CFG["vocab_size"], CFG["hidden_size"]) * 0.05}
    layers = []
    for i in range(CFG["num_hidden_layers"]):
        layer = DecoderLayer(cfg, i)
        with torch.no_grad():
            for p in layer.parameters():
                p.copy_(torch.randn_like(p) * (0.05 if p.ndim == 2 else 0.2) + (1.0 if p.ndim == 1 else 0.0))
        layers.append(layer)
        tensors.update({f"model.layers.{i}.{k}": v.clone() for k, v in layer.state_dict().items()})
    os.makedirs(path, exist_ok=True)
    names = sorted(tensors)
    shards = {"model-00001-of-00002.safetensors": names[::2], "model-00002-of-00002.safetensors": names[1::2]}
    for file, keys in shards.items():
        save_file({k: tensors[k].contiguous() for k in keys}, os.path.join(path, file))
    with open(os.path.join(path, "model.safetensors.index.json"), "w") as fh:
        json.dump({"weight_map": {k: f for f, keys in shards.items() for k in keys}}, fh)
    with open(os.path.join(path, "config.json"), "w") as fh:
        json.dump(CFG, fh)
    return tensors["model.embed_tokens.weight"], layers


def _checkpoint_worker(rank, world, port, ckpt, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ids, doc, pos = _inputs()
    tp = TensorParallelVerifier.from_pretrained(ckpt, device="cpu", dtype=torch.float32)
    out = tp.forward(ids, [1, 3], document_ids=doc, position_ids=pos)  # counted ids: states after 1 and after 3 layers
    torch.save(out, f"{out_path}.{rank}")
    dist.barrier()
    dist.destroy_process_group()
    os._exit(0)


def test_tensor_parallel_verifier_loads_checkpoint_slices(tmp_path):
    from speculators_b200.models.eagle3.attention import causal_document_interval
    from speculators_b200.models.layers import RotaryTable
    from speculators_b200.layer_config import TransformerLayerConfig
    from speculators_b200.ops import AttnSpec

    ckpt = str(tmp_path / "ckpt")
    embed, layers = _write_checkpoint(ckpt)
    ids, doc, pos = _inputs()
    lo, hi = causal_document_interval(doc)
    rotary = RotaryTable(TransformerLayerConfig(**CFG))
    with torch.no_grad():  # the plain single-device forward over the full layers
        h = torch.nn.functional.embedding(ids, embed)
        kept = {}
        for i, layer in enumerate(layers):
            h = layer(h, pos, rotary, AttnSpec(lo=lo, hi=hi))
            kept[i] = h
    want = {"hidden_states": torch.cat([kept[0], kept[2]], dim=-1), "verifier_last_hidden_states": h}
    out = tmp_path / "tpck"
    mp.spawn(_checkpoint_worker, args=(2, 29683, ckpt, str(out)), nprocs=2, join=True)
    for rank in range(2):
        got = torch.load(f"{out}.{rank}")
        for key in want:
            assert torch.allclose(got[key], want[key], atol=2e-5, rtol=1e-4), (rank, key, float((got[key] - want[key]).abs().max()))


def test_row_parallel_biases_are_refused(monkeypatch):
    import pytest

    from speculators_b200.verifier import tp as tp_mod

    assert TensorParallelVerifier(dict(CFG, attention_bias=True)).world == 1  # one rank: nothing is summed over ranks
    monkeypatch.setattr(tp_mod.dist, "is_initialized", lambda: True)
    monkeypatch.setattr(tp_mod.dist, "get_world_size", lambda group=None: 2)
    monkeypatch.setattr(tp_mod.dist, "get_rank", lambda group=None: 0)
    with pytest.raises(ValueError, match="attention_bias"):
        TensorParallelVerifier(dict(CFG, attention_bias=True))
    with pytest.raises(ValueError, match="mlp_bias"):
        TensorParallelVerifier(dict(CFG, mlp_bias=True))
