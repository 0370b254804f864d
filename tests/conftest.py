import json
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

os.environ.setdefault("SB200_NO_TQDM", "1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "multi_gpu: needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multi_gpu" in item.keywords:
            item.add_marker(skip)


TINY_VERIFIER = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 64, "num_hidden_layers": 4,
    "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "intermediate_size": 96, "vocab_size": 128,
    "rms_norm_eps": 1e-5, "rope_theta": 10000.0, "max_position_embeddings": 512, "hidden_act": "silu",
}


@pytest.fixture()
def tiny_verifier_dir(tmp_path):
    from safetensors.torch import save_file

    d = tmp_path / "verifier"
    d.mkdir()
    (d / "config.json").write_text(json.dumps(TINY_VERIFIER))
    g = torch.Generator().manual_seed(0)
    save_file(
        {
            "model.embed_tokens.weight": torch.randn(128, 64, generator=g),
            "lm_head.weight": torch.randn(128, 64, generator=g),
            "model.norm.weight": torch.rand(64, generator=g) + 0.5,
        },
        str(d / "model.safetensors"),
    )
    return str(d)


@pytest.fixture()
def tiny_vocab_maps():
    g = torch.Generator().manual_seed(1)
    t2d = torch.zeros(128, dtype=torch.bool)
    t2d[torch.randperm(128, generator=g)[:32]] = True
    kept = torch.nonzero(t2d).squeeze(1)
    d2t = kept - torch.arange(32)
    return t2d, d2t


def make_tiny_eagle3(verifier_dir, maps, num_layers=1, **overrides):
    import speculators_b200 as sb
    from speculators_b200.layer_config import TransformerLayerConfig

    t2d, d2t = maps
    kw = dict(draft_vocab_size=32, norm_before_residual=True, ttt_steps=3, verifier_name_or_path=verifier_dir,
              target_layer_ids=[1, 2, 3], norm_before_fc=True, norm_output=True)
    kw.update(overrides)
    torch.manual_seed(0)
    return sb.Eagle3DraftModel.from_training_args(
        TransformerLayerConfig(**dict(TINY_VERIFIER, num_hidden_layers=num_layers)), t2d=t2d, d2t=d2t, **kw
    )


def make_tiny_batch(T=40, seed=0, docs=(13, 17, 6), pad=4, hidden=64, aux=3, vocab=128):
    g = torch.Generator().manual_seed(seed)
    doc = torch.cat([torch.full((n,), i) for i, n in enumerate(docs)] + [torch.full((pad,), -1)])[:T]
    pos = torch.cat([torch.arange(1, n + 1) for n in docs] + [torch.arange(1, pad + 1)])[:T]
    return dict(
        hidden_states=torch.randn(1, T, aux * hidden, generator=g),
        input_ids=torch.randint(0, vocab, (1, T), generator=g),
        document_ids=doc.unsqueeze(0),
        loss_mask=(torch.rand(1, T, generator=g) > 0.3) & (doc != -1).unsqueeze(0),
        position_ids=pos.unsqueeze(0),
        verifier_last_hidden_states=torch.randn(1, T, hidden, generator=g),
    )
