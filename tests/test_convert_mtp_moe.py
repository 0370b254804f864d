"""Converters (EAGLE-3, DFlash, MTP incl. MoE expert fusing), the MTP model and the
MoE block (single process and 2-rank expert parallel over gloo)."""

import json
import os

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
from safetensors.torch import load_file, save_file

import speculators_b200 as sb
from speculators_b200.__main__ import main as cli_main
from speculators_b200.convert.entrypoints import convert_model, maybe_convert_external_checkpoint
from speculators_b200.convert.mtp.converter import MTPConverter
from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.models.dflash import DFlashDraftModel
from speculators_b200.models.moe import SparseMoeBlock, expert_forward
from speculators_b200.models.mtp import MTPDraftModel

from conftest import TINY_VERIFIER, make_tiny_eagle3

QWEN = dict(TINY_VERIFIER, model_type="qwen3", architectures=["Qwen3ForCausalLM"])


def test_eagle3_research_checkpoint_conversion(tiny_verifier_dir, tiny_vocab_maps, tmp_path):
    model = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps, norm_before_fc=False, norm_output=False)
    sd = {k: v for k, v in model.state_dict().items() if k not in ("verifier_lm_head.weight", "verifier_norm.weight", "embed_tokens.weight")}
    research = {(k.replace("layers.0.", "midlayer.") if k.startswith("layers.0.") else k): v.contiguous() for k, v in sd.items()}
    src = tmp_path / "research"
    src.mkdir()
    save_file(research, str(src / "model.safetensors"))
    (src / "config.json").write_text(json.dumps({"hidden_size": 64, "intermediate_size": 96, "num_attention_heads": 4, "num_key_value_heads": 2,
                                                 "head_dim": 16, "draft_vocab_size": 32, "rms_norm_eps": 1e-5, "num_hidden_layers": 1}))
    out = tmp_path / "converted"
    assert cli_main(["convert", str(src), "--verifier", tiny_verifier_dir, "--algorithm", "eagle3", "--output-path", str(out),
                     "--validate-device", "cpu", "--algorithm-kwargs", '{"norm_before_residual": true, "eagle_aux_hidden_state_layer_ids": [1, 2, 3]}']) == 0
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["speculators_model_type"] == "eagle3" and cfg["norm_before_residual"] is True and cfg["transformer_layer_config"]["vocab_size"] == 128
    conv = load_file(str(out / "model.safetensors"))
    assert "layers.0.self_attn.q_proj.weight" in conv and not any(k.startswith("midlayer.") for k in conv)
    loaded = sb.SpeculatorModel.from_pretrained(str(out))
    assert torch.equal(loaded.fc.weight, model.fc.weight) and not torch.isnan(loaded.embed_tokens.weight).any()


def test_dflash_external_checkpoint_with_fused_qkv(tiny_verifier_dir, tmp_path):
    torch.manual_seed(0)
    cfg = TransformerLayerConfig(**dict(QWEN, num_hidden_layers=2, layer_types=["full_attention", "sliding_attention"], sliding_window=8))
    ref = DFlashDraftModel(sb.models.dflash.DFlashSpeculatorConfig(transformer_layer_config=cfg, draft_vocab_size=128, block_size=4,
                                                                   aux_hidden_state_layer_ids=[1, 2, 3], mask_token_id=5))
    ext = {}
    for k, v in ref.state_dict().items():
        if k in ("embed_tokens.weight", "lm_head.weight", "verifier_lm_head.weight", "verifier_norm.weight"):
            continue
        ext[k] = v.contiguous()
    # external layout: fused qkv, an extra gate projection and aux norms, a wider fc
    for i in range(2):
        q, k_, v = (ext.pop(f"layers.{i}.self_attn.{n}_proj.weight") for n in "qkv")
        ext[f"layers.{i}.self_attn.qkv_proj.weight"] = torch.cat([q, k_, v])
        ext[f"layers.{i}.self_attn.g_proj.weight"] = torch.zeros(4, 4)
    ext["aux_hidden_norms.0.weight"] = torch.ones(64)
    ext["fc.weight"] = torch.cat([ext["fc.weight"], torch.zeros(64, 64)], dim=1)
    src = tmp_path / "ext"
    src.mkdir()
    save_file(ext, str(src / "model.safetensors"))
    source_cfg = dict(cfg.to_dict(), architectures=["DFlashDraftModel"], block_size=4, dflash_config={"target_layer_ids": [0, 1, 2, 3], "mask_token_id": 5})
    (src / "config.json").write_text(json.dumps(source_cfg))
    with pytest.raises(ValueError, match="requires a verifier"):
        maybe_convert_external_checkpoint(str(src))
    loaded = sb.SpeculatorModel.from_pretrained(str(src), verifier=tiny_verifier_dir)  # auto-conversion path
    assert isinstance(loaded, DFlashDraftModel) and loaded.config.aux_hidden_state_layer_ids == [1, 2, 3]
    assert torch.equal(loaded.layers[1].self_attn.qkv_proj.weight, ref.layers[1].self_attn.qkv_proj.weight)
    assert loaded.fc.weight.shape == (64, 192) and not torch.isnan(loaded.lm_head.weight).any()
    with pytest.raises(NotImplementedError):
        maybe_convert_external_checkpoint(tiny_verifier_dir, verifier=tiny_verifier_dir)


def _verifier_with_mtp(tmp_path, moe=False):
    d = tmp_path / "v_mtp"
    d.mkdir()
    cfg = dict(QWEN)
    if moe:
        cfg.update(model_type="qwen3_next", num_experts=4, num_experts_per_tok=2, moe_intermediate_size=24, shared_expert_intermediate_size=24,
                   partial_rotary_factor=0.5, layer_types=["linear_attention", "full_attention"] * 2)
    (d / "config.json").write_text(json.dumps(cfg))
    g = torch.Generator().manual_seed(0)
    r = lambda *s: torch.randn(*s, generator=g) * 0.05  # noqa: E731
    w = {"model.embed_tokens.weight": r(128, 64), "lm_head.weight": r(128, 64), "model.norm.weight": torch.ones(64),
         "mtp.fc.weight": r(64, 128), "mtp.norm.weight": torch.ones(64), "mtp.pre_fc_norm_hidden.weight": torch.ones(64),
         "mtp.pre_fc_norm_embedding.weight": torch.ones(64), "mtp.layers.0.input_layernorm.weight": torch.ones(64),
         "mtp.layers.0.post_attention_layernorm.weight": torch.ones(64), "mtp.layers.0.self_attn.k_proj.weight": r(32, 64),
         "mtp.layers.0.self_attn.v_proj.weight": r(32, 64), "mtp.layers.0.self_attn.o_proj.weight": r(64, 64),
         "mtp.layers.0.self_attn.q_norm.weight": torch.ones(16), "mtp.layers.0.self_attn.k_norm.weight": torch.ones(16)}
    if moe:
        w["mtp.layers.0.self_attn.q_proj.weight"] = r(128, 64)
        w["mtp.layers.0.mlp.gate.weight"] = r(4, 64)
        for e in range(4):
            w[f"mtp.layers.0.mlp.experts.{e}.gate_proj.weight"] = r(24, 64)
            w[f"mtp.layers.0.mlp.experts.{e}.up_proj.weight"] = r(24, 64)
            w[f"mtp.layers.0.mlp.experts.{e}.down_proj.weight"] = r(64, 24)
        for n, s in (("gate_proj", (24, 64)), ("up_proj", (24, 64)), ("down_proj", (64, 24))):
            w[f"mtp.layers.0.mlp.shared_expert.{n}.weight"] = r(*s)
        w["mtp.layers.0.mlp.shared_expert_gate.weight"] = r(1, 64)
    else:
        w["mtp.layers.0.self_attn.q_proj.weight"] = r(64, 64)
        for n, s in (("gate_proj", (96, 64)), ("up_proj", (96, 64)), ("down_proj", (64, 96))):
            w[f"mtp.layers.0.mlp.{n}.weight"] = r(*s)
    save_file(w, str(d / "model.safetensors"))
    return str(d), w


@pytest.mark.parametrize("moe", [False, True])
def test_mtp_extract_train_and_convert(moe, tmp_path):
    vdir, raw = _verifier_with_mtp(tmp_path, moe)
    sd = MTPConverter().convert_to_state_dict(vdir)
    assert "mtp_layers.0.input_proj.weight" in sd and "mtp_layers.0.hidden_layernorm.weight" in sd
    if moe:
        assert sd["mtp_layers.0.mlp.experts.gate_up_proj"].shape == (4, 48, 64) and sd["mtp_layers.0.mlp.experts.down_proj"].shape == (4, 64, 24)
        assert torch.equal(sd["mtp_layers.0.mlp.experts.gate_up_proj"][2, 24:], raw["mtp.layers.0.mlp.experts.2.up_proj.weight"])
    from speculators_b200.models.utils import get_verifier_config

    model = MTPDraftModel.from_training_args(get_verifier_config(vdir), num_speculative_steps=2, verifier_name_or_path=vdir)
    assert not hasattr(model, "verifier_lm_head") and not torch.isnan(model.lm_head.weight).any()
    T = 20
    g = torch.Generator().manual_seed(1)
    kw, _ = MTPDraftModel.get_trainer_kwargs(num_speculative_steps=2, step_weight_beta=0.6)
    logits, loss, metrics = model(input_ids=torch.randint(0, 128, (1, T), generator=g), hidden_states=torch.randn(1, T, 64, generator=g),
                                  loss_mask=torch.ones(1, T), **kw)
    loss.backward()
    assert len(logits) == 2 and logits[0].shape == (1, T - 3, 128) and {"loss_step_0", "loss_step_1", "loss_sum"} <= set(metrics)
    assert model.mtp_layers[0].input_proj.weight.grad is not None
    out = tmp_path / "mtp_conv"
    convert_model(vdir, verifier=vdir, algorithm="mtp", output_path=str(out), validate_device="cpu", num_speculative_steps=2)
    saved = load_file(str(out / "model.safetensors"))
    assert all(k.startswith("mtp_layers.") for k in saved)
    cfg = json.loads((out / "config.json").read_text())
    assert cfg["speculators_model_type"] == "mtp" and cfg["num_nextn_predict_layers"] == 1
    with pytest.raises(ValueError, match="Non-contiguous"):
        MTPConverter.fuse_moe_experts({"a.experts.0.gate_proj.weight": torch.zeros(1, 1), "a.experts.2.gate_proj.weight": torch.zeros(1, 1)})


def test_mtp_degenerate_lengths(tmp_path):
    vdir, _ = _verifier_with_mtp(tmp_path)
    from speculators_b200.models.utils import get_verifier_config

    model = MTPDraftModel.from_training_args(get_verifier_config(vdir), num_speculative_steps=3, verifier_name_or_path=vdir)
    logits, loss, _ = model(input_ids=torch.zeros(1, 2, dtype=torch.long), hidden_states=torch.zeros(1, 2, 64))
    assert logits == [] and float(loss) == 0.0
    with pytest.raises(ValueError):
        model(input_ids=torch.zeros(1, 9, dtype=torch.long), hidden_states=torch.zeros(1, 9, 64), step_weights=[1.0])


def _moe_cfg():
    return TransformerLayerConfig(**dict(QWEN, model_type="qwen3_next", num_experts=8, num_experts_per_tok=2, moe_intermediate_size=16,
                                         shared_expert_intermediate_size=16))


def test_moe_block_matches_dense_definition():
    torch.manual_seed(0)
    block = SparseMoeBlock(_moe_cfg())
    x = torch.randn(13, 64)
    top_p, top_e = block.route(x)
    ref = torch.zeros_like(x)
    for k in range(2):
        ref += top_p[:, k : k + 1] * expert_forward(x, top_e[:, k], block.experts.gate_up_proj, block.experts.down_proj)
    ref += torch.sigmoid(block.shared_expert_gate(x)) * block.shared_expert(x)
    assert torch.allclose(block(x), ref, atol=1e-5)
    assert torch.allclose(top_p.sum(-1), torch.ones(13), atol=1e-5)


def _ep_worker(rank, world, port, out_path):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    full = SparseMoeBlock(_moe_cfg())  # identical on both ranks (same seed)
    ep = SparseMoeBlock(_moe_cfg(), ep_group=dist.group.WORLD)
    ep.gate.load_state_dict(full.gate.state_dict())
    ep.shared_expert.load_state_dict(full.shared_expert.state_dict())
    ep.shared_expert_gate.load_state_dict(full.shared_expert_gate.state_dict())
    lo = rank * ep.num_local
    with torch.no_grad():
        ep.experts.gate_up_proj.copy_(full.experts.gate_up_proj[lo : lo + ep.num_local])
        ep.experts.down_proj.copy_(full.experts.down_proj[lo : lo + ep.num_local])
    torch.manual_seed(100 + rank)
    x = torch.randn(9 + rank, 64, requires_grad=True)
    y = ep(x)
    y.sum().backward()
    xr = x.detach().clone().requires_grad_()
    yr = full(xr)
    yr.sum().backward()
    ok = torch.allclose(y, yr, atol=1e-5) and torch.allclose(x.grad, xr.grad, atol=1e-5)
    gathered = [None] * world
    dist.all_gather_object(gathered, bool(ok))
    if rank == 0:
        with open(out_path, "w") as fh:
            json.dump(gathered, fh)
    dist.barrier()
    dist.destroy_process_group()
    os._exit(0)  # skip interpreter teardown: gloo aborts there now and then


def test_moe_expert_parallel_two_ranks_gloo(tmp_path):
    out = tmp_path / "ep.json"
    mp.spawn(_ep_worker, args=(2, 29631, str(out)), nprocs=2, join=True)
    assert json.loads(out.read_text()) == [True, True]
