import os
import sys

import pytest
import torch

import speculators_b200 as sb
from speculators_b200.models.eagle3.attention import causal_document_interval, dense_ttt_mask, ttt_attn_spec
from speculators_b200.models.eagle3.data import shift_batch
from speculators_b200.ops import masked_attention_reference

from conftest import ROOT, TINY_VERIFIER, make_tiny_batch, make_tiny_eagle3


@pytest.mark.parametrize("window", [None, 5])
@pytest.mark.parametrize("step", [0, 1, 3])
def test_ttt_spec_equals_mask_definition(step, window):
    doc = torch.tensor([0] * 7 + [1] * 9 + [2] * 3 + [-1] * 4)
    spec = ttt_attn_spec(doc, step, sliding_window=window)
    T = doc.numel()
    assert torch.equal(spec.dense(T, step * T), dense_ttt_mask(doc, step, window))


def test_interval_padding_and_restart():
    doc = torch.tensor([3, 3, 3, 8, 8, -1, -1])
    lo, hi = causal_document_interval(doc)
    assert lo.tolist() == [0, 0, 0, 3, 3, 5, 6] and hi.tolist() == [1, 2, 3, 4, 5, 6, 7]


def test_attention_oracle_with_extras_matches_dense_softmax():
    torch.manual_seed(0)
    T, nh, nkv, hd, s = 12, 4, 2, 8, 2
    doc = torch.tensor([0] * 5 + [1] * 5 + [-1] * 2)
    q = torch.randn(T, nh, hd)
    ks = [torch.randn(T, nkv, hd) for _ in range(s + 1)]
    vs = [torch.randn(T, nkv, hd) for _ in range(s + 1)]
    out = masked_attention_reference(q, ks[0], vs[0], ttt_attn_spec(doc, s), torch.cat(ks[1:]), torch.cat(vs[1:]))
    mask = dense_ttt_mask(doc, s)
    K = torch.cat(ks).repeat_interleave(2, 1)
    V = torch.cat(vs).repeat_interleave(2, 1)
    sc = torch.einsum("qhd,khd->hqk", q, K) * hd**-0.5
    ref = torch.einsum("hqk,khd->qhd", sc.masked_fill(~mask[None], float("-inf")).softmax(-1), V)
    assert torch.allclose(out, ref, atol=1e-5)


def test_shift_batch():
    b = dict(input_ids=torch.arange(5), hidden_states=torch.arange(10.0).reshape(5, 2),
             verifier_last_hidden_states=torch.arange(5.0).reshape(5, 1), loss_mask=torch.ones(5), lengths=torch.tensor([5]),
             position_ids=torch.arange(5))
    s = shift_batch(b)
    assert s["input_ids"].tolist() == [1, 2, 3, 4] and s["hidden_states"][:, 0].tolist() == [0, 2, 4, 6]
    assert s["position_ids"].tolist() == [1, 2, 3, 4] and s["lengths"].item() == 4
    assert shift_batch(dict(b, lengths=torch.tensor([0])))["lengths"].item() == 0


def test_forward_backward_metrics_and_frozen_params(tiny_verifier_dir, tiny_vocab_maps):
    model = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps, num_layers=2)
    kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=3, ttt_step_loss_decay=0.8)
    assert kwargs["return_draft_tokens"] is False  # the trainer path skips the argmax over [T, V]
    toks, loss, metrics = model(**make_tiny_batch(), **{**kwargs, "return_draft_tokens": True})
    assert len(toks) == 3 and toks[0].shape == (1, 40)
    assert model(**make_tiny_batch(), **kwargs)[0] == []
    for s in range(3):
        for key in ("loss", "full_acc", "cond_acc"):
            assert f"{key}_{s}_sum" in metrics and f"{key}_{s}_total" in metrics
    assert torch.isclose(metrics["loss_sum"], loss.detach())
    loss.backward()
    trainable = {n for n, p in model.named_parameters() if p.requires_grad}
    assert not {"embed_tokens.weight", "lm_head.weight", "verifier_lm_head.weight", "verifier_norm.weight"} & trainable
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for n, p in model.named_parameters() if p.requires_grad)
    assert not torch.isnan(model.lm_head.weight).any()  # verifier weights were loaded over the NaN sentinels


def test_save_load_round_trip_and_key_layout(tiny_verifier_dir, tiny_vocab_maps, tmp_path):
    from safetensors.torch import load_file

    model = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
    model.save_pretrained(tmp_path)
    keys = set(load_file(str(tmp_path / "model.safetensors")))
    assert {"fc.weight", "layers.0.self_attn.q_proj.weight", "layers.0.self_attn.k_proj.weight", "layers.0.mlp.gate_proj.weight",
            "layers.0.mlp.up_proj.weight", "layers.0.hidden_norm.weight", "norm.weight", "d2t", "t2d", "embed_tokens.weight",
            "lm_head.weight", "input_norm.weight"} <= keys
    assert not {"verifier_lm_head.weight", "verifier_norm.weight"} & keys
    assert not any("qkv_proj" in k or "gate_up_proj" in k for k in keys)
    loaded = sb.SpeculatorModel.from_pretrained(str(tmp_path))
    assert isinstance(loaded, sb.Eagle3DraftModel)
    kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="ce", ttt_steps=2, ttt_step_loss_decay=1.0)
    batch = make_tiny_batch()
    assert torch.allclose(model(**batch, **kwargs)[1], loaded(**batch, **kwargs)[1])


def test_vocab_mapping_validation(tiny_verifier_dir, tiny_vocab_maps):
    model = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps)
    t2d, d2t = tiny_vocab_maps
    with pytest.raises(ValueError):
        model.load_vocab_mappings(t2d, None)
    with pytest.raises(ValueError):
        model.load_vocab_mappings(t2d[:-1], d2t)
    bad = t2d.clone(); bad[:] = False
    with pytest.raises(ValueError):
        model.load_vocab_mappings(bad, d2t)


REF = os.path.join(ROOT, "baseline", "_ref")


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "speculators")), reason="reference not installed under baseline/_ref")
@pytest.mark.parametrize("loss_fn", ["kl_div", '{"ce": 0.3, "jsd": 0.7}'])
def test_numerical_parity_with_reference_sdpa_path(tiny_verifier_dir, tiny_vocab_maps, loss_fn):
    """Same weights, same batch: loss, every metric and the gradients agree with
    the reference implementation (its sdpa attention path, eager losses)."""
    sys.path.insert(0, REF)
    try:
        from transformers import LlamaConfig

        from speculators.models.eagle3.core import Eagle3DraftModel as RefModel
    except Exception as err:  # noqa: BLE001
        pytest.skip(f"reference import failed: {err}")
    finally:
        sys.path.remove(REF)
    t2d, d2t = tiny_vocab_maps
    mine = make_tiny_eagle3(tiny_verifier_dir, tiny_vocab_maps, num_layers=2)
    rc = LlamaConfig(**{k: v for k, v in TINY_VERIFIER.items() if k not in ("model_type", "architectures")})
    rc.num_hidden_layers = 2
    ref = RefModel.from_training_args(
        rc, t2d=t2d, d2t=d2t, draft_attn_impl="sdpa", draft_vocab_size=32, norm_before_residual=True, ttt_steps=3,
        verifier_name_or_path=tiny_verifier_dir, target_layer_ids=[1, 2, 3], norm_before_fc=True, norm_output=True,
    )
    assert not ref.load_state_dict(mine.state_dict(), strict=False).unexpected_keys
    batch = make_tiny_batch()
    mk, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn=loss_fn, ttt_steps=3, ttt_step_loss_decay=0.8)
    rk, _ = RefModel.get_trainer_kwargs(loss_fn=loss_fn, loss_implementation="eager", ttt_steps=3, ttt_step_loss_decay=0.8)
    _, l1, m1 = mine(**batch, **mk)
    _, l2, m2 = ref(**{k: v.clone() for k, v in batch.items()}, **rk)
    assert torch.allclose(l1, l2, atol=1e-5)
    assert set(m1) == set(m2)
    for k in m1:
        assert abs(float(m1[k]) - float(m2[k])) < 1e-4, k
    l1.backward(); l2.backward()
    assert torch.allclose(mine.fc.weight.grad, ref.fc.weight.grad, atol=1e-5)
    nq = ref.layers[0].self_attn.q_proj.weight.shape[0]
    assert torch.allclose(mine.layers[0].self_attn.qkv_proj.weight.grad[:nq], ref.layers[0].self_attn.q_proj.weight.grad, atol=1e-6)


def test_component_table_and_partial_rotary_oracle():
    from speculators_b200 import ops
    from speculators_b200.models.base_components import model_classes, override_components
    from speculators_b200.models.eagle3.core import Eagle3FirstLayer
    from speculators_b200.models.eagle3.rotary_partial import install_partial_neox_rotary, partial_neox_apply_rotary_pos_emb

    comps = override_components("llama", first_layer_class=Eagle3FirstLayer)
    assert comps.first_layer_class is Eagle3FirstLayer and comps.decoder_layer_class is model_classes["llama"].decoder_layer_class
    assert {"llama", "qwen3", "qwen3_next", "qwen3_5_moe_text"} <= set(model_classes)
    with pytest.raises(KeyError):
        override_components("gpt2")
    install_partial_neox_rotary()
    # the package's rotary op in partial mode equals the reference-signature function
    torch.manual_seed(0)
    T, heads, hd, rot = 9, 3, 16, 8
    x = torch.randn(T, heads * hd)
    pos = torch.arange(T)
    ang = torch.outer(torch.arange(32, dtype=torch.float32), 1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot)))
    cos_t, sin_t = ang.cos(), ang.sin()
    ours = ops.rope_(x.clone(), pos, cos_t, sin_t, heads, hd, rot).view(T, heads, hd)
    cos_full, sin_full = torch.cat([cos_t, cos_t], -1)[pos], torch.cat([sin_t, sin_t], -1)[pos]
    q = x.view(T, heads, hd).transpose(0, 1).unsqueeze(0)  # [1, heads, T, hd]
    ref, _ = partial_neox_apply_rotary_pos_emb(q, q, cos_full.unsqueeze(0), sin_full.unsqueeze(0))
    torch.testing.assert_close(ours, ref[0].transpose(0, 1), atol=1e-5, rtol=1e-5)


def test_block_mask_interop_helpers():
    """Extending a flex-attention block mask by one pass adds the diagonal key block per
    query block, twice in a row, and the dense conversion equals the element mask."""
    from torch.nn.attention.flex_attention import create_block_mask, create_mask

    from speculators_b200.models.eagle3.attention import (
        block_mask_to_dense_attention_mask, create_combined_mask_mod, extend_mask_for_draft_tokens,
    )

    T, B = 16, 4
    doc = torch.tensor([0] * 6 + [1] * 7 + [-1] * 3)
    mod = create_combined_mask_mod(doc, T)
    bm = create_block_mask(mod, None, None, T, T, device="cpu", BLOCK_SIZE=B)
    base = bm.to_dense()[0, 0].bool()
    grown = bm
    for step in (1, 2):
        grown = extend_mask_for_draft_tokens(grown)
        assert grown.seq_lengths == (T, T * (step + 1))
        blocks = grown.to_dense()[0, 0].bool()
        assert blocks.shape == (T // B, (T // B) * (step + 1))
        assert torch.equal(blocks[:, : T // B], base)
        for p in range(1, step + 1):
            assert torch.equal(blocks[:, p * (T // B): (p + 1) * (T // B)], torch.eye(T // B, dtype=torch.bool))
        dense = block_mask_to_dense_attention_mask(grown, torch.device("cpu"), torch.bool)
        want = create_mask(mod, None, None, T, T * (step + 1), device="cpu")
        assert torch.equal(dense, want)
    assert grown.mask_mod is bm.mask_mod
