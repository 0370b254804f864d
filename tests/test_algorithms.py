"""P-EAGLE, DFlash, DSpark and MTP: mask specs against their definitions, forward /
backward sanity, and numerical parity with the reference where it is installed."""

import os
import sys

import pytest
import torch

import speculators_b200 as sb
from speculators_b200.layer_config import TransformerLayerConfig
from speculators_b200.models.dflash import DFlashDraftModel
from speculators_b200.models.dflash.attention import anchor_block_attn_spec, dense_anchor_block_mask
from speculators_b200.models.dflash.utils import get_base_indices_for_anchored_blocks, select_anchors
from speculators_b200.models.dspark import DSparkDraftModel
from speculators_b200.models.mtp import compute_step_weights
from speculators_b200.models.peagle import PEagleDraftModel
from speculators_b200.models.peagle.attention import dense_peagle_mask, peagle_attn_spec
from speculators_b200.models.peagle.data import generate_cod_sample_indices

from conftest import ROOT, TINY_VERIFIER, make_tiny_batch

REF = os.path.join(ROOT, "baseline", "_ref")
HAVE_REF = os.path.isdir(os.path.join(REF, "speculators"))
QWEN = dict(TINY_VERIFIER, model_type="qwen3", architectures=["Qwen3ForCausalLM"])


def _import_ref(path):
    sys.path.insert(0, REF)
    try:
        import importlib

        return importlib.import_module(path)
    except Exception as err:  # noqa: BLE001
        pytest.skip(f"reference import failed: {err}")
    finally:
        sys.path.remove(REF)


# ------------------------------------------------------------------ P-EAGLE
def test_cod_sampling_shapes_and_chains():
    torch.manual_seed(0)
    T = 64
    mask = (torch.rand(1, T) > 0.3).float()
    a, d = generate_cod_sample_indices(T, mask, num_depths=4, down_sample_ratio=0.7, down_sample_ratio_min=0.2)
    assert (d[:T] == 0).all() and torch.equal(a[:T], torch.arange(T))
    assert (a >= -1).all() and (a + d < T).all()  # a valid position 0 sampled at depth 1 has anchor -1, as in the reference
    pairs = set(zip(a.tolist(), d.tolist()))
    for ai, di in pairs:  # every rollout member has its predecessor
        assert di == 0 or ai < 0 or (ai, di - 1) in pairs
    deep = d >= 1
    assert (mask[0, (a + d)[deep]] == 1).all()


@pytest.mark.parametrize("window", [None, 6])
def test_peagle_spec_equals_mask_definition(window):
    torch.manual_seed(1)
    T = 48
    doc = torch.cat([torch.zeros(20), torch.ones(22), torch.full((6,), -1)]).long()
    mask = ((torch.rand(1, T) > 0.2) & (doc != -1)).float()
    a, d = generate_cod_sample_indices(T, mask, num_depths=4)
    spec = peagle_attn_spec(a, d, doc, 4, window)
    dense = dense_peagle_mask(a, d, doc, window)
    assert torch.equal(spec.dense(T, a.numel() - T), dense)


def _peagle(tiny_verifier_dir, maps, layers=1):
    t2d, d2t = maps
    torch.manual_seed(0)
    return PEagleDraftModel.from_training_args(
        TransformerLayerConfig(**dict(TINY_VERIFIER, num_hidden_layers=layers)), t2d=t2d, d2t=d2t, draft_vocab_size=32,
        norm_before_residual=True, verifier_name_or_path=tiny_verifier_dir, target_layer_ids=[1, 2, 3], mask_token_id=5, num_depths=4,
    )


def test_peagle_forward_backward(tiny_verifier_dir, tiny_vocab_maps):
    model = _peagle(tiny_verifier_dir, tiny_vocab_maps, layers=2)
    kw, _ = PEagleDraftModel.get_trainer_kwargs(loss_fn="kl_div", num_depths=4)
    _, loss, metrics = model(**make_tiny_batch(), **kw)
    loss.backward()
    assert torch.isfinite(loss) and model.mask_hidden.grad is not None and model.embed_tokens.weight.grad is not None
    assert {"position_0_acc_sum", "position_3_acc_total", "full_acc_sum"} <= set(metrics)


def test_cod_fixed_shape_sampler_and_inert_padding(tiny_verifier_dir, tiny_vocab_maps):
    from speculators_b200.models.peagle.data import cod_capacities, generate_cod_sample_indices_fixed

    torch.manual_seed(0)
    T, D = 64, 4
    mask = (torch.rand(1, T) > 0.3).float()
    caps = cod_capacities(T, D, 0.7, 0.2)
    assert caps == [64, int(63 * 0.7), int(62 * 0.49), int(61 * 0.343)]
    a, d, ok = generate_cod_sample_indices_fixed(T, mask, num_depths=D)
    assert a.shape == d.shape == ok.shape == (sum(caps),) and ok[:T].all() and torch.equal(a[:T], torch.arange(T))
    # the shape depends on the arguments only, not on the mask
    assert generate_cod_sample_indices_fixed(T, torch.zeros(1, T), num_depths=D)[0].shape == a.shape
    assert not generate_cod_sample_indices_fixed(T, torch.zeros(1, T), num_depths=D)[2][T:].any()
    va, vd = a[ok], d[ok]
    pairs = set(zip(va.tolist(), vd.tolist()))
    for ai, di in pairs:  # every rollout member has its predecessor, and stands on a supervised token
        assert di == 0 or ai < 0 or (ai, di - 1) in pairs
    deep = vd >= 1
    assert (mask[0, (va + vd)[deep]] == 1).all()
    # same law as the variable-shape sampler: depth 1 keeps int((n_valid - 1) * 0.7) rows (the pool is large enough)
    n_valid = int(mask.sum())
    assert int((ok & (d == 1)).sum()) == int((n_valid - 1) * 0.7)
    ref_a, ref_d = generate_cod_sample_indices(T, mask, num_depths=D)
    assert int((ref_d == 1).sum()) == int((n_valid - 1) * 0.7)
    # max_anchors caps the seeds
    a2, d2, ok2 = generate_cod_sample_indices_fixed(T, mask, num_depths=D, max_anchors=10)
    assert a2.numel() == sum(cod_capacities(T, D, 0.7, 0.2, 10)) and int((ok2 & (d2 == 1)).sum()) == int(9 * 0.7)

    # padding rows are inert: a variable-shape sample and the same sample padded to the
    # fixed shape (in depth-major order) give the same loss and metrics
    model = _peagle(tiny_verifier_dir, tiny_vocab_maps, layers=2)
    batch = make_tiny_batch()
    T = batch["input_ids"].shape[1]
    kw, _ = PEagleDraftModel.get_trainer_kwargs(loss_fn="kl_div", num_depths=D)
    torch.manual_seed(3)
    va, vd = generate_cod_sample_indices(T, batch["loss_mask"], num_depths=D)
    caps = cod_capacities(T, D, 0.7, 0.2)
    pa, pd, pv = [], [], []
    for depth_i, cap in enumerate(caps):
        rows = va[vd == depth_i]
        pad = cap - rows.numel()
        pa.append(torch.cat([rows, torch.zeros(pad, dtype=torch.long)]))
        pd.append(torch.full((cap,), depth_i, dtype=torch.long))
        pv.append(torch.cat([torch.ones(rows.numel(), dtype=torch.bool), torch.zeros(pad, dtype=torch.bool)]))
    _, loss_var, m_var = model(**batch, **kw, cod_sample=(va, vd))
    _, loss_fix, m_fix = model(**batch, **kw, cod_sample=(torch.cat(pa), torch.cat(pd), torch.cat(pv)))
    torch.testing.assert_close(loss_fix, loss_var, rtol=1e-5, atol=1e-6)
    for key in m_var:
        torch.testing.assert_close(m_fix[key].float(), m_var[key].float(), rtol=1e-5, atol=1e-6)
    assert kw["fixed_shape"] is False  # opt-in: cod_fixed_shape=True or SB200_PEAGLE_FIXED_SHAPE=1
    assert not model.graph_safe_with(kw) and model.graph_safe_with({**kw, "fixed_shape": True})
    kw_fixed, _ = PEagleDraftModel.get_trainer_kwargs(loss_fn="kl_div", num_depths=D, cod_fixed_shape=True)
    _, loss_drawn, _ = model(**batch, **kw_fixed)
    loss_drawn.backward()
    assert torch.isfinite(loss_drawn) and model.mask_hidden.grad is not None


@pytest.mark.skipif(not HAVE_REF, reason="reference not installed")
def test_peagle_parity_with_reference(tiny_verifier_dir, tiny_vocab_maps):
    ref_core = _import_ref("speculators.models.peagle.core")
    from transformers import LlamaConfig

    mine = _peagle(tiny_verifier_dir, tiny_vocab_maps, layers=2)
    t2d, d2t = tiny_vocab_maps
    rc = LlamaConfig(**{k: v for k, v in TINY_VERIFIER.items() if k not in ("model_type", "architectures")})
    rc.num_hidden_layers = 2
    ref = ref_core.PEagleDraftModel.from_training_args(
        rc, t2d=t2d, d2t=d2t, draft_attn_impl="sdpa", draft_vocab_size=32, norm_before_residual=True,
        verifier_name_or_path=tiny_verifier_dir, target_layer_ids=[1, 2, 3], mask_token_id=5, num_depths=4,
    )
    ref.load_state_dict(mine.state_dict(), strict=False)
    batch = make_tiny_batch()
    kw, _ = PEagleDraftModel.get_trainer_kwargs(loss_fn="kl_div", num_depths=4)
    rkw, _ = ref_core.PEagleDraftModel.get_trainer_kwargs(loss_fn="kl_div", loss_implementation="eager", num_depths=4)
    torch.manual_seed(7)
    _, l1, m1 = mine(**batch, **kw)
    torch.manual_seed(7)
    _, l2, m2 = ref(**{k: v.clone() for k, v in batch.items()}, **rkw)
    assert torch.allclose(l1, l2, atol=1e-5), (float(l1), float(l2))
    for k in m2:
        assert abs(float(m1[k]) - float(m2[k])) < 1e-4, k


# ------------------------------------------------------------------ DFlash / DSpark
def test_select_anchors_contract():
    torch.manual_seed(0)
    mask = torch.zeros(1, 40)
    mask[0, [3, 7, 9, 20, 36, 38]] = 1
    anchors, valid = select_anchors(mask, 8, block_size=4)
    assert anchors.shape == (8,) and valid.sum() == 4  # 36 and 38 fall in the excluded tail
    kept = anchors[valid]
    assert torch.equal(kept, kept.sort().values) and set(kept.tolist()) == {3, 7, 9, 20}
    assert (anchors[~valid] == 0).all()
    anchors2, valid2 = select_anchors(mask, 2, block_size=4)
    assert valid2.all() and set(anchors2.tolist()) <= {3, 7, 9, 20}
    assert get_base_indices_for_anchored_blocks(torch.tensor([2, 9]), 3).tolist() == [2, 3, 4, 9, 10, 11]
    with pytest.raises(ValueError):
        select_anchors(mask[0], 2, 4)


@pytest.mark.parametrize("window,non_causal", [(None, False), (5, False), (5, True)])
def test_anchor_block_spec_equals_mask_definition(window, non_causal):
    doc = torch.cat([torch.zeros(14), torch.ones(15), torch.full((3,), -1)]).long()
    anchors = torch.tensor([2, 9, 16, 25, 0])
    spec = anchor_block_attn_spec(doc, anchors, 4, window, non_causal)
    dense = dense_anchor_block_mask(doc, 32, anchors, 4, window, non_causal)
    assert torch.equal(spec.dense(32, 20), dense)


def _dflash_cfg(layers=2):
    return TransformerLayerConfig(**dict(QWEN, num_hidden_layers=layers, sliding_window=6, layer_types=["full_attention"] + ["sliding_attention"] * (layers - 1)))


def _dflash_batch():
    b = make_tiny_batch()
    b["position_ids"] = b["position_ids"] - 1
    return b


@pytest.mark.parametrize("cls,extra", [(DFlashDraftModel, {}), (DSparkDraftModel, {"markov_rank": 8, "markov_head_type": "gated"}), (DSparkDraftModel, {"markov_rank": 8, "markov_head_type": "rnn"})])
def test_dflash_family_forward_backward(cls, extra, tiny_verifier_dir, tiny_vocab_maps):
    t2d, d2t = tiny_vocab_maps
    torch.manual_seed(0)
    model = cls.from_training_args(_dflash_cfg(), t2d=t2d, d2t=d2t, draft_vocab_size=32, block_size=4, verifier_name_or_path=tiny_verifier_dir,
                                   target_layer_ids=[1, 2, 3], mask_token_id=5, **extra)
    kw, _ = cls.get_trainer_kwargs(loss_fn="ce", max_anchors=6, per_position_loss_weight="dpace")
    _, loss, metrics = model(**_dflash_batch(), **kw)
    loss.backward()
    assert torch.isfinite(loss)
    assert all(torch.isfinite(p.grad).all() for p in model.parameters() if p.requires_grad and p.grad is not None)
    assert "full_acc_sum" in metrics and ("eal_sum" in metrics or "accept_len_sum" in metrics)
    sd = model.state_dict()
    assert "layers.0.self_attn.q_proj.weight" in sd and "layers.0.self_attn.q_norm.weight" in sd and "hidden_norm.weight" in sd
    if cls is DSparkDraftModel:
        assert "markov_head.markov_w1.weight" in sd and "confidence_head.proj.weight" in sd


@pytest.mark.skipif(not HAVE_REF, reason="reference not installed")
@pytest.mark.parametrize("algo", ["dflash", "dspark"])
def test_dflash_family_parity_with_reference(algo, tiny_verifier_dir, tiny_vocab_maps, monkeypatch):
    ref_core = _import_ref(f"speculators.models.{algo}.core")
    ref_dflash_core = _import_ref("speculators.models.dflash.core")
    from transformers.models.qwen3.configuration_qwen3 import Qwen3Config

    import speculators_b200.models.dflash.core as my_core

    fixed = (torch.tensor([2, 9, 15, 24, 0, 0]), torch.tensor([True, True, True, True, False, False]))
    monkeypatch.setattr(my_core, "select_anchors", lambda *a, **k: fixed)
    monkeypatch.setattr(ref_dflash_core, "select_anchors", lambda *a, **k: fixed)
    t2d, d2t = tiny_vocab_maps
    MyCls = DFlashDraftModel if algo == "dflash" else DSparkDraftModel
    RefCls = getattr(ref_core, "DFlashDraftModel" if algo == "dflash" else "DSparkDraftModel")
    extra = {} if algo == "dflash" else {"markov_rank": 8}
    torch.manual_seed(0)
    mine = MyCls.from_training_args(_dflash_cfg(), t2d=t2d, d2t=d2t, draft_vocab_size=32, block_size=4,
                                    verifier_name_or_path=tiny_verifier_dir, target_layer_ids=[1, 2, 3], mask_token_id=5, **extra)
    rc = Qwen3Config(**{k: v for k, v in QWEN.items() if k not in ("model_type", "architectures")})
    rc.num_hidden_layers = 2
    rc.sliding_window = 6
    rc.layer_types = ["full_attention", "sliding_attention"]
    ref = RefCls.from_training_args(rc, t2d=t2d, d2t=d2t, draft_attn_impl="sdpa", draft_vocab_size=32, block_size=4,
                                    verifier_name_or_path=tiny_verifier_dir, target_layer_ids=[1, 2, 3], mask_token_id=5, **extra)
    res = ref.load_state_dict(mine.state_dict(), strict=False)
    assert not res.unexpected_keys, res.unexpected_keys
    batch = _dflash_batch()
    kw, _ = MyCls.get_trainer_kwargs(loss_fn="ce", max_anchors=6, per_position_loss_weight="dpace")
    rkw, _ = RefCls.get_trainer_kwargs(loss_fn="ce", loss_implementation="eager", max_anchors=6, per_position_loss_weight="dpace")
    _, l1, m1 = mine(**batch, **kw)
    _, l2, m2 = ref(**{k: v.clone() for k, v in batch.items()}, **rkw)
    assert torch.allclose(l1, l2, atol=1e-5), (float(l1), float(l2))
    assert set(m1) == set(m2)
    for k in m2:
        assert abs(float(m1[k]) - float(m2[k])) < 1e-4, k
    l1.backward(); l2.backward()
    assert torch.allclose(mine.fc.weight.grad, ref.fc.weight.grad, atol=1e-5)


# ------------------------------------------------------------------ MTP
def test_mtp_step_weights():
    w = compute_step_weights(0.6, 3)
    assert abs(sum(w) - 1) < 1e-9 and abs(w[1] / w[0] - 0.6) < 1e-9
