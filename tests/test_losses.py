import math

import pytest
import torch

from speculators_b200 import losses
from speculators_b200.losses import eager


def _pair(T=7, V=19, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(1, T, V, generator=g), torch.randn(1, T, V, generator=g)


def test_eager_matches_textbook_definitions():
    x, t = _pair()
    q, p = x.softmax(-1), t.softmax(-1)
    assert torch.allclose(eager.kl_div_loss(x, t), (p * (p.log() - q.log())).sum(-1), atol=1e-5)
    assert torch.allclose(eager.reverse_kl_div_loss(x, t), (q * (q.log() - p.log())).sum(-1), atol=1e-5)
    m = 0.5 * (p + q)
    jsd = 0.5 * (p * (p.log() - m.log())).sum(-1) + 0.5 * (q * (q.log() - m.log())).sum(-1)
    assert torch.allclose(eager.js_div_loss(x, t), jsd, atol=1e-5)
    assert (eager.js_div_loss(x, t) <= math.log(2) + 1e-6).all()
    ce = -q.log().gather(-1, t.argmax(-1, keepdim=True)).squeeze(-1)
    assert torch.allclose(eager.ce_loss(x, t), ce, atol=1e-5)
    tv = 1 - torch.minimum(p, q).sum(-1)
    assert torch.allclose(eager.tv_loss(x, t), tv, atol=1e-6)
    assert torch.allclose(eager.neg_log_acceptance_loss(x, t), -(1 - tv).clamp_min(1e-5).log(), atol=1e-5)
    lam = torch.exp(-3.0 * (1 - tv))
    assert torch.allclose(eager.lk_hybrid_loss(x, t), lam * eager.kl_div_loss(x, t) + (1 - lam) * tv, atol=1e-5)


@pytest.mark.parametrize("name", ["kl_div", "rkl", "jsd", "ce", "tv", "nla", "lk_hybrid"])
def test_fused_falls_back_to_dense_on_cpu(name):
    x, t = _pair(seed=3)
    f = losses.resolve_loss_config(name, "fused")[name][0]
    e = losses.resolve_loss_config(name, "eager")[name][0]
    assert torch.allclose(f(x, t), e(x, t), atol=1e-5)


def test_resolve_loss_config_forms():
    cfg = losses.resolve_loss_config('{"ce": 0.1, "tv": 0.9}')
    assert list(cfg) == ["ce", "tv"] and cfg["tv"][1] == 0.9
    for bad in ("nope", "[1]", "{}", '{"nope": 1}', '{"ce": "x"}'):
        with pytest.raises(ValueError):
            losses.resolve_loss_config(bad)
    with pytest.raises(ValueError):
        losses.resolve_loss_config("ce", "triton")


def test_decays():
    pos = torch.tensor([[0, 1, 2, 3, 0, 1, 2, 3]])
    w = losses.dflash_loss_decay(pos, gamma=2.0)
    assert torch.allclose(w[0, :4], torch.tensor([0.0, 1.0, math.exp(-0.5), math.exp(-1.0)]))
    w2 = losses.dflash_loss_decay(pos, gamma=2.0, sample_from_anchor=True)
    assert torch.allclose(w2[0, :3], torch.tensor([1.0, math.exp(-0.5), math.exp(-1.0)]))
    assert torch.allclose(losses.exp_loss_decay(pos.float(), 0.5)[0, :3], torch.tensor([1.0, 0.5, 0.25]))


def test_dpace_weights_by_hand():
    ce = torch.tensor([[0.0, math.log(2.0), math.log(4.0), 0.0]])  # q = 1, .5, .25, 1
    mask = torch.tensor([[1, 1, 0, 1]])
    w = losses.dpace_loss_decay(None, mask, block_size=4, dpace_alpha=0.0, elementwise_loss=ce)
    # prefixes (masked slot counts as 1): 1, .5, .5, .5 ; masked prefix*mask: 1, .5, 0, .5
    assert torch.allclose(w, torch.tensor([[2.0, 1.0, 0.0, 0.5]]))
    with pytest.raises(ValueError):
        losses.dpace_loss_decay(None, mask[:, :3], block_size=4, dpace_alpha=0.0, elementwise_loss=ce[:, :3])


def test_masked_reduction_and_compound():
    x, t = _pair(T=6)
    mask = torch.tensor([[1, 1, 0, 0, 1, 0]])
    pos = torch.zeros(1, 6)
    val = losses.loss_function(x, t, mask, pos, loss_fn=eager.kl_div_loss)
    ref = (eager.kl_div_loss(x, t) * mask).sum() / (3 + 1e-5)
    assert torch.allclose(val, ref)
    total, parts = losses.compound_loss(x, t, mask, pos, losses.resolve_loss_config('{"ce": 0.25, "tv": 0.75}', "eager"))
    assert set(parts) == {"ce_loss", "tv_loss"}
    assert torch.allclose(total, 0.25 * parts["ce_loss"] + 0.75 * parts["tv_loss"])
    _, parts1 = losses.compound_loss(x, t, mask, pos, losses.resolve_loss_config("kl_div", "eager"))
    assert parts1 == {}


def test_skipped_rows_get_no_gradient_whatever_the_upstream_weight():
    """Rows switched off (``keep`` / ``active`` false) cost 0 and receive a zero gradient even when
    the upstream gradient of those rows is not zero (the MTP loss divides a plain sum by the count)."""
    import torch

    from speculators_b200 import ops

    torch.manual_seed(0)
    T, V = 12, 50
    keep = torch.tensor([True, False] * (T // 2))
    labels = torch.randint(0, V, (T,))
    x = torch.randn(T, V, requires_grad=True)
    loss = ops.token_cross_entropy(x, labels, keep)
    (loss.sum() / keep.sum()).backward()
    assert (loss[~keep] == 0).all() and (x.grad[~keep] == 0).all() and (x.grad[keep].abs().sum(-1) > 0).all()

    y = torch.randn(T, V, requires_grad=True)
    t = torch.randn(T, V)
    for op in ("kl_div", "ce", "tv"):
        y.grad = None
        row, _, _ = ops.fused_row_loss(op, y, t, active=keep)
        row.sum().backward()
        assert (row[~keep] == 0).all() and (y.grad[~keep] == 0).all()
