"""Numerics of every sm_100a kernel against a plain PyTorch fp32 formulation."""

import pytest
import torch

from speculators_b200 import ops
from speculators_b200.ops import _row_loss_ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol=2e-2):
    torch.testing.assert_close(a.float(), b.float(), atol=atol, rtol=rtol)


def test_extension_is_loaded_from_tree():
    nat = ops.native()
    assert hasattr(nat, "rmsnorm_fwd")
    assert ops._ext.loaded_library_path().endswith("_sb200.so")


@pytest.mark.parametrize("rows,H", [(1, 64), (127, 4096), (300, 8192), (65, 12288), (129, 256), (70001, 128), (5000, 64), (333, 264)])
def test_rmsnorm_fwd_bwd(rows, H):
    torch.manual_seed(0)
    x = torch.randn(rows, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.rand(H, device=DEV) + 0.5).to(torch.bfloat16).requires_grad_()
    dy = torch.randn(rows, H, device=DEV, dtype=torch.bfloat16)
    y = ops.rms_norm(x, w, 1e-5)
    y.backward(dy)
    xf = x.detach().float().requires_grad_(); wf = w.detach().float().requires_grad_()
    yf = wf * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5))
    yf.backward(dy.float())
    _close(y, yf, atol=3e-2)
    _close(x.grad, xf.grad, atol=3e-2)
    _close(w.grad, wf.grad, atol=0.05 * float(wf.grad.abs().max()) + 0.05)


def test_eagle3_input_concat():
    torch.manual_seed(0)
    T, H = 200, 512
    e = torch.randn(T, H, device=DEV, dtype=torch.bfloat16)
    h = torch.randn(T, H, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    we = (torch.rand(H, device=DEV) + 0.5).to(torch.bfloat16).requires_grad_()
    wh = (torch.rand(H, device=DEV) + 0.5).to(torch.bfloat16).requires_grad_()
    out = ops.eagle3_input_concat(e, h, we, wh, 1e-5)
    d = torch.randn_like(out)
    out.backward(d)
    ref = torch.cat([ops._rms_norm_ref(e.float(), we.float(), 1e-5), ops._rms_norm_ref(h.float(), wh.float(), 1e-5)], -1)
    _close(out, ref, atol=3e-2)
    hf = h.detach().float().requires_grad_()
    ops._rms_norm_ref(hf, wh.detach().float(), 1e-5).backward(d[:, H:].float())
    _close(h.grad, hf.grad, atol=3e-2)
    assert we.grad is not None and torch.isfinite(we.grad).all()


@pytest.mark.parametrize("rows,I", [(1, 64), (333, 14336), (130, 688 - 688 % 16)])
def test_swiglu(rows, I):
    torch.manual_seed(0)
    gu = torch.randn(rows, 2 * I, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    d = torch.randn(rows, I, device=DEV, dtype=torch.bfloat16)
    out = ops.swiglu(gu)
    out.backward(d)
    gf = gu.detach().float().requires_grad_()
    g, u = gf.chunk(2, -1)
    ref = torch.nn.functional.silu(g) * u
    ref.backward(d.float())
    _close(out, ref, atol=3e-2)
    _close(gu.grad, gf.grad, atol=5e-2)


@pytest.mark.parametrize("rot", [64, 32])
def test_rope_matches_reference_and_inverts(rot):
    torch.manual_seed(0)
    T, heads, hd = 77, 6, 64
    x = torch.randn(T, heads * hd + 128, device=DEV, dtype=torch.bfloat16)
    pos = torch.randint(0, 500, (T,), device=DEV)
    ang = torch.outer(torch.arange(512, dtype=torch.float64), 1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot)))
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    ref = ops._rope_ref(x.float(), pos, cos, sin, heads, hd, rot, 1.0)
    y = x.clone()
    ops.native().rope_(y, pos, cos, sin, heads, hd, rot, 1.0)
    _close(y, ref, atol=2e-2)
    assert torch.equal(y[:, heads * hd:], x[:, heads * hd:])
    ops.native().rope_(y, pos, cos, sin, heads, hd, rot, -1.0)
    _close(y, x, atol=3e-2)


@pytest.mark.parametrize("hd,rot", [(128, 128), (64, 64), (64, 24)])
def test_rope_split_matches_separate_ops(hd, rot):
    """The fused rotate+split (vectorised kernel when rot/2 % 8 == 0, one concatenated
    gradient) against the fp32 rotation followed by plain slicing, values and grads."""
    torch.manual_seed(1)
    T, nh, nkv = 50, 4, 2
    nq, nk = nh * hd, nkv * hd
    base = torch.randn(T, nq + 2 * nk, device=DEV)
    pos = torch.randint(0, 300, (T,), device=DEV)
    ang = torch.outer(torch.arange(512, dtype=torch.float64), 1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot)))
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    wq, wk, wv = (torch.randn(T, n, device=DEV) for n in (nq, nk, nk))

    x = base.to(torch.bfloat16).requires_grad_()
    q, k, v = ops.rope_split(x * 1.0, pos, cos, sin, nh + nkv, hd, rot, nq, nk)
    ((q.float() * wq).sum() + (k.float() * wk).sum() + 2 * (k.float() * wk).sum() + (v.float() * wv).sum()).backward()

    xr = base.to(torch.bfloat16).float().requires_grad_()
    yr = ops._rope_ref(xr, pos, cos, sin, nh + nkv, hd, rot, 1.0)
    qr, kr, vr = yr[:, :nq], yr[:, nq:nq + nk], yr[:, nq + nk:]
    ((qr * wq).sum() + 3 * (kr * wk).sum() + (vr * wv).sum()).backward()
    _close(q, qr, atol=3e-2)
    _close(k, kr, atol=3e-2)
    assert torch.equal(v.float(), vr)
    _close(x.grad, xr.grad, atol=5e-2, rtol=2e-2)


@pytest.mark.parametrize("op", ["kl_div", "rkl", "jsd", "ce", "tv"])
@pytest.mark.parametrize("T,V,shift", [(33, 1000, 0), (64, 32000, 2), (5, 151936, 1), (17, 1003, 0)])
def test_row_loss_fwd_bwd(op, T, V, shift):
    torch.manual_seed(0)
    scale = 3.0
    x = (torch.randn(T, V, device=DEV) * scale).to(torch.bfloat16).requires_grad_()
    t = (torch.randn(T, V, device=DEV) * scale).to(torch.bfloat16)
    rows = T - shift
    w = torch.rand(rows, device=DEV)
    w[::3] = 0.0  # exact-zero upstream rows must produce exact-zero gradients
    loss, am_d, am_t = ops.fused_row_loss(op, x, t, shift=shift, rows=rows)
    (loss * w).sum().backward()
    xf = x.detach().float().requires_grad_()
    ref = _row_loss_ref(op, xf[:rows], t.float()[shift: shift + rows])
    (ref * w).sum().backward()
    _close(loss, ref, atol=2e-3, rtol=2e-3)
    assert torch.equal(am_d, x.detach()[:rows].float().argmax(-1))
    assert torch.equal(am_t, t[shift: shift + rows].float().argmax(-1))
    assert x.grad.shape == x.shape
    _close(x.grad, xf.grad, atol=2e-3, rtol=5e-2)
    assert (x.grad[:rows][::3] == 0).all() and (x.grad[rows:] == 0).all()


def test_row_loss_saturated_rows_and_active_mask():
    x = torch.zeros(4, 512, device=DEV, dtype=torch.bfloat16)
    t = torch.zeros(4, 512, device=DEV, dtype=torch.bfloat16)
    x[0, 3] = 30.0; t[0, 3] = 30.0
    x[1, 5] = 30.0; t[1, 9] = 30.0
    x[2, 7] = -30.0
    active = torch.tensor([True, True, True, False], device=DEV)
    for op in ("kl_div", "rkl", "jsd", "ce", "tv"):
        loss, am_d, am_t = ops.fused_row_loss(op, x, t, active=active)
        ref = _row_loss_ref(op, x.float()[:3], t.float()[:3])
        assert torch.isfinite(loss).all()
        _close(loss[:3], ref, atol=1e-3, rtol=2e-3)
        assert loss[3] == 0 and am_d[3] == -1 and am_t[3] == -2


def test_sum_of_squares_and_adamw_match_torch():
    torch.manual_seed(0)
    n = 1_000_003
    g16 = torch.randn(n, device=DEV).to(torch.bfloat16)
    out = torch.zeros(1, device=DEV)
    ops.sum_of_squares(g16, out)
    _close(out[0], g16.float().pow(2).sum(), atol=1.0, rtol=1e-4)
    ops.sum_of_squares(g16, out, accumulate=True)
    _close(out[0], 2 * g16.float().pow(2).sum(), atol=2.0, rtol=1e-4)

    p = torch.randn(n, device=DEV)
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=1e-2, weight_decay=0.01)
    m = torch.zeros(n, device=DEV); v = torch.zeros(n, device=DEV)
    w16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    hyper = torch.zeros(ops.HYPER_LEN, device=DEV)
    for step in range(1, 4):
        g = torch.randn(n, device=DEV).to(torch.bfloat16)
        ns = torch.zeros(1, device=DEV)
        ops.sum_of_squares(g, ns)
        hyper[:9] = torch.tensor([1e-2, 0.9, 0.999, 1e-8, 0.01, 1 - 0.9**step, 1 - 0.999**step, 1.0, 1.0])
        ops.adamw_step_(p, m, v, g, w16, hyper, ns)
        ref.grad = g.float()
        torch.nn.utils.clip_grad_norm_([ref], 1.0)
        opt.step()
    _close(p, ref.detach(), atol=1e-5, rtol=1e-4)
    _close(w16, p, atol=2e-2)


@pytest.mark.parametrize("T,V", [(33, 1000), (20, 32000), (7, 1003)])
def test_token_cross_entropy_fwd_bwd(T, V):
    """Cross-entropy against integer labels (the MTP loss), with rows switched off by ``keep``."""
    torch.manual_seed(0)
    x = (torch.randn(T, V, device=DEV) * 3.0).to(torch.bfloat16).requires_grad_()
    labels = torch.randint(0, V, (T,), device=DEV)
    keep = torch.rand(T, device=DEV) > 0.3
    w = torch.rand(T, device=DEV)
    loss = ops.token_cross_entropy(x, labels, keep)
    (loss * w).sum().backward()
    xf = x.detach().float().requires_grad_()
    ref = torch.nn.functional.cross_entropy(xf, labels, reduction="none")
    ref = torch.where(keep, ref, torch.zeros_like(ref))
    (ref * w).sum().backward()
    _close(loss, ref, atol=2e-3, rtol=2e-3)
    assert (loss[~keep] == 0).all()
    _close(x.grad, xf.grad, atol=2e-3, rtol=5e-2)
    assert (x.grad[~keep] == 0).all()


@pytest.mark.parametrize("op", ["kl_div", "ce"])
@pytest.mark.parametrize("T,H,V,shift", [(300, 256, 1024, 0), (520, 192, 1000, 2), (2048, 512, 32000, 1), (257, 136, 264, 0)])
def test_lm_head_fused_with_row_loss(op, T, H, V, shift, monkeypatch):
    """``lm_head_loss_raw`` (head GEMM whose epilogue reduces the tiles for the loss) against the
    head GEMM followed by the row-loss kernel, and against the fp32 formula: row losses, both
    argmaxes, the gradient of the hidden states; inactive rows and zero upstream rows included."""
    monkeypatch.setenv("SB200_FUSED_HEAD", "1")
    torch.manual_seed(0)
    hidden = (torch.randn(T, H, device=DEV) * 0.7).to(torch.bfloat16).requires_grad_()
    weight = (torch.randn(V, H, device=DEV) * 0.2).to(torch.bfloat16)
    targets = (torch.randn(T, V, device=DEV) * 3.0).to(torch.bfloat16)
    rows = T - shift
    active = torch.rand(rows, device=DEV) > 0.2
    up = torch.rand(rows, device=DEV)
    up[::3] = 0.0
    fused = ops.lm_head_loss_raw(op, hidden, weight, targets, shift, rows, active)
    assert fused is not None
    loss, am_d, am_t = fused
    (loss * up).sum().backward()
    ops.check_gemm_status()
    g_fused = hidden.grad.clone()
    hidden.grad = None
    logits = ops.linear(hidden, weight)
    loss2, am_d2, am_t2 = ops.fused_row_loss_raw(op, logits, targets, shift, rows, active)
    (loss2 * up).sum().backward()
    _close(loss, loss2, atol=1e-4, rtol=1e-4)  # same bf16 logits, same statistics, another order of summation
    assert torch.equal(am_t, am_t2)
    lg = logits.detach().float()[:rows]
    same = am_d == am_d2
    picked = torch.gather(lg, 1, am_d.clamp_min(0).long().unsqueeze(1)).squeeze(1)
    assert (same | (picked == lg.max(-1).values)).all()  # equal maxima may pick either index only on exact ties
    _close(hidden.grad, g_fused, atol=1e-3, rtol=1e-2)
    ref = _row_loss_ref(op, lg, targets.float()[shift: shift + rows])
    ref = torch.where(active, ref, torch.zeros_like(ref))
    _close(loss, ref, atol=3e-3, rtol=3e-3)
    assert (loss[~active] == 0).all() and (am_d[~active] == -1).all() and (am_t[~active] == -2).all()


def test_lm_head_fused_saturated_rows(monkeypatch):
    monkeypatch.setenv("SB200_FUSED_HEAD", "1")
    T, H, V = 256, 128, 512
    hidden = torch.zeros(T, H, device=DEV, dtype=torch.bfloat16)
    hidden[:, 0] = 1.0
    weight = torch.zeros(V, H, device=DEV, dtype=torch.bfloat16)
    weight[3, 0] = 30.0
    weight[7, 0] = -30.0
    targets = torch.zeros(T, V, device=DEV, dtype=torch.bfloat16)
    targets[0::2, 3] = 30.0
    targets[1::2, 9] = 30.0
    for op in ("kl_div", "ce"):
        loss, am_d, am_t = ops.lm_head_loss_raw(op, hidden, weight, targets, 0, T, None)
        ref = _row_loss_ref(op, (hidden.float() @ weight.float().t()), targets.float())
        assert torch.isfinite(loss).all()
        _close(loss, ref, atol=2e-3, rtol=2e-3)
        assert (am_d == 3).all() and (am_t[0::2] == 3).all() and (am_t[1::2] == 9).all()
