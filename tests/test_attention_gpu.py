"""Masked-attention kernels (forward + backward) against the dense fp32 oracle."""

import pytest
import torch

from speculators_b200.models.eagle3.attention import ttt_attn_spec
from speculators_b200.ops import AttnSpec, masked_attention, masked_attention_reference

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _docs(T, pattern):
    if pattern == "single":
        return torch.zeros(T, dtype=torch.long)
    if pattern == "multi_pad":
        a, b = T // 3, T // 2
        return torch.cat([torch.zeros(a), torch.ones(b), torch.full((T - a - b - 5,), 2), torch.full((5,), -1)]).long()
    raise ValueError(pattern)


def _run(T, nh, nkv, hd, step, window, pattern, fused_buffer=False, seed=0):
    torch.manual_seed(seed)
    doc = _docs(T, pattern).to(DEV)
    spec = ttt_attn_spec(doc, step, sliding_window=window)
    if fused_buffer:
        width = (nh + 2 * nkv) * hd
        qkv = torch.randn(T, width, device=DEV).to(torch.bfloat16)
        q = qkv[:, : nh * hd].view(T, nh, hd)
        k = qkv[:, nh * hd: (nh + nkv) * hd].view(T, nkv, hd)
        v = qkv[:, (nh + nkv) * hd:].view(T, nkv, hd)
    else:
        q = torch.randn(T, nh, hd, device=DEV).to(torch.bfloat16)
        k = torch.randn(T, nkv, hd, device=DEV).to(torch.bfloat16)
        v = torch.randn(T, nkv, hd, device=DEV).to(torch.bfloat16)
    ke = ve = None
    if step > 0:
        ke = torch.randn(step * T, nkv, hd, device=DEV).to(torch.bfloat16)
        ve = torch.randn(step * T, nkv, hd, device=DEV).to(torch.bfloat16)
    leaves = [t.detach().clone().requires_grad_() for t in (q, k, v) + ((ke, ve) if step else ())]
    out = masked_attention(leaves[0], leaves[1], leaves[2], spec, *(leaves[3:] if step else (None, None)))
    dout = torch.randn_like(out)
    out.backward(dout)
    ref_leaves = [t.detach().float().requires_grad_() for t in (q, k, v) + ((ke, ve) if step else ())]
    ref = masked_attention_reference(ref_leaves[0], ref_leaves[1], ref_leaves[2], spec, *(ref_leaves[3:] if step else (None, None)))
    ref.backward(dout.float())
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    names = ["dq", "dk", "dv", "dk_ext", "dv_ext"]
    for name, a, b in zip(names, leaves, ref_leaves):
        tol = 3e-2 * float(b.grad.abs().max()) + 2e-2
        assert float((a.grad.float() - b.grad).abs().max()) < tol, (name, float((a.grad.float() - b.grad).abs().max()), tol)


@pytest.mark.parametrize("hd", [64, 128, 256])
@pytest.mark.parametrize("T", [64, 127, 128, 129, 200, 257])
def test_causal_single_document(T, hd):
    _run(T, 4, 2, hd, step=0, window=None, pattern="single")


@pytest.mark.parametrize("step", [1, 2])
@pytest.mark.parametrize("window", [None, 48])
def test_ttt_steps_multi_document_padding(step, window):
    _run(330, 8, 2, 128, step=step, window=window, pattern="multi_pad")


@pytest.mark.parametrize("step,window,pattern", [(0, None, "multi_pad"), (1, 48, "multi_pad"), (2, None, "single")])
def test_head_dim_256_gqa_documents_and_extra_keys(step, window, pattern):
    """The gated full-attention heads of Qwen3-Next style MTP layers: 16 query heads on 2 KV heads of 256."""
    _run(330, 16, 2, 256, step=step, window=window, pattern=pattern)


def test_views_into_fused_projection_buffer():
    _run(192, 4, 1, 64, step=1, window=None, pattern="multi_pad", fused_buffer=True)


def test_no_gqa_and_sliding_window():
    _run(300, 2, 2, 128, step=0, window=17, pattern="single")


def test_rows_without_any_key_return_zero():
    T, nh, hd = 70, 2, 64
    q = torch.randn(T, nh, hd, device=DEV).to(torch.bfloat16).requires_grad_()
    k = torch.randn(T, nh, hd, device=DEV).to(torch.bfloat16).requires_grad_()
    v = torch.randn(T, nh, hd, device=DEV).to(torch.bfloat16).requires_grad_()
    lo = torch.zeros(T, dtype=torch.int32, device=DEV)
    hi = torch.arange(1, T + 1, dtype=torch.int32, device=DEV)
    hi[10:20] = 0  # empty interval
    out = masked_attention(q, k, v, AttnSpec(lo=lo, hi=hi))
    assert (out[10:20] == 0).all() and torch.isfinite(out).all()
    out.sum().backward()
    assert torch.isfinite(q.grad).all() and (q.grad[10:20] == 0).all()


@pytest.mark.parametrize("impl", ["tc", "mma"])
def test_implementations_head_dim_128(impl, monkeypatch):
    """tcgen05 kernels (TMA tiles, TMEM accumulators) and the mma.sync kernels, forward and
    backward, against the fp32 oracle on multi-tile, multi-document sequences read from a
    fused q|k|v buffer."""
    from speculators_b200.ops import attention_cuda, check_gemm_status

    monkeypatch.setattr(attention_cuda, "FWD_IMPL", impl)
    monkeypatch.setattr(attention_cuda, "BWD_IMPL", impl)
    _run(1100, 8, 2, 128, step=2, window=None, pattern="multi_pad", fused_buffer=True, seed=3)
    _run(700, 4, 4, 128, step=0, window=150, pattern="single", seed=4)
    check_gemm_status()


def test_tc_forward_rows_without_any_key():
    from speculators_b200.ops import check_gemm_status

    T, nh, hd = 300, 2, 128
    q = torch.randn(T, nh, hd, device=DEV).to(torch.bfloat16)
    k = torch.randn(T, nh, hd, device=DEV).to(torch.bfloat16)
    v = torch.randn(T, nh, hd, device=DEV).to(torch.bfloat16)
    lo = torch.zeros(T, dtype=torch.int32, device=DEV)
    hi = torch.arange(1, T + 1, dtype=torch.int32, device=DEV)
    hi[120:140] = 0
    hi[256:] = 0  # a whole query tile without keys
    spec = AttnSpec(lo=lo, hi=hi)
    out = masked_attention(q, k, v, spec)
    ref = masked_attention_reference(q.float(), k.float(), v.float(), spec)
    assert (out[120:140] == 0).all() and (out[256:] == 0).all()
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    check_gemm_status()


def test_tc_kernels_with_separate_query_and_context_lengths_and_many_extras():
    """Block drafting shape: Tq != Tc, every query sees a prefix of the context plus up to
    eight individually addressed extra keys (some slots unused, rows shared between queries)."""
    from speculators_b200.ops import check_gemm_status

    torch.manual_seed(7)
    Tq, Tc, Te, nh, nkv, hd, E = 389, 530, 389, 8, 2, 128, 8
    q = torch.randn(Tq, nh, hd, device=DEV).to(torch.bfloat16)
    k = torch.randn(Tc, nkv, hd, device=DEV).to(torch.bfloat16)
    v = torch.randn(Tc, nkv, hd, device=DEV).to(torch.bfloat16)
    ke = torch.randn(Te, nkv, hd, device=DEV).to(torch.bfloat16)
    ve = torch.randn(Te, nkv, hd, device=DEV).to(torch.bfloat16)
    hi = torch.randint(0, Tc + 1, (Tq,), device=DEV, dtype=torch.int32)
    lo = (hi.float() * torch.rand(Tq, device=DEV)).to(torch.int32)
    block = torch.arange(Tq, device=DEV) // E * E
    ext = block[:, None] + torch.arange(E, device=DEV)[None, :]  # the query's own block of extra rows
    ext = torch.where((ext <= torch.arange(Tq, device=DEV)[:, None]) & (ext < Te), ext, torch.full_like(ext, -1)).to(torch.int32)
    spec = AttnSpec(lo=lo, hi=hi, extra_idx=ext)
    leaves = [t.detach().clone().requires_grad_() for t in (q, k, v, ke, ve)]
    out = masked_attention(leaves[0], leaves[1], leaves[2], spec, leaves[3], leaves[4])
    dout = torch.randn_like(out)
    out.backward(dout)
    refs = [t.detach().float().requires_grad_() for t in (q, k, v, ke, ve)]
    ref = masked_attention_reference(refs[0], refs[1], refs[2], spec, refs[3], refs[4])
    ref.backward(dout.float())
    torch.testing.assert_close(out.float(), ref, atol=2e-2, rtol=2e-2)
    for name, a, b in zip(["dq", "dk", "dv", "dk_ext", "dv_ext"], leaves, refs):
        tol = 3e-2 * float(b.grad.abs().max()) + 2e-2
        assert float((a.grad.float() - b.grad).abs().max()) < tol, name
    check_gemm_status()


@pytest.mark.parametrize("window,non_causal", [(None, False), (64, False), (64, True)])
@pytest.mark.parametrize("n_anchors,block", [(24, 16), (21, 8), (8, 16)])
def test_anchored_blocks_run_their_block_keys_as_a_tile(window, non_causal, n_anchors, block):
    """DFlash / DSpark masks: the block keys of a query tile as one block-diagonal key tile on the tensor
    cores (forward, dQ, and the extra keys' dK / dV) against the fp32 oracle and the per-row extra-key path."""
    from speculators_b200.models.dflash.attention import anchor_block_attn_spec
    from speculators_b200.ops import attention_cuda

    torch.manual_seed(0)
    T, nh, nkv, hd = 300, 4, 2, 128
    doc = _docs(T, "multi_pad").to(DEV)
    real = torch.nonzero(doc != -1).squeeze(1)
    anchors = real[torch.randperm(real.numel(), device=DEV)[:n_anchors]].sort().values
    spec = anchor_block_attn_spec(doc, anchors, block, window, non_causal)
    assert spec.extra_block == block and spec.extra_block_causal == (window is not None and not non_causal)
    Tq = n_anchors * block
    base = [torch.randn(n, h, hd, device=DEV).to(torch.bfloat16) for n, h in ((Tq, nh), (T, nkv), (T, nkv), (Tq, nkv), (Tq, nkv))]
    dout = torch.randn(Tq, nh, hd, device=DEV).to(torch.bfloat16)

    def run(block_path):
        attention_cuda.BLOCK_EXTRAS = block_path
        try:
            leaves = [t.detach().clone().requires_grad_() for t in base]
            out = masked_attention(leaves[0], leaves[1], leaves[2], spec, leaves[3], leaves[4])
            out.backward(dout)
            return out, [t.grad for t in leaves]
        finally:
            attention_cuda.BLOCK_EXTRAS = True

    out_b, g_b = run(True)
    out_r, g_r = run(False)
    ref_leaves = [t.detach().float().requires_grad_() for t in base]
    ref = masked_attention_reference(ref_leaves[0], ref_leaves[1], ref_leaves[2], spec, ref_leaves[3], ref_leaves[4])
    ref.backward(dout.float())
    torch.testing.assert_close(out_b.float(), ref, atol=2e-2, rtol=2e-2)
    torch.testing.assert_close(out_b.float(), out_r.float(), atol=2e-2, rtol=2e-2)
    for name, a, b, c in zip(["dq", "dk", "dv", "dk_ext", "dv_ext"], g_b, ref_leaves, g_r):
        tol = 3e-2 * float(b.grad.abs().max()) + 2e-2
        assert float((a.float() - b.grad).abs().max()) < tol, (name, float((a.float() - b.grad).abs().max()), tol)
        assert float((a.float() - c.float()).abs().max()) < tol, (name, "vs per-row path")
