"""tcgen05 / TMEM / TMA GEMM against an fp32 PyTorch matmul of the same bf16 operands."""

import pytest
import torch

from speculators_b200 import ops

pytestmark = pytest.mark.gpu


def _run(M, N, K, epilogue=0, lda_pad=0, seed=0, variant=0):
    torch.manual_seed(seed)
    a_full = (torch.randn(M, K + lda_pad, device="cuda") * 0.5).to(torch.bfloat16)
    a = a_full[:, :K]
    b = (torch.randn(N, K, device="cuda") * 0.5).to(torch.bfloat16)
    out = (torch.randn(M, N, device="cuda")).to(torch.bfloat16)
    res = (torch.randn(M, N, device="cuda")).to(torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ref = a.float() @ b.float().t()
    if epilogue == 1:
        ref = ref + out.float()
    elif epilogue == 2:
        ref = ref + res.float()
    ops.native().gemm_tn_variant(a, b, out, res if epilogue == 2 else None, epilogue, status, variant)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"kernel reported wait timeout code {int(status.item())}"
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 0.01 * scale + 0.05, (M, N, K, epilogue, err, scale)


def test_single_tile():
    _run(128, 256, 64, variant=1)


def test_single_pair_tile():
    """One 256x256 tile on one CTA pair (tcgen05 cta_group::2), one k-block."""
    _run(256, 256, 64, variant=2)
    _run(256, 256, 64, variant=3)


@pytest.mark.parametrize("M,N,K", [(128, 256, 512), (256, 512, 256), (200, 300, 136), (2048, 4096, 1024), (77, 1000, 72), (1000, 520, 4096)])
@pytest.mark.parametrize("variant", [1, 2, 3])
def test_shapes_including_ragged_edges(M, N, K, variant):
    _run(M, N, K, variant=variant)


@pytest.mark.parametrize("variant", [1, 2, 3])
def test_strided_a_and_epilogues(variant):
    _run(256, 512, 192, lda_pad=64, variant=variant)
    _run(384, 768, 320, epilogue=1, variant=variant)
    _run(384, 768, 320, epilogue=2, variant=variant)
    _run(130, 260, 72, epilogue=1, variant=variant)


def test_many_tiles_per_pair_wraps_the_ring():
    """More tiles than CTA pairs and more k-blocks than pipeline stages: exercises the
    phase wrap of every barrier and both accumulator buffers."""
    for variant in (2, 3):
        _run(2048, 6144, 1024, variant=variant)
        _run(4096, 5120, 640, epilogue=2, variant=variant)
        _run(512, 768, 192, variant=variant)  # K not a multiple of the 128-wide stage: zero-filled tail


# ---- transposed operands read in place (the backward products of a linear layer) -----------
def _run_ex(M, N, K, a_mn, b_mn, epilogue=0, pad=0, seed=0):
    """a stored [K, M] when a_mn else [M, K]; b stored [K, N] when b_mn else [N, K]; ``pad``
    extra columns make the row strides larger than the row lengths (views into wider buffers)."""
    torch.manual_seed(seed)

    def operand(rows, cols):
        full = (torch.randn(rows, cols + pad, device="cuda") * 0.5).to(torch.bfloat16)
        return full[:, :cols]

    a = operand(K, M) if a_mn else operand(M, K)
    b = operand(K, N) if b_mn else operand(N, K)
    out_full = torch.randn(M, N + pad, device="cuda").to(torch.bfloat16)
    out = out_full[:, :N]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    ref = af @ bf
    if epilogue == 1:
        ref = ref + out.float()
    guard = out_full[:, N:].clone()
    ops.native().gemm(a, b, out, epilogue, a_mn, b_mn, status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0, f"kernel reported wait timeout code {int(status.item())}"
    err = (out.float() - ref).abs().max().item()
    scale = ref.abs().max().item()
    assert err <= 0.01 * scale + 0.05, (M, N, K, a_mn, b_mn, epilogue, err, scale)
    assert torch.equal(out_full[:, N:], guard)  # nothing written past the matrix


LAYOUTS = [(False, True), (True, True), (True, False), (False, False)]  # NN (dgrad), TN (wgrad), TT, NT


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
def test_layouts_single_tile_and_one_stage(a_mn, b_mn):
    _run_ex(256, 256, 128, a_mn, b_mn)


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
@pytest.mark.parametrize("M,N,K", [(256, 512, 256), (200, 304, 136), (2048, 4096, 1024), (80, 1000, 72), (1000, 520, 4096), (264, 8, 200)])
def test_layouts_ragged_shapes(a_mn, b_mn, M, N, K):
    _run_ex(M, N, K, a_mn, b_mn)


@pytest.mark.parametrize("a_mn,b_mn", LAYOUTS)
def test_layouts_strided_views_and_accumulate(a_mn, b_mn):
    _run_ex(384, 768, 320, a_mn, b_mn, pad=64)
    _run_ex(384, 768, 320, a_mn, b_mn, epilogue=1)
    _run_ex(136, 264, 72, a_mn, b_mn, epilogue=1, pad=8)


def test_layouts_many_tiles_wrap_the_ring():
    _run_ex(2048, 4096, 32000 // 8, False, True)   # dgrad through a tall weight
    _run_ex(6144, 8192, 2048, True, True, epilogue=1)  # wgrad accumulate, more tiles than CTA pairs


def test_linear_backward_runs_on_the_own_kernel():
    """dX and dW of ``ops.linear`` against fp32 autograd, with the weight gradient accumulated
    into an attached flat buffer over two passes (what the training engine sets up)."""
    torch.manual_seed(0)
    T, IN, OUT = 640, 512, 768
    x = (torch.randn(T, IN, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = torch.nn.Parameter((torch.randn(OUT, IN, device="cuda") * 0.05).to(torch.bfloat16))
    w._flat_grad = torch.zeros_like(w)
    w._grad_fresh = True
    dy = (torch.randn(T, OUT, device="cuda") * 0.1).to(torch.bfloat16)
    before = ops.native().launch_count()
    for _ in range(2):
        y = ops.linear(x, w)
        (dx,) = torch.autograd.grad(y, x, dy, retain_graph=False)
    torch.cuda.synchronize()
    assert ops.native().launch_count() - before == 6  # forward, dgrad, wgrad per pass: no library GEMM
    ops.check_gemm_status()
    xf, wf, dyf = x.detach().float(), w.detach().float(), dy.float()
    assert (dx.float() - dyf @ wf).abs().max() <= 0.01 * (dyf @ wf).abs().max() + 0.02
    want = 2 * (dyf.t() @ xf)
    assert (w._flat_grad.float() - want).abs().max() <= 0.01 * want.abs().max() + 0.05


# ---- grouped (mixture-of-experts) products --------------------------------------------------
@pytest.mark.parametrize("counts", [[300, 0, 17, 512, 129, 1, 0, 255], [0, 0, 640, 0], [128] * 16, [5]])
def test_grouped_linear_forward_and_gradients(counts):
    """Rows sorted by expert through ``grouped_linear`` (padded expert order, tile schedule from
    device-side counts) against one fp32 matmul per expert: outputs, input gradient and the
    per-expert weight gradients; experts without rows get an all-zero weight gradient."""
    torch.manual_seed(0)
    E, K, N = len(counts), 256, 512
    R = sum(counts)
    cnt = torch.tensor(counts, device="cuda")
    x = (torch.randn(R, K, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(E, N, K, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_()
    plan = ops.GroupPlan(cnt, R)
    assert plan.capacity % 128 == 0 and int(plan.seg[-1]) <= plan.capacity and (plan.seg % 128 == 0).all()
    y = plan.unpad(ops.grouped_linear(plan.pad(x), w, plan))
    dy = (torch.randn(R, N, device="cuda") * 0.3).to(torch.bfloat16)
    y.backward(dy)
    torch.cuda.synchronize()
    ops.check_gemm_status()
    xf, wf = x.detach().float(), w.detach().float()
    ref, dxr, dwr = torch.zeros(R, N, device="cuda"), torch.zeros(R, K, device="cuda"), torch.zeros_like(wf)
    off = 0
    for e, c in enumerate(counts):
        rows = slice(off, off + c)
        ref[rows] = xf[rows] @ wf[e].t()
        dxr[rows] = dy.float()[rows] @ wf[e]
        dwr[e] = dy.float()[rows].t() @ xf[rows]
        off += c
    assert (y.float() - ref).abs().max() <= 0.01 * ref.abs().max() + 0.03
    assert (x.grad.float() - dxr).abs().max() <= 0.01 * dxr.abs().max() + 0.03
    assert (w.grad.float() - dwr).abs().max() <= 0.01 * dwr.abs().max() + 0.05
    for e, c in enumerate(counts):
        if c == 0:
            assert (w.grad[e] == 0).all()


def test_moe_block_runs_its_experts_on_the_grouped_kernel():
    """A sparse MoE block at kernel-friendly widths: bf16 CUDA forward / backward through the
    grouped tcgen05 path against the same block with the dense per-expert loop in fp32."""
    import copy

    from speculators_b200.layer_config import TransformerLayerConfig
    from speculators_b200.models.moe import SparseMoeBlock

    cfg = TransformerLayerConfig(model_type="qwen3_next", hidden_size=256, intermediate_size=512, num_hidden_layers=1, num_attention_heads=4,
                                 num_key_value_heads=2, head_dim=64, vocab_size=512, num_experts=8, num_experts_per_tok=2,
                                 moe_intermediate_size=256, shared_expert_intermediate_size=256, norm_topk_prob=True)
    torch.manual_seed(0)
    ref = SparseMoeBlock(cfg)
    gpu = copy.deepcopy(ref).to("cuda", torch.bfloat16)
    x = torch.randn(700, 256) * 0.5
    xg = x.to("cuda", torch.bfloat16).requires_grad_()
    before = ops.native().launch_count()
    yg = gpu(xg)
    yg.float().pow(2).mean().backward()
    torch.cuda.synchronize()
    ops.check_gemm_status()
    assert ops.native().launch_count() - before >= 6  # plan, two grouped forwards, their gradients
    xr = x.to(torch.bfloat16).float().requires_grad_()
    for p_ref, p_gpu in zip(ref.parameters(), gpu.parameters()):
        p_ref.data = p_gpu.data.detach().float().cpu()
    yr = ref(xr)
    yr.pow(2).mean().backward()
    assert (yg.float().cpu() - yr).abs().max() < 0.03 * yr.abs().max() + 0.02
    gmax = xr.grad.abs().max()
    assert (xg.grad.float().cpu() - xr.grad).abs().max() < 0.05 * gmax + 1e-4
    wr, wg = ref.experts.gate_up_proj.grad, gpu.experts.gate_up_proj.grad.float().cpu()
    assert (wg - wr).abs().max() < 0.05 * wr.abs().max() + 1e-4


# ---- gate | up product with SwiGLU in the epilogue ---------------------------------------------------
@pytest.mark.parametrize("T,H,I", [(300, 256, 384), (2048, 512, 1024), (130, 128, 128), (257, 384, 1792)])
def test_gate_up_product_with_swiglu_epilogue_matches_two_step_form(T, H, I, monkeypatch):
    from speculators_b200 import ops

    torch.manual_seed(T + I)
    x = (torch.randn(T, H, device="cuda") * 0.8).to(torch.bfloat16)
    w = (torch.randn(2 * I, H, device="cuda") * 0.08).to(torch.bfloat16)
    dh = (torch.randn(T, I, device="cuda")).to(torch.bfloat16)

    def run(fused):
        monkeypatch.setenv("SB200_FUSED_SWIGLU", "1" if fused else "0")
        xa, wa = x.clone().requires_grad_(), w.clone().requires_grad_()
        h = ops.linear_swiglu(xa, wa) if fused else None
        if not fused:
            assert ops.linear_swiglu(xa, wa) is None
            h = ops.swiglu(ops.linear(xa, wa))
        h.backward(dh)
        return h.detach(), xa.grad, wa.grad

    h1, dx1, dw1 = run(True)
    h0, dx0, dw0 = run(False)
    ops.check_gemm_status()
    # fp32 reference of the op: silu(x Wg^T) * (x Wu^T) from bf16-rounded gate / up
    gu = (x.float() @ w.float().t()).to(torch.bfloat16).float()
    g, u = gu[:, :I], gu[:, I:]
    ref = (torch.nn.functional.silu(g).to(torch.bfloat16).float() * u)
    torch.testing.assert_close(h1.float(), ref, rtol=2e-2, atol=2e-2)
    # same accumulation and the same rounding points as the two-step form
    assert torch.equal(h1, h0)
    assert torch.equal(dx1, dx0) and torch.equal(dw1, dw0)
