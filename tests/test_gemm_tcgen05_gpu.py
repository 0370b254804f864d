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
