"""Row-parallel product of a tensor-parallel group (``parallel/tp_comm.py``): the GEMM whose epilogue
scatters its tiles to the owning ranks' staging areas, then the reduce / broadcast kernel.  One
device, the ranks as virtual ranks of this process run one after another (no kernel waits for another)."""

import pytest
import torch

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)

from speculators_b200 import ops  # noqa: E402
from speculators_b200.parallel.tp_comm import TpComm  # noqa: E402

DEV = torch.device("cuda", 0)


@pytest.mark.parametrize("world,T,N,K", [(2, 300, 1024, 256), (4, 257, 1024, 384), (4, 2048, 2048, 512), (1, 130, 512, 128)])
@pytest.mark.parametrize("with_residual", [False, True])
def test_scatter_product_and_reduce_broadcast_match_fp32_sum(world, T, N, K, with_residual):
    torch.manual_seed(world * 1000 + T)
    comms = [TpComm(None, rows=max(T, 512), width=N, device=DEV, rank=r, world=world, spin_limit=1 << 20) for r in range(world)]
    TpComm.connect_local(comms)
    try:
        xs = [(torch.randn(T, K, device=DEV) * 0.5).to(torch.bfloat16) for _ in range(world)]
        ws = [(torch.randn(N, K, device=DEV) * 0.1).to(torch.bfloat16) for _ in range(world)]
        residual = (torch.randn(T, N, device=DEV)).to(torch.bfloat16) if with_residual else None
        for c, x, w in zip(comms, xs, ws):
            c.scatter_product(x, w)
        outs = [c.reduce_broadcast(T, residual) for c in comms]
        ops.check_gemm_status()
        for c in comms:
            c.check_status()
        # every rank's partial product is rounded to bf16 when it is staged; the sum and the residual add run in fp32
        ref = sum((x.float() @ w.float().t()).to(torch.bfloat16).float() for x, w in zip(xs, ws))
        if residual is not None:
            ref = ref + residual.float()
        for out in outs:  # every rank holds the complete result
            torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=6e-2)  # one bf16 rounding of sums of magnitude up to 8
            assert torch.equal(out, outs[0])
        # a second round lands in the other buffer and leaves the first result intact
        first = outs[0].clone()
        for c, x, w in zip(comms, xs, ws):
            c.scatter_product(x, w)
        again = [c.reduce_broadcast(T, outs[i]) for i, c in enumerate(comms)]
        assert torch.equal(outs[0], first)
        torch.testing.assert_close(again[0].float(), (ref - (residual.float() if residual is not None else 0)) + first.float(), rtol=2e-2, atol=1.2e-1)
    finally:
        for c in comms:
            c.close()


def test_sizes_the_scatter_epilogue_cannot_take_are_refused():
    assert TpComm.supported(8192, 4) and TpComm.supported(4096, 8) and not TpComm.supported(1024, 8) and not TpComm.supported(1000, 2)
    with pytest.raises(ValueError):
        TpComm(None, rows=128, width=768, device=DEV, rank=0, world=2)
