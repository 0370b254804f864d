"""Kernel microbenchmarks: ``python -m speculators_b200.ops.microbench --op <name>``.

Each op runs the package's own CUDA kernel on one GPU at the shapes it sees in an
EAGLE-3 step for an 8B verifier (overridable), times it with CUDA events on the
launching stream (warm-up first, an L2-sized buffer rewritten between iterations) and
prints one JSON line with the median time, the algorithmic bytes / FLOPs and, when
``--peaks <json>`` names a file with ``hbm_gbs`` and ``bf16_tflops``, the fraction of
those measured peaks.  ``--iters 1 --warmup 0`` gives a short run for a profiler.
"""

from __future__ import annotations

import argparse
import json
import statistics
import sys

import torch


def _timeit(fn, iters: int, warmup: int, flush: torch.Tensor | None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        stop.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(stop))
    return statistics.median(times)


def _bf16(*shape, scale: float = 1.0) -> torch.Tensor:
    return (torch.randn(*shape, device="cuda") * scale).bfloat16()


def _no_grad(fn):
    def run():
        with torch.no_grad():
            return fn()

    return run


def op_gemm(a):
    from speculators_b200 import ops

    nat = ops.native()
    M, N, K = a.m, a.n, a.k
    x, w, out = _bf16(M, K), _bf16(N, K, scale=0.05), torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = lambda: nat.gemm_tn_variant(x, w, out, None, 0, status, a.variant)  # noqa: E731
    return fn, 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N), lambda: {"status": int(status.item())}


def op_gemm_cublas(a):
    M, N, K = a.m, a.n, a.k
    x, w, out = _bf16(M, K), _bf16(N, K, scale=0.05), torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    return (lambda: torch.matmul(x, w.t(), out=out)), 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N), dict


def _layout_operands(a, a_mn: bool, b_mn: bool):
    M, N, K = a.m, a.n, a.k
    x = _bf16(K, M) if a_mn else _bf16(M, K)
    w = _bf16(K, N, scale=0.05) if b_mn else _bf16(N, K, scale=0.05)
    return x, w, torch.zeros(M, N, device="cuda", dtype=torch.bfloat16)


def op_gemm_dgrad(a):
    """out[M,N] = x[M,K] @ w[K,N] (input gradient of a linear layer: M tokens, K out features, N in features)."""
    from speculators_b200 import ops

    x, w, out = _layout_operands(a, False, True)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = lambda: ops.native().gemm(x, w, out, 0, False, True, status)  # noqa: E731
    return fn, 2.0 * a.m * a.n * a.k, 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n), lambda: {"status": int(status.item())}


def op_gemm_dgrad_cublas(a):
    x, w, out = _layout_operands(a, False, True)
    return (lambda: torch.mm(x, w, out=out)), 2.0 * a.m * a.n * a.k, 2.0 * (a.m * a.k + a.n * a.k + a.m * a.n), dict


def op_gemm_wgrad(a):
    """out[M,N] += dy[K,M]^T @ x[K,N] (weight gradient: M out features, N in features, K tokens)."""
    from speculators_b200 import ops

    x, w, out = _layout_operands(a, True, True)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = lambda: ops.native().gemm(x, w, out, 1, True, True, status)  # noqa: E731
    return fn, 2.0 * a.m * a.n * a.k, 2.0 * (a.m * a.k + a.n * a.k + 2 * a.m * a.n), lambda: {"status": int(status.item())}


def op_gemm_wgrad_cublas(a):
    x, w, out = _layout_operands(a, True, True)
    return (lambda: out.addmm_(x.t(), w)), 2.0 * a.m * a.n * a.k, 2.0 * (a.m * a.k + a.n * a.k + 2 * a.m * a.n), dict


def op_gemm_swiglu(a):
    """gate | up product of a gated MLP with silu(gate) * up formed in the GEMM's epilogue: x[M,K], w[2N,K] -> [M,2N] and [M,N]."""
    from speculators_b200 import ops

    M, I, K = a.m, a.n, a.k
    x, w = _bf16(M, K), _bf16(2 * I, K, scale=0.05)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    fn = lambda: ops.native().gemm_swiglu(x, w, status)  # noqa: E731
    return fn, 4.0 * M * I * K, 2.0 * (M * K + 2 * I * K + 3 * M * I), lambda: {"status": int(status.item())}


def op_gemm_swiglu_unfused(a):
    """The same as two launches: the plain GEMM, then the element-wise SwiGLU kernel."""
    from speculators_b200 import ops

    M, I, K = a.m, a.n, a.k
    x, w, out = _bf16(M, K), _bf16(2 * I, K, scale=0.05), torch.empty(M, 2 * I, device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def fn():
        ops.native().gemm(x, w, out, 0, False, False, status)
        ops.native().swiglu_fwd(out)

    return fn, 4.0 * M * I * K, 2.0 * (M * K + 2 * I * K + 5 * M * I), lambda: {"status": int(status.item())}


def _head_inputs(a):
    T, H, V = a.t, a.hidden, a.vocab
    hidden, weight, targets = _bf16(T, H, scale=0.7), _bf16(V, H, scale=0.05), _bf16(T, V, scale=3.0)
    active = torch.ones(T, dtype=torch.bool, device="cuda")
    return hidden, weight, targets, active, 2.0 * T * V * H, 2.0 * (T * H + V * H + 2 * T * V)


def op_lmhead_fused(a):
    """lm_head GEMM whose epilogue reduces the tiles for the KL loss + the per-row combine kernel."""
    from speculators_b200 import ops

    import os

    os.environ["SB200_FUSED_HEAD"] = "1"
    hidden, weight, targets, active, flops, nbytes = _head_inputs(a)
    return _no_grad(lambda: ops.lm_head_loss_raw("kl_div", hidden, weight, targets, 0, a.t, active)), flops, nbytes, dict


def op_lmhead_unfused(a):
    """The same result as two steps: lm_head GEMM, then the row-loss forward kernel over logits and targets."""
    from speculators_b200 import ops

    hidden, weight, targets, active, flops, nbytes = _head_inputs(a)
    return _no_grad(lambda: ops.fused_row_loss_raw("kl_div", ops.linear(hidden, weight), targets, 0, a.t, active)), flops, nbytes + 2.0 * 2 * a.t * a.vocab, dict


def _attn_inputs(a):
    from speculators_b200.models.eagle3.attention import ttt_attn_spec

    T, nh, nkv, hd, step = a.t, a.heads, a.kv_heads, a.head_dim, a.ttt_step
    doc = torch.zeros(T, dtype=torch.long, device="cuda")
    spec = ttt_attn_spec(doc, step)
    q, k, v = (_bf16(T, h, hd).requires_grad_() for h in (nh, nkv, nkv))
    ke = _bf16(step * T, nkv, hd).requires_grad_() if step else None
    ve = _bf16(step * T, nkv, hd).requires_grad_() if step else None
    flops = 4.0 * T * T * nh * hd / 2 + 4.0 * T * step * nh * hd  # causal half + one extra key per earlier pass
    nbytes = 2.0 * hd * (2 * T * nh + 2 * T * nkv * (1 + step))
    return q, k, v, ke, ve, spec, flops, nbytes


def op_attn_fwd(a):
    from speculators_b200.ops import masked_attention

    q, k, v, ke, ve, spec, flops, nbytes = _attn_inputs(a)
    return _no_grad(lambda: masked_attention(q, k, v, spec, ke, ve)), flops, nbytes, dict


def op_attn_bwd(a):
    from speculators_b200.ops import masked_attention

    q, k, v, ke, ve, spec, flops, nbytes = _attn_inputs(a)
    out = masked_attention(q, k, v, spec, ke, ve)
    go = torch.ones_like(out)
    return (lambda: out.backward(go, retain_graph=True)), 2.5 * flops, 2.5 * nbytes, dict


def op_loss(a):
    from speculators_b200 import ops

    T, V = a.t, a.vocab
    logits, targets = _bf16(T, V), _bf16(T, V)
    active = torch.ones(T, dtype=torch.bool, device="cuda")
    return _no_grad(lambda: ops.fused_row_loss("kl_div", logits, targets, 0, None, active)), 0.0, 2.0 * 2 * T * V, dict


def op_rmsnorm(a):
    from speculators_b200 import ops

    T, H = a.t, a.hidden
    x, w = _bf16(T, H), torch.ones(H, device="cuda", dtype=torch.bfloat16)
    return _no_grad(lambda: ops.rms_norm(x, w, 1e-5)), 0.0, 2.0 * 2 * T * H, dict


def op_rmsnorm_bwd(a):
    from speculators_b200 import ops

    T, H = a.t, a.hidden
    x = _bf16(T, H).requires_grad_()
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = ops.rms_norm(x, w, 1e-5)
    gy = torch.randn_like(y)
    return (lambda: y.backward(gy, retain_graph=True)), 0.0, 2.0 * 3 * T * H, dict


def op_adamw(a):
    from speculators_b200 import ops

    n = a.numel
    master, m, v = (torch.zeros(n, device="cuda") for _ in range(3))
    g, w16 = _bf16(n, scale=0.01), torch.zeros(n, device="cuda", dtype=torch.bfloat16)
    hyper = torch.zeros(ops.HYPER_LEN, device="cuda")
    ops.native().set_hyper(hyper, [1e-4, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001, 1.0, 1.0])
    norm_sq = torch.ones(1, device="cuda")
    fn = lambda: ops.adamw_step_(master, m, v, g, w16, hyper, norm_sq)  # noqa: E731
    return fn, 0.0, n * (3 * 4 * 2 + 2 + 2.0), dict


OPS = {"gemm_swiglu": op_gemm_swiglu, "gemm_swiglu_unfused": op_gemm_swiglu_unfused, "gemm": op_gemm, "gemm_cublas": op_gemm_cublas, "gemm_dgrad": op_gemm_dgrad, "gemm_dgrad_cublas": op_gemm_dgrad_cublas,
       "gemm_wgrad": op_gemm_wgrad, "gemm_wgrad_cublas": op_gemm_wgrad_cublas, "lmhead_fused": op_lmhead_fused, "lmhead_unfused": op_lmhead_unfused, "attn_fwd": op_attn_fwd, "attn_bwd": op_attn_bwd, "loss": op_loss,
       "rmsnorm": op_rmsnorm, "rmsnorm_bwd": op_rmsnorm_bwd, "adamw": op_adamw}


def main(argv: list[str] | None = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", choices=sorted(OPS), required=True)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true", help="do not rewrite an L2-sized buffer between iterations")
    ap.add_argument("--peaks", default=None, help="JSON file with measured hbm_gbs and bf16_tflops")
    ap.add_argument("--variant", type=int, default=0, help="gemm: 0 choose, 1 one CTA per tile, 2 CTA pairs")
    ap.add_argument("-m", type=int, default=2048)
    ap.add_argument("-n", type=int, default=6144)
    ap.add_argument("-k", type=int, default=8192)
    ap.add_argument("-t", type=int, default=2048, help="tokens")
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--ttt-step", type=int, default=0)
    ap.add_argument("--vocab", type=int, default=32000)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--numel", type=int, default=1 << 28)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print(json.dumps({"op": args.op, "unavailable": "no CUDA device"}))
        return 0
    torch.manual_seed(0)
    fn, flops, nbytes, extra = OPS[args.op](args)
    flush = None if args.no_flush else torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ms = _timeit(fn, args.iters, args.warmup, flush)
    rec = {"op": args.op, "ms": round(ms, 4), "tflops": round(flops / ms / 1e9, 1), "gbs": round(nbytes / ms / 1e6, 1),
           "iters": args.iters, "warmup": args.warmup, "l2_flush": not args.no_flush}
    rec.update(extra())
    if args.peaks:
        with open(args.peaks) as fh:
            peaks = json.load(fh)
        if flops and peaks.get("bf16_tflops"):
            rec["frac_of_measured_bf16"] = round(rec["tflops"] / peaks["bf16_tflops"], 3)
        if peaks.get("hbm_gbs"):
            rec["frac_of_measured_hbm"] = round(rec["gbs"] / peaks["hbm_gbs"], 3)
    print(json.dumps(rec))
    return 0


if __name__ == "__main__":
    sys.exit(main())
