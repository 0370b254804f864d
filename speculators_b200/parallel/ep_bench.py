"""Time the expert-parallel token exchange of one sparse MoE block, per transport.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29541 \\
        -m speculators_b200.parallel.ep_bench --tokens 4096 --hidden 2048 --experts 64 --top-k 8

Every rank routes ``--tokens`` rows of width ``--hidden`` to ``--top-k`` of ``--experts``
experts (uniform random router weights) and runs the block forward + backward ``--iters``
times after a warm-up: once with the rows moved by the NVLink peer-memory kernels
(``SB200_EP_COMM=p2p``) and once through the process group's all-to-all
(``SB200_EP_COMM=nccl``).  ``--exchange-only`` replaces the experts by the identity so that
only routing, dispatch and combine are timed.  CUDA events on the device, maximum over
ranks; rank 0 prints one JSON line per transport.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=64)
    ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--inter", type=int, default=512)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--modes", default="p2p,nccl")
    ap.add_argument("--exchange-only", action="store_true")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from speculators_b200.layer_config import TransformerLayerConfig
    from speculators_b200.models import moe

    cfg = TransformerLayerConfig(model_type="qwen3_next", hidden_size=args.hidden, intermediate_size=args.inter, num_attention_heads=8,
                                 num_key_value_heads=2, head_dim=128, vocab_size=128, num_experts=args.experts,
                                 num_experts_per_tok=args.top_k, moe_intermediate_size=args.inter, shared_expert_intermediate_size=0)
    torch.manual_seed(0)
    block = moe.SparseMoeBlock(cfg, ep_group=dist.group.WORLD).to(dev).to(torch.bfloat16)
    if args.exchange_only:
        moe._grouped_expert_forward = lambda x, counts, gate_up, down: x * 1.0  # noqa: ARG005 - identity experts
    torch.manual_seed(1 + rank)
    x = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16).requires_grad_()
    dout = torch.randn(args.tokens, args.hidden, device=dev).to(torch.bfloat16)

    def step():
        x.grad = None
        block(x).backward(dout)

    for mode in [m for m in args.modes.split(",") if m]:
        os.environ["SB200_EP_COMM"] = mode
        for _ in range(args.warmup):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.iters):
            step()
        stop.record()
        torch.cuda.synchronize()
        if block._comm is not None:
            block._comm.check_status()
        ms = torch.tensor([start.elapsed_time(stop) / args.iters], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if rank == 0:
            rows = args.tokens * args.top_k
            moved = 4 * rows * args.hidden * 2 * (world - 1) / world  # x, y, dy, dx rows that leave the rank (uniform routing)
            print(json.dumps({"transport": mode, "world": world, "tokens_per_rank": args.tokens, "hidden": args.hidden,
                              "experts": args.experts, "top_k": args.top_k, "exchange_only": bool(args.exchange_only),
                              "ms_fwd_bwd": round(float(ms), 4), "gb_leaving_rank": round(moved / 1e9, 3)}))
        dist.barrier()
    if block._comm is not None:
        block._comm.close()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
