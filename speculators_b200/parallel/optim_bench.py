"""Time the sharded optimizer step alone, per communication mode.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29540 \\
        -m speculators_b200.parallel.optim_bench --params 293601280 --iters 20

Every rank holds a flat bf16 gradient / weight buffer of ``--params`` elements (default:
the trainable size of a 1-layer EAGLE-3 draft for an 8B verifier) and runs
``TrainEngine.step()`` (gradient reduce-scatter, global norm, AdamW on the shard, weight
all-gather) ``--iters`` times after a warm-up, timed with CUDA events on the device;
rank 0 prints one JSON line per mode with the maximum over ranks.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--params", type=int, default=293601280)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--modes", default="nccl,p2p,nvls")
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from speculators_b200.parallel import EngineConfig, TrainEngine

    cols = 4096
    rows = max(8, args.params // cols)
    for mode in [m for m in args.modes.split(",") if m]:
        model = torch.nn.Linear(cols, rows, bias=False)
        try:
            eng = TrainEngine(model, EngineConfig(lr=1e-4, shard=world > 1, comm=mode if world > 1 else "auto", compute_dtype=torch.bfloat16),
                              device=f"cuda:{local}")
        except Exception as err:  # noqa: BLE001
            if rank == 0:
                print(json.dumps({"mode": mode, "unavailable": str(err)[:200]}))
            continue
        eng.flat_g.normal_(0, 0.01)
        eng.mark_grads_written()
        for _ in range(args.warmup):
            eng.step()
        torch.cuda.synchronize()
        dist.barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(args.iters):
            eng.mark_grads_written()
            eng.step()
        stop.record()
        torch.cuda.synchronize()
        eng.check_status()
        ms = torch.tensor([start.elapsed_time(stop) / args.iters], device="cuda")
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        if rank == 0:
            nbytes = eng.total * 2
            print(json.dumps({"mode": mode, "world": world, "params": eng.total, "ms_per_step": round(float(ms), 4),
                              "nvls": bool(eng.nvls), "p2p": bool(eng.p2p),
                              "per_rank_link_gb_each_way": round(2 * nbytes * (world - 1) / world / 1e9, 3)}))
        eng.close()
        del eng, model
        torch.cuda.empty_cache()
        dist.barrier()
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
