#!/usr/bin/env python
"""Headline benchmark: EAGLE-3 draft training throughput for a Llama-3.1-8B-shaped
verifier (hidden 4096, 32 heads / 8 KV heads, intermediate 14336, vocab 128256),
1 draft layer, draft vocab 32000, aux layers (2, 16, 29), TTT length 3, AdamW
lr 1e-4, bf16, sequence 2048 with micro-batch 1 per GPU, sharded data parallel
over N GPUs.  Synthetic seeded tokens, random-init weights.

    python bench.py --gpus N --steps K --warmup W            # this framework
    python bench.py --impl reference --gpus N --steps K ...   # unmodified reference (baseline/_ref)

For N > 1 launch under ``python -m torch.distributed.run --nproc-per-node N``.
Rank 0 prints one JSON line.  ``value`` is whole-job tokens/s from K steps timed
with CUDA events between barriers (max over ranks) with the batch already on the
device; ``e2e`` repeats the measurement through ``Trainer.train_step_async`` with the
batch in pinned host memory (H2D copy every step, started one step ahead on a side
stream) and a device-to-host read of every step's loss (the host reads step n's loss once
step n + 1 is enqueued; the last one at once).
"""

from __future__ import annotations

import argparse
import json
import os
import shutil
import statistics
import subprocess
import sys
import tempfile
import time

REPO = os.path.dirname(os.path.abspath(__file__))

LLAMA31_8B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": 4096, "num_hidden_layers": 32,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "intermediate_size": 14336,
    "vocab_size": 128256, "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "max_position_embeddings": 131072,
    "hidden_act": "silu", "attention_bias": False, "mlp_bias": False, "tie_word_embeddings": False,
    "initializer_range": 0.02,
}
TINY = dict(LLAMA31_8B, hidden_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2,
            head_dim=64, intermediate_size=688, vocab_size=1024, rope_theta=10000.0, max_position_embeddings=4096)
AUX_LAYERS = {"llama31_8b": [2, 16, 29], "tiny": [1, 2, 3]}
METRIC = "EAGLE3-8B draft-train tokens/s at 1/2/4/8 B200 (device max over ranks)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--model", choices=["llama31_8b", "tiny"], default="llama31_8b")
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--draft-vocab", type=int, default=None)
    ap.add_argument("--ttt-steps", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-verifier-forward", action="store_true", help="draw hidden states from N(0,1) instead of running the random-init verifier")
    ap.add_argument("--device", default=None)
    return ap.parse_args()


# ----------------------------------------------------------------------------- helpers
class ClockSampler:
    """nvidia-smi sampled every 200 ms while the timed region runs (rank 0 only)."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.proc, self.path = gpu_index, None, None

    def start(self):
        if shutil.which("nvidia-smi") is None:
            return
        fd, self.path = tempfile.mkstemp(suffix=".csv")
        os.close(fd)
        self.proc = subprocess.Popen(
            ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu_index)],
            stdout=open(self.path, "w"), stderr=subprocess.DEVNULL,
        )

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, power, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in open(self.path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        os.unlink(self.path)
        # keep the samples taken under load (top half by power) for the median
        if sm:
            cut = sorted(power)[len(power) // 2]
            loaded = [s for s, p in zip(sm, power) if p >= cut] or sm
            return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(mx), "power_w_max": max(power), "samples": len(sm), "reasons": sorted(reasons)}
        return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}


def dist_env():
    return int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))


def build_vocab_maps(torch, vocab_size: int, draft_vocab: int, seq_len: int, seed: int = 0):
    """Top-``draft_vocab`` ids by frequency in a seeded uniform token stream."""
    from speculators_b200.train.vocab_mapping import build_vocab_mappings_from_distribution, token_frequency_from_ids

    gen = torch.Generator().manual_seed(seed + 17)
    stream = torch.randint(0, vocab_size, (64 * seq_len,), generator=gen)
    return build_vocab_mappings_from_distribution(token_frequency_from_ids(stream), draft_vocab, vocab_size)


def verifier_dir(torch, cfg: dict, tag: str, local_rank: int, barrier) -> str:
    """config.json + embed / lm_head / norm safetensors of the random verifier,
    written once per node by local rank 0."""
    from speculators_b200.verifier import write_random_verifier_stub

    path = os.path.join(tempfile.gettempdir(), f"sb200_bench_verifier_{tag}")
    done = os.path.join(path, ".done")
    if local_rank == 0 and not os.path.exists(done):
        dev = "cuda" if torch.cuda.is_available() else "cpu"
        write_random_verifier_stub(path, cfg, seed=0, dtype=torch.bfloat16, device=dev)
        open(done, "w").close()
    barrier()
    return path


def make_batches(torch, args, cfg, rank: int, device, n_batches: int = 2):
    from speculators_b200.train.synthetic import make_eagle3_batch
    from speculators_b200.verifier import RandomVerifier

    aux = AUX_LAYERS[args.model]
    verifier = None
    if not args.no_verifier_forward:
        verifier = RandomVerifier(cfg, seed=0, device=device, dtype=torch.bfloat16 if device.type == "cuda" else torch.float32)
    out = []
    for i in range(n_batches):
        out.append(make_eagle3_batch(
            args.seq_len, cfg["hidden_size"], len(aux), cfg["vocab_size"], seed=1000 * rank + i, mask_p=0.6,
            mask_span=max(1, min(64, args.seq_len // 32)), dtype=torch.bfloat16, verifier=verifier, layer_ids=aux, pin=device.type == "cuda",
        ))
    del verifier
    return out


def timed_region(torch, dist, world, device, fn_step, batches, steps, warmup, lookahead=False):
    """W untimed + K timed steps; returns per-rank milliseconds for the K steps.  With
    ``lookahead`` the step function also receives the batch of the following step (None for
    the last warm-up step and the last timed step, so that every timed step's input copy
    starts and ends inside the timed region)."""
    cuda = device.type == "cuda"

    def barrier():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def call(i, last):
        b = batches[i % len(batches)]
        if lookahead:
            fn_step(b, None if last else batches[(i + 1) % len(batches)])
        else:
            fn_step(b)

    for i in range(warmup):
        call(i, i == warmup - 1)
    barrier()
    if cuda:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
    t0 = time.perf_counter()
    for i in range(steps):
        call(warmup + i, i == steps - 1)
    if cuda:
        end.record()
    barrier()
    ms = start.elapsed_time(end) if cuda else (time.perf_counter() - t0) * 1000.0
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


# ----------------------------------------------------------------------------- this framework
def run_ours(args):
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REPO)
    import speculators_b200 as sb
    from speculators_b200 import ops
    from speculators_b200.layer_config import TransformerLayerConfig
    from speculators_b200.parallel import maybe_destroy_distributed, maybe_setup_distributed
    from speculators_b200.train import Trainer, TrainerConfig
    from speculators_b200.train.synthetic import SyntheticLoader

    rank, local_rank, world = dist_env()
    maybe_setup_distributed()
    device = torch.device(args.device) if args.device else (torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu"))
    cfg = dict(LLAMA31_8B if args.model == "llama31_8b" else TINY)
    draft_vocab = args.draft_vocab or (32000 if args.model == "llama31_8b" else 512)
    torch.manual_seed(0)

    def barrier():
        if world > 1:
            dist.barrier()

    vdir = verifier_dir(torch, cfg, args.model, local_rank, barrier)
    d2t, t2d = build_vocab_maps(torch, cfg["vocab_size"], draft_vocab, args.seq_len)
    draft_cfg = TransformerLayerConfig(**dict(cfg, num_hidden_layers=1, sliding_window=2048, layer_types=["sliding_attention"]))
    model = sb.Eagle3DraftModel.from_training_args(
        draft_cfg, t2d=t2d, d2t=d2t, draft_vocab_size=draft_vocab, norm_before_residual=True, norm_before_fc=True,
        norm_output=True, ttt_steps=args.ttt_steps, verifier_name_or_path=vdir, target_layer_ids=AUX_LAYERS[args.model],
    )
    train_kwargs, _ = sb.Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", ttt_steps=args.ttt_steps, ttt_step_loss_decay=1.0)
    batches = make_batches(torch, args, cfg, rank, device)
    loader = SyntheticLoader(batches, args.steps + args.warmup)
    trainer = Trainer(model, TrainerConfig(
        lr=1e-4, num_epochs=1, save_path=os.path.join(tempfile.gettempdir(), "sb200_bench_unused"), train_call_kwargs=train_kwargs,
        optimizer="adamw", scheduler_type="none", log_freq=10**9, fsdp_shard=world > 1,
        use_cuda_graph=not args.no_graph, device=str(device),
    ), loader)
    trainer.model.train()
    tokens_per_step = sum(int((b["document_ids"] != -1).sum()) for b in batches) / len(batches)

    # (1) device-resident inputs
    dev_batches = [{k: v.to(device) for k, v in b.items()} for b in batches]
    sampler = ClockSampler(local_rank)
    cuda = device.type == "cuda"
    count0 = ops.native().launch_count() if cuda else 0

    def step_dev(b):
        trainer.train_step(b)

    if rank == 0 and cuda:
        sampler.start()
    ms = timed_region(torch, dist, world, device, step_dev, dev_batches, args.steps, args.warmup)
    clocks = sampler.stop() if (rank == 0 and cuda) else {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    launches = _count_launches(trainer, ops, count0, args.steps, args.warmup, cuda)

    # (2) end to end: pinned host batch -> H2D every step, loss read back every step
    last = {}

    def step_e2e(b, upcoming):
        # the public training call: this step's batch plus the one that follows, whose
        # host-to-device copy the trainer overlaps with this step's compute.  Every step's loss
        # is read back on the host; the read of step n happens once step n + 1 is enqueued, so
        # the device does not idle while the host reads (the last step is read at once).
        handle = trainer.train_step_async(b, upcoming)
        if last.get("pending") is not None:
            last["loss"] = last["pending"].value()
        last["pending"] = handle
        if upcoming is None:
            last["loss"] = handle.value()
            last["pending"] = None

    ms_e2e = timed_region(torch, dist, world, device, step_e2e, batches, args.steps, min(args.warmup, 3), lookahead=True)
    h2d = sum(v.numel() * v.element_size() for v in batches[0].values())

    value = world * tokens_per_step * args.steps / (ms / 1000.0)
    e2e = world * tokens_per_step * args.steps / (ms_e2e / 1000.0)
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if cuda else "fp32",
            "data": "synthetic (seeded uniform tokens; random-init verifier forward for hidden states; random-init draft)",
            "impl": "ours",
            "config": {"model": "eagle3 1-layer draft for llama-3.1-8b-arch verifier" if args.model == "llama31_8b" else "tiny", "global_batch": world,
                       "seq_len": args.seq_len, "parallelism": f"dp{world}" + ("-sharded" if world > 1 else ""),
                       "optimizer_comm": ("nvls multimem" if getattr(trainer.engine, "nvls", False) else "nvlink p2p" if getattr(trainer.engine, "p2p", False)
                                          else "nccl" if world > 1 else "none"),
                       "draft_vocab": draft_vocab,
                       "ttt_steps": args.ttt_steps, "optimizer": "adamw lr 1e-4",
                       "cuda_graph": trainer._graphed is not None,
                       "l2": "per-step working set (1.9 GB of weights + activations) exceeds the 126 MB L2; 2 distinct input batches alternate"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "last_loss": last.get("loss")},
            "gpu_launches": launches,
        }))
    maybe_destroy_distributed()


def _count_launches(trainer, ops, count0, steps, warmup, cuda):
    if not cuda:
        return 0
    g = trainer._graphed
    if g is not None and g.cache:
        per_step = max(getattr(g, "launches_per_capture", {}).values(), default=0)
        extra = ops.native().launch_count() - count0 - getattr(g, "capture_launch_total", 0)
        # launches recorded at capture time are replayed once per step; launches made
        # eagerly (outside the graph) are counted directly and scaled to the timed steps
        return int(per_step * steps + max(0, extra) * steps / max(1, steps + warmup))
    return int((ops.native().launch_count() - count0) * steps / max(1, steps + warmup))


# ----------------------------------------------------------------------------- reference arm
def run_reference(args):
    ref_root = os.path.join(REPO, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_root, "speculators")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed (pip --target install of the reference missing)"}))
        return
    sys.path.insert(0, ref_root)
    try:
        import torch
        import torch.distributed as dist
        from transformers import LlamaConfig

        from speculators.models.eagle3.core import Eagle3DraftModel
        from speculators.train.distributed import maybe_destroy_distributed, maybe_setup_distributed
        from speculators.train.trainer import Trainer, TrainerConfig
    except Exception as err:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"reference import failed: {type(err).__name__}: {err}"[:300]}))
        return
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "no CUDA device (the reference trainer places the model on an accelerator)"}))
        return

    rank, local_rank, world = dist_env()
    maybe_setup_distributed()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    cfg = dict(LLAMA31_8B if args.model == "llama31_8b" else TINY)
    draft_vocab = args.draft_vocab or (32000 if args.model == "llama31_8b" else 512)
    torch.manual_seed(0)

    def barrier():
        if world > 1:
            dist.barrier()

    # data and the verifier stub directory are plain tensors / files; building them
    # with this repo's helpers keeps both arms on identical inputs
    sys.path.insert(1, REPO)
    vdir = verifier_dir(torch, cfg, args.model, local_rank, barrier)
    d2t, t2d = build_vocab_maps(torch, cfg["vocab_size"], draft_vocab, args.seq_len)
    batches = make_batches(torch, args, cfg, rank, device)

    hf_cfg = LlamaConfig(**{k: v for k, v in cfg.items() if k not in ("architectures", "model_type", "rope_theta")})
    hf_cfg.num_hidden_layers = 1
    hf_cfg.sliding_window = 2048
    hf_cfg.layer_types = ["sliding_attention"]
    try:
        hf_cfg.rope_parameters = {"rope_type": "default", "rope_theta": cfg["rope_theta"]}
    except Exception:  # noqa: BLE001
        hf_cfg.rope_theta = cfg["rope_theta"]
    model = Eagle3DraftModel.from_training_args(
        hf_cfg, t2d=t2d, d2t=d2t, draft_vocab_size=draft_vocab, norm_before_residual=True, norm_before_fc=True,
        norm_output=True, ttt_steps=args.ttt_steps, verifier_name_or_path=vdir, target_layer_ids=AUX_LAYERS[args.model],
    )
    train_kwargs, _ = Eagle3DraftModel.get_trainer_kwargs(loss_fn="kl_div", loss_implementation="fused", ttt_steps=args.ttt_steps, ttt_step_loss_decay=1.0)
    tokens_per_step = sum(int((b["document_ids"] != -1).sum()) for b in batches) / len(batches)

    class TimedLoader:
        """Feeds W + K batches to the stock ``Trainer.train_epoch`` loop and brackets the
        last K with barrier + synchronize + CUDA events from inside the iterator."""

        class _Sampler:
            def set_epoch(self, _e):
                pass

        def __init__(self, items, warmup, steps):
            self.items, self.warmup, self.steps = items, warmup, steps
            self.batch_sampler = self._Sampler()
            self.ms = None

        def __len__(self):
            return self.warmup + self.steps

        def __iter__(self):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for i in range(self.warmup + self.steps):
                if i == self.warmup:
                    barrier(); torch.cuda.synchronize(); start.record()
                yield self.items[i % len(self.items)]
            end.record()
            barrier(); torch.cuda.synchronize()
            self.ms = start.elapsed_time(end)

    def run(items, warmup):
        loader = TimedLoader(items, warmup, args.steps)
        if run.trainer is None:
            run.trainer = Trainer(model, TrainerConfig(
                lr=1e-4, num_epochs=1, save_path=os.path.join(tempfile.gettempdir(), "sb200_ref_unused"), resume_from_checkpoint=False,
                train_call_kwargs=train_kwargs, optimizer="adamw", scheduler_type="none", log_freq=10**9, fsdp_shard=world > 1,
            ), loader)
        else:
            run.trainer.train_loader = loader
            run.trainer.global_step = 1  # keep the once-per-log_freq profiling sync out of the timed steps
        run.trainer.train_epoch(0)
        ms = loader.ms
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    run.trainer = None
    sampler = ClockSampler(local_rank)
    dev_batches = [{k: v.to(device) for k, v in b.items()} for b in batches]
    try:
        run(dev_batches, max(args.warmup, 3))  # first call pays torch.compile; discard
        if rank == 0:
            sampler.start()
        ms = run(dev_batches, args.warmup)
        clocks = sampler.stop() if rank == 0 else {}
        ms_e2e = run(batches, min(args.warmup, 3))
    except Exception as err:  # noqa: BLE001
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference run failed: {type(err).__name__}: {err}"[:400]}))
        maybe_destroy_distributed()
        return
    value = world * tokens_per_step * args.steps / (ms / 1000.0)
    e2e = world * tokens_per_step * args.steps / (ms_e2e / 1000.0)
    h2d = sum(v.numel() * v.element_size() for v in batches[0].values())
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (same generator as the `ours` arm)", "impl": "reference",
            "config": {"model": "eagle3 1-layer draft for llama-3.1-8b-arch verifier" if args.model == "llama31_8b" else "tiny", "global_batch": world,
                       "seq_len": args.seq_len, "parallelism": f"dp{world}" + ("-fsdp2" if world > 1 else ""), "draft_vocab": draft_vocab,
                       "ttt_steps": args.ttt_steps, "optimizer": "adamw lr 1e-4",
                       "path": "speculators.train.trainer.Trainer.train_epoch, torch.compile + flex attention + fused Triton loss (stock)"},
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
        }))
    maybe_destroy_distributed()


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
