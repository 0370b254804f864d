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
TINY = dict(LLAMA31_8B, hidden_size=256, num_hidden_layers=6, num_attention_heads=4, num_key_value_heads=2,
            head_dim=64, intermediate_size=688, vocab_size=1024, rope_theta=10000.0, max_position_embeddings=4096)
QWEN3_8B = dict(LLAMA31_8B, architectures=["Qwen3ForCausalLM"], model_type="qwen3", num_hidden_layers=36, intermediate_size=12288,
                vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1000000.0, max_position_embeddings=40960)
LLAMA33_70B = dict(LLAMA31_8B, hidden_size=8192, num_hidden_layers=80, num_attention_heads=64, intermediate_size=28672)
# the MTP layer of a Qwen3-Next-80B-A3B-shaped verifier: gated full attention (head dim 256), 512 experts top-10 + shared expert
QWEN3_NEXT_MTP = {
    "architectures": ["Qwen3NextForCausalLM"], "model_type": "qwen3_next", "hidden_size": 2048, "num_hidden_layers": 48,
    "num_attention_heads": 16, "num_key_value_heads": 2, "head_dim": 256, "intermediate_size": 5632, "vocab_size": 151936,
    "rms_norm_eps": 1e-6, "rope_theta": 10000000.0, "partial_rotary_factor": 0.25, "max_position_embeddings": 262144,
    "hidden_act": "silu", "attention_bias": False, "tie_word_embeddings": False, "initializer_range": 0.02,
    "num_experts": 512, "num_experts_per_tok": 10, "moe_intermediate_size": 512, "shared_expert_intermediate_size": 512,
    "norm_topk_prob": True, "decoder_sparse_step": 1, "mlp_only_layers": [],
}
TINY_MOE = dict(QWEN3_NEXT_MTP, hidden_size=256, num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                vocab_size=1024, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256, shared_expert_intermediate_size=256,
                max_position_embeddings=4096)
VERIFIERS = {"llama31_8b": LLAMA31_8B, "tiny": TINY, "qwen3_8b": QWEN3_8B, "llama33_70b": LLAMA33_70B, "qwen3_next_mtp": QWEN3_NEXT_MTP,
             "tiny_moe": TINY_MOE}
METRIC = "EAGLE3-8B draft-train tokens/s at 1/2/4/8 B200 (device max over ranks)"
PARITY_STEPS = 6  # optimizer steps from the common initial weights whose losses both arms record
PARITY_RTOL = 0.03

# One entry per measured configuration.  ``model`` / ``train``: keyword arguments that both
# frameworks' ``from_training_args`` / ``get_trainer_kwargs`` take under the same names.
CONFIGS = {
    # EAGLE-3, 1 draft layer for a Llama-3.1-8B-shaped verifier (the headline; the default)
    "eagle3": dict(
        algo="eagle3", verifier="llama31_8b", seq_len=2048, draft_vocab=32000, aux=[2, 16, 29], draft_layers=1,
        layer_types=["sliding_attention"], sliding_window=2048, verifier_forward=True,
        model=dict(norm_before_residual=True, norm_before_fc=True, norm_output=True, ttt_steps=3),
        train=dict(loss_fn="kl_div", ttt_steps=3, ttt_step_loss_decay=1.0),
        label="eagle3 1-layer draft for llama-3.1-8b-arch verifier",
    ),
    # DFlash / DSpark for a Qwen3-8B-shaped verifier: 5 layers, blocks of 16, 512 anchors, window 2048 except layer 0
    "dflash": dict(
        algo="dflash", verifier="qwen3_8b", seq_len=4096, draft_vocab=32000, aux=[2, 10, 18, 26, 33], draft_layers=5,
        layer_types=["full_attention"] + ["sliding_attention"] * 4, sliding_window=2048, verifier_forward=False,
        model=dict(block_size=16, mask_token_id=151935),
        train=dict(loss_fn="ce", per_position_loss_weight="dpace", dpace_alpha=0.5, dflash_decay_gamma=4.0, max_anchors=512),
        label="dflash 5-layer draft (block 16, 512 anchors) for qwen3-8b-arch verifier",
    ),
    "dspark": dict(
        algo="dspark", verifier="qwen3_8b", seq_len=4096, draft_vocab=32000, aux=[2, 10, 18, 26, 33], draft_layers=5,
        layer_types=["full_attention"] + ["sliding_attention"] * 4, sliding_window=2048, verifier_forward=False,
        model=dict(block_size=16, mask_token_id=151935, markov_rank=256, markov_head_type="vanilla", enable_confidence_head=True,
                   confidence_head_with_markov=True),
        train=dict(loss_fn="kl_div", per_position_loss_weight="fixed-exp-decay", dflash_decay_gamma=4.0, max_anchors=512,
                   confidence_head_alpha=1.0),
        label="dspark 5-layer draft (block 16, 512 anchors, markov + confidence heads) for qwen3-8b-arch verifier",
    ),
    # P-EAGLE, 1 draft layer at the width of a Llama-3.3-70B-shaped verifier, 4 parallel depths
    "peagle": dict(
        algo="peagle", verifier="llama33_70b", seq_len=2048, draft_vocab=32000, aux=[2, 40, 77], draft_layers=1,
        layer_types=["sliding_attention"], sliding_window=2048, verifier_forward=False,
        model=dict(norm_before_residual=True, norm_before_fc=True, norm_output=True, num_depths=4, mask_token_id=128255),
        train=dict(loss_fn="kl_div", num_depths=4, down_sample_ratio=0.7, down_sample_ratio_min=0.2),
        label="peagle 1-layer draft (4 depths) for llama-3.3-70b-arch verifier",
    ),
    # the same draft trained online on one box: first half of the GPUs run the 70B-shaped verifier tensor-parallel and
    # write hidden states into the trainer GPUs' rings over NVLink, second half train (needs >= 2 GPUs)
    "peagle_online": dict(
        algo="peagle", verifier="llama33_70b", seq_len=2048, draft_vocab=32000, aux=[2, 40, 77], draft_layers=1,
        layer_types=["sliding_attention"], sliding_window=2048, verifier_forward=False, online=True,
        model=dict(norm_before_residual=True, norm_before_fc=True, norm_output=True, num_depths=4, mask_token_id=128255),
        train=dict(loss_fn="kl_div", num_depths=4, down_sample_ratio=0.7, down_sample_ratio_min=0.2),
        label="peagle 1-layer draft (4 depths), online: llama-3.3-70b-arch verifier tensor-parallel on half of the GPUs",
    ),
    # MTP-head fine-tuning for a Qwen3-Next-80B-A3B-shaped MTP layer, experts split over the ranks (expert parallel)
    "mtp_moe": dict(
        algo="mtp", verifier="qwen3_next_mtp", seq_len=4096, draft_vocab=None, aux=[48], draft_layers=1, layer_types=None,
        sliding_window=None, verifier_forward=False, model=dict(num_speculative_steps=3),
        train=dict(num_speculative_steps=3, step_weight_beta=0.6),
        label="mtp head (gated attention hd 256, 512 experts top-10 + shared) for qwen3-next-80b-a3b-arch verifier",
    ),
    # the CPU / gloo plumbing configuration (tiny Llama verifier run for the hidden states)
    "tiny": dict(
        algo="eagle3", verifier="tiny", seq_len=128, draft_vocab=512, aux=[1, 2, 3], draft_layers=1,
        layer_types=["sliding_attention"], sliding_window=2048, verifier_forward=True,
        model=dict(norm_before_residual=True, norm_before_fc=True, norm_output=True, ttt_steps=3),
        train=dict(loss_fn="kl_div", ttt_steps=3, ttt_step_loss_decay=1.0),
        label="tiny",
    ),
}


def resolve_config(args) -> dict:
    """The configuration entry with the command line's overrides applied."""
    name = args.config or ("tiny" if args.model == "tiny" else "eagle3")
    c = {k: (dict(v) if isinstance(v, dict) else v) for k, v in CONFIGS[name].items()}
    c["name"] = name
    if args.seq_len:
        c["seq_len"] = args.seq_len
    if args.draft_vocab:
        c["draft_vocab"] = args.draft_vocab
    if args.ttt_steps and c["algo"] == "eagle3":
        c["model"]["ttt_steps"] = c["train"]["ttt_steps"] = args.ttt_steps
    if args.no_verifier_forward:
        c["verifier_forward"] = False
    if args.scale == "tiny" and name != "tiny":
        # the same algorithm and flags at plumbing size (CPU checks of this script)
        c.update(verifier="tiny_moe" if c["algo"] == "mtp" else "tiny", seq_len=args.seq_len or 256,
                 draft_vocab=None if c["algo"] == "mtp" else (args.draft_vocab or 512), aux=list(range(1, len(c["aux"]) + 1)))
        if "mask_token_id" in c["model"]:
            c["model"]["mask_token_id"] = TINY["vocab_size"] - 1
        if "max_anchors" in c["train"]:
            c["train"]["max_anchors"] = 16
        c["label"] += " (tiny scale)"
        c["name"] += "_tiny"
    c["metric"] = METRIC if name in ("eagle3", "tiny") else f"{c['algo'].upper()} draft-train tokens/s at 1/2/4/8 B200 (device max over ranks)"
    return c


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--regions", type=int, default=5, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--config", choices=sorted(CONFIGS), default=None, help="measured configuration (default: eagle3, the headline)")
    ap.add_argument("--model", choices=["llama31_8b", "tiny"], default="llama31_8b", help="'tiny' = --config tiny")
    ap.add_argument("--scale", choices=["full", "tiny"], default="full", help="'tiny': the chosen configuration at plumbing size")
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--draft-vocab", type=int, default=None)
    ap.add_argument("--ttt-steps", type=int, default=None)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-expert-parallel", action="store_true", help="mtp_moe on several GPUs: keep all experts on every rank")
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


def inputs_tag(c: dict, device_type: str) -> str:
    return f"{c['name']}_s{c['seq_len']}_v{c['draft_vocab']}_{'vf' if c['verifier_forward'] else 'rand'}_{device_type}"


def config_record(c: dict, world: int, regions: int) -> dict:
    """What is being measured: identical in both arms (how each arm runs it goes under ``impl_detail``)."""
    return {
        "model": c["label"], "global_batch": world, "seq_len": c["seq_len"], "parallelism": f"dp{world}" + ("-sharded" if world > 1 else ""),
        "draft_vocab": c["draft_vocab"], "algorithm": c["algo"], "model_kwargs": c["model"], "train_kwargs": c["train"],
        "optimizer": "adamw lr 1e-4", "regions": regions, "parity_steps": PARITY_STEPS,
        "l2": "per-step working set (GBs of weights + activations) exceeds the 126 MB L2; 2 distinct input batches alternate",
    }


def parity_steps_compared(c: dict) -> int:
    return PARITY_STEPS if c["algo"] == "eagle3" else 1


def data_note(c: dict) -> str:
    hs = "hidden states from a plain-PyTorch forward of the random-init verifier" if c["verifier_forward"] else "hidden states drawn N(0, 1)"
    return f"synthetic (seeded uniform tokens; {hs}; seeded draft init; both arms read the same files)"


def draft_layer_config(c: dict) -> dict:
    """Decoder hyper-parameters of the draft: the verifier's widths, ``draft_layers`` layers (MTP: the
    verifier's own configuration, whose MTP layer is what gets trained)."""
    v = VERIFIERS[c["verifier"]]
    if c["algo"] == "mtp":
        return dict(v)
    return dict(v, num_hidden_layers=c["draft_layers"], sliding_window=c["sliding_window"], layer_types=list(c["layer_types"]))


def timed_region(torch, dist, world, device, fn_step, batches, steps, offset=0, lookahead=False):
    """K timed steps between barrier + synchronize on both sides; returns the K steps' device
    milliseconds (max over ranks).  With ``lookahead`` the step function also receives the
    batch of the following step (None for the last timed step, so that every timed step's
    input copy starts and ends inside the timed region)."""
    cuda = device.type == "cuda"

    def barrier():
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    barrier()
    if cuda:
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
    t0 = time.perf_counter()
    for i in range(steps):
        b = batches[(offset + i) % len(batches)]
        if lookahead:
            fn_step(b, None if i == steps - 1 else batches[(offset + i + 1) % len(batches)])
        else:
            fn_step(b)
    if cuda:
        end.record()
    barrier()
    ms = start.elapsed_time(end) if cuda else (time.perf_counter() - t0) * 1000.0
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def spread(values: list[float]) -> dict:
    return {"median": statistics.median(values), "min": min(values), "max": max(values), "n": len(values)}


def loss_parity(mine: list[float] | None, other: list[float] | None, compared: int = PARITY_STEPS) -> dict:
    """Both arms start from the same draft weights and see the same batches; their losses over
    the first ``compared`` steps must agree within ``PARITY_RTOL`` (bf16 compute on different
    kernels).  Algorithms that draw anchors / depths at random in every step (each arm from its
    own generator) are compared on the first step only: from the second step on the two arms
    train on different samples of the same batch."""
    if not mine or not other:
        return {"loss_parity": None, "loss_parity_note": "the other arm's record is not on this machine"}
    n = min(len(mine), len(other), compared)
    gaps = [abs(a - b) / max(abs(b), 1e-6) for a, b in zip(mine[:n], other[:n])]
    return {"loss_parity": bool(max(gaps) <= PARITY_RTOL), "loss_parity_max_rel_gap": max(gaps), "loss_parity_rtol": PARITY_RTOL,
            "loss_parity_steps_compared": n, "loss_trace_other_arm": other[:len(mine)]}


# ----------------------------------------------------------------------------- this framework
def run_ours_online(args, c):
    """Verifier / trainer split on one box (``OnlineSplit``): tokens/s of the trainer half with the
    verifier half producing its hidden states at the same time, everything device to device."""
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REPO)
    import bench_inputs
    from speculators_b200 import ops
    from speculators_b200.layer_config import TransformerLayerConfig
    from speculators_b200.model import SpeculatorModel
    from speculators_b200.parallel import maybe_destroy_distributed, maybe_setup_distributed
    from speculators_b200.train import Trainer, TrainerConfig
    from speculators_b200.train.online import OnlineSplit
    from speculators_b200.train.synthetic import SyntheticLoader

    rank, local_rank, world = dist_env()
    if world < 2:
        print(json.dumps({"impl": "ours", "config": {"model": c["label"]}, "unavailable": "the online split needs at least 2 GPUs (one verifier, one trainer)"}))
        return
    os.environ.setdefault("SB200_COMM", "nccl")  # the trainer half is a sub-group: library collectives for its optimizer step
    maybe_setup_distributed()
    device = torch.device(args.device) if args.device else (torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu"))
    cuda = device.type == "cuda"
    if cuda:
        torch.cuda.set_device(device)
    cfg, draft_vocab = VERIFIERS[c["verifier"]], c["draft_vocab"]
    torch.manual_seed(0)
    root = bench_inputs.ensure_inputs(cfg, inputs_tag(c, device.type), seq_len=c["seq_len"], draft_vocab=draft_vocab, layer_ids=c["aux"], rank=rank,
                                      local_rank=local_rank, n_batches=0, device=device, verifier_forward=False, barrier=dist.barrier)
    # the verifier runs seq_len tokens per sample (a multiple of the GEMM tile); the pairing shift leaves seq_len - 1 trained positions
    split = OnlineSplit(cfg, c["aux"], c["seq_len"], device, n_slots=4, timeout_s=60.0, sample_tokens=c["seq_len"])
    topo = split.topo
    trainer = None
    last = {}
    if not topo.is_verifier:
        d2t, t2d = bench_inputs.load_vocab_maps(root)
        model_class = SpeculatorModel.registry[c["algo"]]
        model = model_class.from_training_args(
            TransformerLayerConfig(**draft_layer_config(c)), t2d=t2d, d2t=d2t, draft_vocab_size=draft_vocab,
            verifier_name_or_path=os.path.join(root, "verifier"), target_layer_ids=c["aux"], **c["model"],
        )
        model.load_state_dict(bench_inputs.seeded_draft_init({k: tuple(v.shape) for k, v in model.state_dict().items()}), strict=False)
        train_kwargs, _ = model_class.get_trainer_kwargs(**c["train"])
        trainer = Trainer(model, TrainerConfig(
            lr=1e-4, num_epochs=1, save_path=os.path.join(tempfile.gettempdir(), "sb200_bench_unused"), train_call_kwargs=train_kwargs,
            optimizer="adamw", scheduler_type="none", log_freq=10**9, fsdp_shard=topo.n_trainer > 1, use_cuda_graph=not args.no_graph,
            device=str(device), process_group=split.trainer_group,
        ), SyntheticLoader([], 0))
        trainer.model.train()

    def step(batch):
        handle = trainer.train_step_async(batch)
        if last.get("pending") is not None:
            last["loss"] = last["pending"].value()  # every step's loss reaches the host (read one step late)
        last["pending"] = handle

    count0 = ops.native().launch_count() if cuda else 0
    sampler = ClockSampler(local_rank)
    if rank == 0 and cuda:
        sampler.start()
    region_ms = [split.run(step, args.warmup if r == 0 else 0, args.steps) for r in range(args.regions)]
    clocks = sampler.stop() if (rank == 0 and cuda) else {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    if trainer is not None and last.get("pending") is not None:
        last["loss"] = last["pending"].value()
    launches = int((ops.native().launch_count() - count0) * args.steps / max(1, args.steps * args.regions + args.warmup)) if cuda else 0
    if cuda:
        ops.check_gemm_status()
    loss_t = torch.tensor([last.get("loss") or 0.0, 0.0 if topo.is_verifier else 1.0], dtype=torch.float64, device=device)
    dist.all_reduce(loss_t)
    ms = statistics.median(region_ms)
    tokens = topo.n_trainer * (c["seq_len"] - 1)
    value = tokens * args.steps / (ms / 1000.0)
    if rank == 0:
        record = {
            "metric": "PEAGLE online draft-train tokens/s on one box split between verifier and trainer GPUs (device max over ranks)",
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if cuda else "fp32",
            "data": "synthetic (seeded uniform tokens; hidden states computed by the random-init verifier during the run; seeded draft init)",
            "impl": "ours", "config": dict(config_record(c, world, args.regions), parallelism=f"tp{topo.n_verifier} verifier + dp{topo.n_trainer}-sharded trainer",
                                            global_batch=topo.n_trainer),
            "impl_detail": {"verifier": f"TensorParallelVerifier over {topo.n_verifier} GPUs, weights resident",
                            "verifier_comm": os.environ.get("SB200_TP_COMM", "peer (GEMM epilogue scatter + reduce / broadcast kernel) where the sizes allow"),
                            "handoff": "NVLink peer-memory ring, batch built on the trainer GPU",
                            "optimizer_comm": os.environ.get("SB200_COMM"), "path": "speculators_b200.train.online.OnlineSplit.run / Trainer.train_step_async"},
            "regions_ms_per_step": spread([m / args.steps for m in region_ms]), "clocks": clocks,
            "e2e": {"value": value, "unit": "tokens/s", "ms_per_step": ms / args.steps, "h2d_bytes_per_step": 8 * c["seq_len"] * topo.n_trainer,
                    "d2h_bytes_per_step": 4 * topo.n_trainer,
                    "note": "the timed region is end to end already: token ids are the only host input, hidden states go GPU to GPU, every step's loss is read on the host"},
            "last_loss": float(loss_t[0] / max(1.0, float(loss_t[1]))), "gpu_launches": launches,
        }
        print(json.dumps(record))
    split.close()
    maybe_destroy_distributed()


def run_ours(args):
    if resolve_config(args).get("online"):
        return run_ours_online(args, resolve_config(args))
    import torch
    import torch.distributed as dist

    sys.path.insert(0, REPO)
    import bench_inputs
    import speculators_b200 as sb
    from speculators_b200 import ops
    from speculators_b200.layer_config import TransformerLayerConfig
    from speculators_b200.model import SpeculatorModel
    from speculators_b200.parallel import maybe_destroy_distributed, maybe_setup_distributed
    from speculators_b200.train import Trainer, TrainerConfig
    from speculators_b200.train.synthetic import SyntheticLoader

    rank, local_rank, world = dist_env()
    maybe_setup_distributed()
    device = torch.device(args.device) if args.device else (torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu"))
    cuda = device.type == "cuda"
    if cuda:
        torch.cuda.set_device(device)
    c = resolve_config(args)
    cfg, draft_vocab = VERIFIERS[c["verifier"]], c["draft_vocab"]
    torch.manual_seed(0)

    def barrier():
        if world > 1:
            dist.barrier()

    tag = inputs_tag(c, device.type)
    root = bench_inputs.ensure_inputs(
        cfg, tag, seq_len=c["seq_len"], draft_vocab=draft_vocab, layer_ids=c["aux"], rank=rank, local_rank=local_rank,
        n_batches=2, device=device, verifier_forward=c["verifier_forward"], barrier=barrier, kind=c["algo"],
    )
    batches = bench_inputs.load_batches(root, rank, pin=cuda)
    model_class = SpeculatorModel.registry[c["algo"]]
    expert_parallel = False
    if c["algo"] == "mtp":
        from speculators_b200.config import SpeculatorsConfig, VerifierConfig
        from speculators_b200.models.mtp.config import MTPSpeculatorConfig
        from speculators_b200.proposals.greedy import GreedyTokenProposalConfig

        expert_parallel = world > 1 and not args.no_expert_parallel
        spec_cfg = MTPSpeculatorConfig(
            transformer_layer_config=TransformerLayerConfig(**draft_layer_config(c)),
            speculators_config=SpeculatorsConfig(
                algorithm="mtp", proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=c["model"]["num_speculative_steps"])],
                default_proposal_method="greedy", verifier=VerifierConfig.from_pretrained(os.path.join(root, "verifier")),
            ),
        )
        model = model_class(spec_cfg, ep_group=dist.group.WORLD if expert_parallel else None)
        model.load_verifier_weights()
    else:
        d2t, t2d = bench_inputs.load_vocab_maps(root)
        model = model_class.from_training_args(
            TransformerLayerConfig(**draft_layer_config(c)), t2d=t2d, d2t=d2t, draft_vocab_size=draft_vocab,
            verifier_name_or_path=os.path.join(root, "verifier"), target_layer_ids=c["aux"], **c["model"],
        )
    shapes = {k: tuple(v.shape) for k, v in model.state_dict().items()}
    if expert_parallel:  # initial values are drawn for the stack of all experts; every rank loads its own slice
        shapes = {k: ((v[0] * world, *v[1:]) if ".experts." in k else v) for k, v in shapes.items()}
    init = bench_inputs.seeded_draft_init(shapes)
    missing = model.load_state_dict(init, strict=False)
    assert not missing.unexpected_keys, missing.unexpected_keys
    train_kwargs, _ = model_class.get_trainer_kwargs(**c["train"])
    loader = SyntheticLoader(batches, args.steps + args.warmup)
    trainer = Trainer(model, TrainerConfig(
        lr=1e-4, num_epochs=1, save_path=os.path.join(tempfile.gettempdir(), "sb200_bench_unused"), train_call_kwargs=train_kwargs,
        optimizer="adamw", scheduler_type="none", log_freq=10**9, fsdp_shard=world > 1,
        use_cuda_graph=not args.no_graph, device=str(device),
    ), loader)
    trainer.model.train()
    tokens_per_step = sum(int((b["document_ids"] != -1).sum()) for b in batches) / len(batches)
    dev_batches = [{k: v.to(device) for k, v in b.items()} for b in batches]
    count0 = ops.native().launch_count() if cuda else 0

    # (0) the first optimizer steps from the common initial weights: their losses are compared
    # with the other arm's (they also serve as warm-up)
    trace = []
    for i in range(PARITY_STEPS):
        loss, _ = trainer.train_step(dev_batches[i % len(dev_batches)])
        trace.append(loss.detach().float().reshape(1).clone())
    trace_t = torch.cat(trace)
    if world > 1:
        dist.all_reduce(trace_t, op=dist.ReduceOp.SUM)
        trace_t /= world
    loss_trace = [float(x) for x in trace_t.cpu()]

    # (1) device-resident inputs
    def step_dev(b):
        trainer.train_step(b)

    for i in range(max(0, args.warmup - PARITY_STEPS)):
        step_dev(dev_batches[i % 2])
    sampler = ClockSampler(local_rank)
    if rank == 0 and cuda:
        sampler.start()
    region_ms = [timed_region(torch, dist, world, device, step_dev, dev_batches, args.steps, offset=r) for r in range(args.regions)]
    clocks = sampler.stop() if (rank == 0 and cuda) else {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
    timed_steps = args.steps * args.regions
    launches = _count_launches(trainer, ops, count0, args.steps, timed_steps + max(args.warmup, PARITY_STEPS), cuda)
    ms = statistics.median(region_ms)

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

    for i in range(min(args.warmup, 3)):
        step_e2e(batches[i % 2], None)
    e2e_ms = [timed_region(torch, dist, world, device, step_e2e, batches, args.steps, offset=r, lookahead=True) for r in range(args.regions)]
    ms_e2e = statistics.median(e2e_ms)
    h2d = sum(v.numel() * v.element_size() for v in batches[0].values())
    comm = _exposed_comm(torch, dist, trainer, ops, world, cuda)
    if cuda:
        ops.check_gemm_status()
        trainer.engine.check_status()

    value = world * tokens_per_step * args.steps / (ms / 1000.0)
    e2e = world * tokens_per_step * args.steps / (ms_e2e / 1000.0)
    if rank == 0:
        record = {
            "metric": c["metric"], "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16" if cuda else "fp32",
            "data": data_note(c),
            "impl": "ours",
            "config": config_record(c, world, args.regions),
            "impl_detail": {
                "optimizer_comm": ("nvls multimem" if getattr(trainer.engine, "nvls", False) else "nvlink p2p" if getattr(trainer.engine, "p2p", False)
                                   else ("nccl" if cuda else "gloo") if world > 1 else "none"),
                "cuda_graph": trainer._graphed is not None,
                "expert_parallel": (os.environ.get("SB200_EP_COMM", "nvlink p2p") if cuda else "gloo all-to-all") if expert_parallel else False,
                "path": "speculators_b200.train.Trainer.train_step / train_step_async",
            },
            "regions_ms_per_step": spread([m / args.steps for m in region_ms]),
            "clocks": clocks,
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                    "regions_ms_per_step": spread([m / args.steps for m in e2e_ms]), "last_loss": last.get("loss")},
            "exposed_comm_ms_per_step": comm,
            "loss_trace": loss_trace, "last_loss": last.get("loss"),
            "gpu_launches": launches,
        }
        record.update(loss_parity(loss_trace, (bench_inputs.read_result(tag, "reference", world) or {}).get("loss_trace"), parity_steps_compared(c)))
        bench_inputs.write_result(tag, "ours", world, {"loss_trace": loss_trace})
        print(json.dumps(record))
    maybe_destroy_distributed()


def _exposed_comm(torch, dist, trainer, ops, world, cuda):
    """Milliseconds per step that the training stream spends in communication.  One GPU: none.
    Library collectives: their own CUDA-event time over a few optimizer steps (they run on the
    training stream, nothing overlaps them).  Fused peer-memory step: the two kernels hold the
    transfers and the AdamW arithmetic together, so the figure is their time minus that of the
    local AdamW kernel over a buffer of the shard's size."""
    if world == 1 or not cuda:
        return 0.0 if world == 1 else None
    eng = trainer.engine
    reps = 5

    def timed(fn):
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / reps], dtype=torch.float64, device=eng.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    if getattr(eng, "p2p", False):
        eng.mark_grads_written()
        fused = timed(eng.step)
        n = eng.hi - eng.lo
        g = torch.zeros(n, dtype=torch.bfloat16, device=eng.device)
        w = torch.zeros(n, dtype=torch.bfloat16, device=eng.device)
        m, v, master = (torch.zeros(n, dtype=torch.float32, device=eng.device) for _ in range(3))
        nsq = torch.zeros(1, dtype=torch.float32, device=eng.device)

        def local():
            ops.sum_of_squares(g, nsq, accumulate=False)
            ops.adamw_step_(master, m, v, g, w, eng.hyper, nsq)

        return max(0.0, fused - timed(local))
    eng.account_comm(True)
    eng.mark_grads_written()
    for _ in range(reps):
        eng.step()
    total = eng.exposed_comm_ms()
    eng.account_comm(False)
    t = torch.tensor([(total or 0.0) / reps], dtype=torch.float64, device=eng.device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _count_launches(trainer, ops, count0, steps, total_steps, cuda):
    """Own-kernel launches inside one timed region of ``steps`` steps."""
    if not cuda:
        return 0
    g = trainer._graphed
    if g is not None and g.cache:
        per_step = max(getattr(g, "launches_per_capture", {}).values(), default=0)
        extra = ops.native().launch_count() - count0 - getattr(g, "capture_launch_total", 0)
        # launches recorded at capture time are replayed once per step; launches made
        # eagerly (outside the graph) are counted directly and scaled to the timed steps
        return int(per_step * steps + max(0, extra) * steps / max(1, total_steps))
    return int((ops.native().launch_count() - count0) * steps / max(1, total_steps))


# ----------------------------------------------------------------------------- reference arm
def run_reference(args):
    """The unmodified reference from ``baseline/_ref`` through its own ``Trainer.train_epoch``.
    Nothing of this framework is imported here: the inputs come from ``bench_inputs`` (plain
    PyTorch) as files that the other arm reads too."""
    ref_root = os.path.join(REPO, "baseline", "_ref")

    def unavailable(why: str) -> None:
        if int(os.environ.get("RANK", "0")) == 0:  # one line per job
            print(json.dumps({"impl": "reference", "unavailable": why[:300]}))

    if not os.path.isdir(os.path.join(ref_root, "speculators")):
        return unavailable("baseline/_ref is not installed (pip --target install of the reference missing)")
    sys.path[:] = [p for p in sys.path if os.path.abspath(p or ".") != REPO]  # the repo root must not shadow or leak packages
    sys.path.insert(0, ref_root)
    try:
        import importlib.util
        import logging

        import torch
        import torch.distributed as dist
        from transformers import LlamaConfig, Qwen3Config

        spec = importlib.util.spec_from_file_location("bench_inputs", os.path.join(REPO, "bench_inputs.py"))
        bench_inputs = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(bench_inputs)

        import speculators.models  # noqa: F401  (registers the algorithms)
        from speculators.model import SpeculatorModel
        from speculators.train.distributed import maybe_destroy_distributed, maybe_setup_distributed
        from speculators.train.trainer import Trainer, TrainerConfig
    except Exception as err:  # noqa: BLE001
        return unavailable(f"reference import failed: {type(err).__name__}: {err}")
    if not torch.cuda.is_available():
        return unavailable("no CUDA device (the reference trainer places the model on an accelerator)")

    rank, local_rank, world = dist_env()
    if resolve_config(args).get("online"):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": "the reference's online mode needs a running vLLM server with verifier weights (scripts/launch_vllm.py); none can be started here"}))
        return
    maybe_setup_distributed()
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    c = resolve_config(args)
    cfg, draft_vocab = VERIFIERS[c["verifier"]], c["draft_vocab"]
    torch.manual_seed(0)

    def barrier():
        if world > 1:
            dist.barrier()

    tag = inputs_tag(c, "cuda")
    root = bench_inputs.ensure_inputs(
        cfg, tag, seq_len=c["seq_len"], draft_vocab=draft_vocab, layer_ids=c["aux"], rank=rank, local_rank=local_rank,
        n_batches=2, device=device, verifier_forward=c["verifier_forward"], barrier=barrier, kind=c["algo"],
    )
    batches = bench_inputs.load_batches(root, rank, pin=True)

    draft = draft_layer_config(c)
    model_class = SpeculatorModel.registry[c["algo"]]
    if c["algo"] == "mtp":
        from transformers import Qwen3NextConfig

        from speculators.config import SpeculatorsConfig, VerifierConfig
        from speculators.models.mtp.config import MTPSpeculatorConfig
        from speculators.proposals.greedy import GreedyTokenProposalConfig

        hf_cfg = Qwen3NextConfig(**{k: v for k, v in draft.items() if k not in ("architectures", "model_type", "rope_theta")})
        try:
            hf_cfg.rope_parameters = {"rope_type": "default", "rope_theta": cfg["rope_theta"], "partial_rotary_factor": cfg["partial_rotary_factor"]}
        except Exception:  # noqa: BLE001
            hf_cfg.rope_theta = cfg["rope_theta"]
        model = model_class(MTPSpeculatorConfig(
            transformer_layer_config=hf_cfg,
            speculators_config=SpeculatorsConfig(
                algorithm="mtp", proposal_methods=[GreedyTokenProposalConfig(speculative_tokens=c["model"]["num_speculative_steps"])],
                default_proposal_method="greedy", verifier=VerifierConfig.from_pretrained(os.path.join(root, "verifier")),
            ),
        ))
        model.load_verifier_weights()
    else:
        d2t, t2d = bench_inputs.load_vocab_maps(root)
        hf_class = Qwen3Config if draft["model_type"] == "qwen3" else LlamaConfig
        hf_cfg = hf_class(**{k: v for k, v in draft.items() if k not in ("architectures", "model_type", "rope_theta")})
        try:
            hf_cfg.rope_parameters = {"rope_type": "default", "rope_theta": cfg["rope_theta"]}
        except Exception:  # noqa: BLE001
            hf_cfg.rope_theta = cfg["rope_theta"]
        model = model_class.from_training_args(
            hf_cfg, t2d=t2d, d2t=d2t, draft_vocab_size=draft_vocab, verifier_name_or_path=os.path.join(root, "verifier"),
            target_layer_ids=c["aux"], **c["model"],
        )
    init = bench_inputs.seeded_draft_init({k: tuple(v.shape) for k, v in model.state_dict().items()})
    with torch.no_grad():
        own = model.state_dict()
        for k, v in init.items():
            own[k].copy_(v)
    train_kwargs, _ = model_class.get_trainer_kwargs(**({} if c["algo"] == "mtp" else {"loss_implementation": "fused"}), **c["train"])
    tokens_per_step = sum(int((b["document_ids"] != -1).sum()) for b in batches) / len(batches)

    class Capture(logging.Handler):
        """Records what the stock trainer logs on its logging steps (its own loss read-back)."""

        def __init__(self):
            super().__init__()
            self.losses, self.n_metrics = [], 0

        def emit(self, record):
            msg = record.msg
            if isinstance(msg, dict) and isinstance(msg.get("train"), dict) and "loss" in msg["train"]:
                self.losses.append(float(msg["train"]["loss"]))

    capture = Capture()
    mlog = logging.getLogger("speculators.metrics")
    mlog.addHandler(capture)
    mlog.setLevel(logging.INFO)

    class TimedLoader:
        """Feeds W + K batches to the stock ``Trainer.train_epoch`` loop and brackets the
        last K with barrier + synchronize + CUDA events from inside the iterator."""

        class _Sampler:
            def set_epoch(self, _e):
                pass

        def __init__(self, items, warmup, steps, offset=0):
            self.items, self.warmup, self.steps, self.offset = items, warmup, steps, offset
            self.batch_sampler = self._Sampler()
            self.ms = None

        def __len__(self):
            return self.warmup + self.steps

        def __iter__(self):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for i in range(self.warmup + self.steps):
                if i == self.warmup:
                    barrier(); torch.cuda.synchronize(); start.record()
                yield self.items[(self.offset + i) % len(self.items)]
            end.record()
            barrier(); torch.cuda.synchronize()
            self.ms = start.elapsed_time(end)

    state = {"trainer": None}

    def run(items, warmup, steps, log_freq, offset=0):
        loader = TimedLoader(items, warmup, steps, offset)
        if state["trainer"] is None:
            state["trainer"] = Trainer(model, TrainerConfig(
                lr=1e-4, num_epochs=1, save_path=os.path.join(tempfile.gettempdir(), "sb200_ref_unused"), resume_from_checkpoint=False,
                train_call_kwargs=train_kwargs, optimizer="adamw", scheduler_type="none", log_freq=log_freq, fsdp_shard=world > 1,
            ), loader)
        tr = state["trainer"]
        tr.train_loader = loader
        tr.config = tr.config._replace(log_freq=log_freq)
        if log_freq > 1:
            tr.global_step = 1  # keeps the once-per-log_freq logging step (synchronize + .item()) out of these steps
        tr.train_epoch(0)
        ms = loader.ms
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local_rank)
    dev_batches = [{k: v.to(device) for k, v in b.items()} for b in batches]
    quiet = 10**9
    try:
        # first optimizer steps from the common initial weights, logged every step through the
        # trainer's own logging path: the loss trace that the other arm is compared with
        # (this call also pays torch.compile)
        run(dev_batches, 0, PARITY_STEPS, 1)
        loss_trace = list(capture.losses[:PARITY_STEPS])
        run(dev_batches, max(args.warmup, 3), 1, quiet)
        if rank == 0:
            sampler.start()
        region_ms = [run(dev_batches, 0, args.steps, quiet, offset=r) for r in range(args.regions)]
        clocks = sampler.stop() if rank == 0 else {}
        # end to end, stock logging path on every step (log_freq=1: synchronize, metric reduce,
        # .item() of every metric = the reference's own loss read-back) ...
        run(batches, min(args.warmup, 3), 1, 1)
        n_before = len(capture.losses)
        e2e_ms = [run(batches, 0, args.steps, 1, offset=r) for r in range(args.regions)]
        logged = len(capture.losses) - n_before
        # ... and without it (no device-to-host read inside the timed steps)
        e2e_nolog_ms = [run(batches, 0, args.steps, quiet, offset=r) for r in range(args.regions)]
    except Exception as err:  # noqa: BLE001
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": f"reference run failed: {type(err).__name__}: {err}"[:400]}))
        maybe_destroy_distributed()
        return
    ms, ms_e2e, ms_nolog = statistics.median(region_ms), statistics.median(e2e_ms), statistics.median(e2e_nolog_ms)
    value = world * tokens_per_step * args.steps / (ms / 1000.0)
    h2d = sum(v.numel() * v.element_size() for v in batches[0].values())
    # the logging step reads the token count (int64) and one fp32 scalar per metric
    with torch.no_grad(), torch.autocast("cuda", dtype=torch.bfloat16):
        n_metrics = len(model(**dev_batches[0], **train_kwargs)[2]) if world == 1 else None
    d2h = 8 + 4 * n_metrics if n_metrics is not None else 12
    if rank == 0:
        record = {
            "metric": c["metric"], "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": data_note(c),
            "impl": "reference",
            "config": config_record(c, world, args.regions),
            "impl_detail": {
                "optimizer_comm": "fsdp2 (nccl)" if world > 1 else "none", "cuda_graph": False,
                "path": "speculators.train.trainer.Trainer.train_epoch, torch.compile + flex attention + fused Triton loss (stock)",
            },
            "regions_ms_per_step": spread([m / args.steps for m in region_ms]),
            "clocks": clocks,
            "e2e": {"value": world * tokens_per_step * args.steps / (ms_e2e / 1000.0), "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "logged_steps": logged,
                    "how": "log_freq=1: the stock trainer's logging step (synchronize, metric reduce, .item() per metric) on every step",
                    "regions_ms_per_step": spread([m / args.steps for m in e2e_ms])},
            "e2e_nolog": {"value": world * tokens_per_step * args.steps / (ms_nolog / 1000.0), "unit": "tokens/s", "ms_per_step": ms_nolog / args.steps,
                          "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 0, "how": "no logging step inside the timed steps"},
            "exposed_comm_ms_per_step": None,
            "loss_trace": loss_trace, "last_loss": capture.losses[-1] if capture.losses else None,
            "gpu_launches": 0,
        }
        record.update(loss_parity(loss_trace, (bench_inputs.read_result(tag, "ours", world) or {}).get("loss_trace"), parity_steps_compared(c)))
        bench_inputs.write_result(tag, "reference", world, {"loss_trace": loss_trace})
        print(json.dumps(record))
    maybe_destroy_distributed()


if __name__ == "__main__":
    a = parse_args()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
