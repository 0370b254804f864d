"""Training benchmark harness: drives the real ``Trainer`` for ``warmup + measured``
steps, collects the per-step phase timings it logs (CUDA-event based on GPU), peak
memory and provenance into one JSON document, and compares two such documents.

Reference surface: scripts/benchmark.py:227 (run_benchmark), :412 (compare_benchmarks).
The result schema (``benchmark_version``, ``provenance``, ``config``, ``memory``,
``timing.<key>.{mean,std,min,max,median,count}``, ``per_step``) is the same, so result
files of either implementation can be compared with ``compare``.
"""

from __future__ import annotations

import argparse
import importlib.metadata
import json
import logging
import socket
import statistics
import subprocess
import sys
from datetime import datetime, timezone
from pathlib import Path

import torch
import torch.distributed as dist

BENCHMARK_VERSION = "1.0"
TIMING_KEYS = ("step_ms", "fwd_ms", "bwd_ms", "opt_ms", "fetch_ms", "tokens_per_s")
_COMPARABILITY = (
    ("config.speculator_type", "Speculator type"), ("config.hidden_size", "Hidden size"),
    ("config.total_seq_len", "Sequence length"), ("config.num_gpus_used", "GPU count"),
    ("config.fsdp_shard", "FSDP shard"), ("config.optimizer", "Optimizer"), ("config.hidden_states_dtype", "Dtype"),
)

__all__ = ["BENCHMARK_VERSION", "TIMING_KEYS", "ProfileCapture", "collect_provenance", "compare_benchmarks",
           "compute_statistics", "create_synthetic_batch", "format_comparison", "run_benchmark"]


class ProfileCapture(logging.Handler):
    """Collects the ``profile`` dicts the trainer sends to the metric logger."""

    def __init__(self):
        super().__init__()
        self.profiles: list[dict] = []

    def emit(self, record: logging.LogRecord) -> None:
        msg = record.msg
        if isinstance(msg, dict) and msg.get("profile") is not None:
            self.profiles.append(msg["profile"])


def _pkg_version(name: str) -> str:
    try:
        return importlib.metadata.version(name)
    except importlib.metadata.PackageNotFoundError:
        return "unknown"


def collect_provenance() -> dict:
    try:
        proc = subprocess.run(["git", "rev-parse", "HEAD"], capture_output=True, text=True, timeout=5, check=False)  # noqa: S607
        sha = proc.stdout.strip() if proc.returncode == 0 else "unknown"
    except OSError:
        sha = "unknown"
    gpus = []
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            props = torch.cuda.get_device_properties(i)
            gpus.append({"name": props.name, "total_memory_gb": round(props.total_memory / 2**30, 2),
                         "compute_capability": [props.major, props.minor]})
    from speculators_b200.version import __version__

    return {
        "git_sha": sha, "timestamp": datetime.now(timezone.utc).isoformat(), "hostname": socket.gethostname(),
        "python_version": sys.version.split()[0], "pytorch_version": torch.__version__,
        "cuda_version": torch.version.cuda or "none", "speculators_version": __version__,
        "transformers_version": _pkg_version("transformers"), "gpu_info": gpus, "num_gpus": len(gpus),
    }


def create_synthetic_batch(total_seq_len: int, hidden_size: int, num_target_layers: int, vocab_size: int = 32000,
                           dtype: torch.dtype = torch.bfloat16, device="cpu") -> dict[str, torch.Tensor]:
    """Random post-collate batch: one document filling the whole packed row, all
    positions supervised."""
    T = total_seq_len
    return {
        "hidden_states": torch.randn(1, T, num_target_layers * hidden_size, dtype=dtype, device=device),
        "input_ids": torch.randint(0, vocab_size, (1, T), device=device),
        "verifier_last_hidden_states": torch.randn(1, T, hidden_size, dtype=dtype, device=device),
        "loss_mask": torch.ones(1, T, dtype=torch.bool, device=device),
        "position_ids": torch.arange(1, T + 1, device=device).unsqueeze(0),
        "document_ids": torch.zeros(1, T, dtype=torch.long, device=device),
    }


def compute_statistics(values: list[float]) -> dict[str, float]:
    return {"mean": statistics.mean(values), "std": statistics.stdev(values) if len(values) > 1 else 0.0,
            "min": min(values), "max": max(values), "median": statistics.median(values), "count": len(values)}


def _train_loader(bench_args, args, model, dtype, total_steps):
    from speculators_b200.train.synthetic import SyntheticLoader

    tlc = model.config.transformer_layer_config
    n_layers = len(model.target_layer_ids)
    if bench_args.synthetic:
        batch = create_synthetic_batch(args.total_seq_len, tlc.hidden_size, n_layers, tlc.vocab_size, dtype)
        if torch.cuda.is_available():
            batch = {k: v.pin_memory() for k, v in batch.items()}
        return SyntheticLoader([batch], total_steps), True
    from speculators_b200.hs_connectors import HiddenStatesBackend
    from speculators_b200.models.eagle3.data import shift_batch
    from speculators_b200.models.mtp.data import shift_batch_mtp
    from speculators_b200.train.dataloader import create_train_val_loaders

    preprocess = {"eagle3": shift_batch, "peagle": shift_batch, "mtp": shift_batch_mtp}.get(args.speculator_type)
    transfer = HiddenStatesBackend.registry[args.hidden_states_backend].from_train_args(args, args.data_path)
    loader, _ = create_train_val_loaders(
        data_path=args.data_path, total_seq_len=args.total_seq_len, hidden_states_dtype=dtype, noise_std=args.noise_std,
        transfer=transfer, vllm_endpoint=args.vllm_endpoint, on_missing=args.on_missing, on_generate=args.on_generate,
        verifier_name_or_path=args.verifier_name_or_path, request_timeout=args.request_timeout, max_retries=args.max_retries,
        hidden_size=tlc.hidden_size, num_target_layers=n_layers, num_workers=args.num_workers,
        prefetch_factor=args.prefetch_factor, preprocess=preprocess, train_data_ratio=args.train_data_ratio,
    )
    return loader, False


def run_benchmark(bench_args: argparse.Namespace, args: argparse.Namespace) -> dict:
    """``bench_args``: synthetic, warmup_steps, measured_steps, output, no_per_step.
    ``args``: the flattened training configuration."""
    from speculators_b200.model import SpeculatorModel
    from speculators_b200.parallel.distributed import get_rank, maybe_destroy_distributed, maybe_setup_distributed
    from speculators_b200.train.entrypoint import build_draft_model, parse_vocab_mappings, set_seed
    from speculators_b200.train.logger import setup_root_logger
    from speculators_b200.train.trainer import Trainer, TrainerConfig

    set_seed(args.seed, getattr(args, "deterministic_cuda", False))
    setup_root_logger()
    maybe_setup_distributed()
    rank = get_rank()
    total_steps = bench_args.warmup_steps + bench_args.measured_steps
    dtype = getattr(torch, args.hidden_states_dtype)
    if args.speculator_type == "mtp":
        d2t = t2d = draft_vocab_size = None
        args.mask_token_id = None
    else:
        d2t, t2d, draft_vocab_size = parse_vocab_mappings(args)
    model_class = SpeculatorModel.registry[args.speculator_type]
    model = build_draft_model(args, model_class, t2d, d2t, draft_vocab_size)
    hidden_size = model.config.transformer_layer_config.hidden_size
    n_layers = len(model.target_layer_ids)
    loader, synthetic = _train_loader(bench_args, args, model, dtype, total_steps)
    train_kwargs, _ = model_class.get_trainer_kwargs(**vars(args))
    trainer = Trainer(model, TrainerConfig(
        lr=args.lr, num_epochs=1, save_path="benchmark_unused", resume_from_checkpoint=False, train_call_kwargs=train_kwargs,
        optimizer=args.optimizer, weight_decay=args.weight_decay, muon_lr=args.muon_lr, muon_momentum=args.muon_momentum,
        muon_weight_decay=args.muon_weight_decay, muon_ns_steps=args.muon_ns_steps, muon_adjust_lr_fn=args.muon_adjust_lr_fn,
        scheduler_type="none", hidden_states_dtype=dtype, log_freq=1, fsdp_shard=args.fsdp_shard, max_steps=total_steps,
    ), loader)
    if rank == 0:
        print(f"Benchmarking: {bench_args.warmup_steps} warmup + {bench_args.measured_steps} measured steps")
    capture = ProfileCapture()
    metric_logger = logging.getLogger("speculators.metrics")
    metric_logger.addHandler(capture)
    on_gpu = torch.cuda.is_available()
    if on_gpu:
        torch.cuda.reset_peak_memory_stats(trainer.local_rank)
    try:
        trainer.train_epoch(0)
    finally:
        metric_logger.removeHandler(capture)
    peak_alloc = torch.cuda.max_memory_allocated(trainer.local_rank) / 2**20 if on_gpu else 0.0
    peak_res = torch.cuda.max_memory_reserved(trainer.local_rank) / 2**20 if on_gpu else 0.0
    measured = capture.profiles[bench_args.warmup_steps:] or capture.profiles
    if len(capture.profiles) <= bench_args.warmup_steps and rank == 0:
        print(f"WARNING: got {len(capture.profiles)} profiles but expected {total_steps}; reporting all of them.")
    results = {
        "benchmark_version": BENCHMARK_VERSION,
        "provenance": collect_provenance(),
        "config": {
            "speculator_type": args.speculator_type, "verifier_name_or_path": args.verifier_name_or_path,
            "total_seq_len": args.total_seq_len, "hidden_size": hidden_size, "num_target_layers": n_layers,
            "optimizer": args.optimizer, "lr": args.lr, "hidden_states_dtype": args.hidden_states_dtype,
            "synthetic_data": synthetic, "fsdp_shard": args.fsdp_shard,
            "num_gpus_used": dist.get_world_size() if dist.is_initialized() else 1,
            "warmup_steps": bench_args.warmup_steps, "measured_steps": bench_args.measured_steps, "seed": args.seed,
        },
        "memory": {"peak_allocated_mb": round(peak_alloc, 2), "peak_reserved_mb": round(peak_res, 2)},
        "timing": {key: compute_statistics([p[key] for p in measured]) for key in TIMING_KEYS} if measured else {},
    }
    if not bench_args.no_per_step:
        results["per_step"] = [{"step": i, **p} for i, p in enumerate(measured)]
    if rank == 0 and bench_args.output:
        out = Path(bench_args.output)
        out.parent.mkdir(parents=True, exist_ok=True)
        out.write_text(json.dumps(results, indent=2))
        print(f"\nResults written to {out}")
        print(format_summary(results))
    del trainer, model
    if on_gpu:
        torch.cuda.empty_cache()
    maybe_destroy_distributed()
    return results


def format_summary(results: dict) -> str:
    lines = [f"\n{'Metric':<16} {'Mean':>10} {'Std':>10} {'Min':>10} {'Max':>10}", "-" * 58]
    for key, s in results["timing"].items():
        lines.append(f"{key:<16} {s['mean']:>10.2f} {s['std']:>10.2f} {s['min']:>10.2f} {s['max']:>10.2f}")
    mem = results["memory"]
    lines.append(f"\nPeak memory: {mem['peak_allocated_mb']:.1f} MB allocated, {mem['peak_reserved_mb']:.1f} MB reserved")
    return "\n".join(lines)


def _dig(doc: dict, dotted: str):
    for part in dotted.split("."):
        if not isinstance(doc, dict):
            return None
        doc = doc.get(part)
    return doc


def _gpu_name(doc: dict) -> str:
    info = doc.get("provenance", {}).get("gpu_info")
    return info[0].get("name", "unknown") if info else "unknown"


def format_comparison(baseline: dict, candidate: dict, baseline_name: str = "baseline", candidate_name: str = "candidate") -> str:
    """Text report: comparability warnings, then timing and memory deltas."""
    lines: list[str] = []
    diffs = [(label, _dig(baseline, key), _dig(candidate, key)) for key, label in _COMPARABILITY]
    diffs = [d for d in diffs if d[1] != d[2]]
    if _gpu_name(baseline) != _gpu_name(candidate):
        diffs.append(("GPU", _gpu_name(baseline), _gpu_name(candidate)))
    if diffs:
        lines.append("COMPARABILITY WARNINGS:")
        lines += [f"  {label}: {a} vs {b}" for label, a, b in diffs]
    for title, doc, name in (("Baseline: ", baseline, baseline_name), ("Candidate:", candidate, candidate_name)):
        lines.append(f"\n{title} {name}")
        lines.append(f"  Git SHA: {doc.get('provenance', {}).get('git_sha', 'unknown')[:12]}")
    w = 26
    lines.append(f"\n{'Metric':<16} {'Baseline (mean +/- std)':<{w}} {'Candidate (mean +/- std)':<{w}} {'Delta':>10} {'Delta %':>10}")
    lines.append("-" * (16 + 2 * w + 22))
    for key in TIMING_KEYS:
        a = baseline.get("timing", {}).get(key, {})
        b = candidate.get("timing", {}).get(key, {})
        am, bm = a.get("mean", 0), b.get("mean", 0)
        delta = bm - am
        pct = delta / am * 100 if am else 0
        lines.append(
            f"{key:<16} {f'{am:>8.2f} +/- {a.get('std', 0):<6.2f}':<{w}} {f'{bm:>8.2f} +/- {b.get('std', 0):<6.2f}':<{w}} "
            f"{delta:>+10.2f} {pct:>+9.1f}%"
        )
    lines.append(f"\n{'Memory':<24} {'Baseline':>12} {'Candidate':>12} {'Delta':>12}")
    lines.append("-" * 62)
    for key in ("peak_allocated_mb", "peak_reserved_mb"):
        a = baseline.get("memory", {}).get(key, 0)
        b = candidate.get("memory", {}).get(key, 0)
        lines.append(f"{key:<24} {a:>9.1f} MB {b:>9.1f} MB {b - a:>+9.1f} MB")
    return "\n".join(lines)


def compare_benchmarks(baseline_path: str, candidate_path: str) -> str:
    report = format_comparison(json.loads(Path(baseline_path).read_text()), json.loads(Path(candidate_path).read_text()),
                               baseline_path, candidate_path)
    print(report)
    return report
