#!/usr/bin/env python3
"""Training benchmark harness (real Trainer, per-step phase timings, peak memory,
provenance; JSON results that can be compared across code changes).

    # synthetic data, no dataset or server needed
    python scripts/benchmark.py run --synthetic -- --verifier-name-or-path Qwen/Qwen3-8B --total-seq-len 4096
    # several GPUs
    torchrun --standalone --nproc_per_node 2 scripts/benchmark.py run --synthetic -- --verifier-name-or-path Qwen/Qwen3-8B
    # compare two result files
    python scripts/benchmark.py compare baseline.json candidate.json

Training flags (the ones ``scripts/train.py`` takes) go after ``--``.
CLI parity: scripts/benchmark.py:588 of the reference.
"""

from __future__ import annotations

import os as _os
import sys as _sys

_REPO_ROOT = _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))
if _REPO_ROOT not in _sys.path:  # run from a checkout without installing the package
    _sys.path.insert(0, _REPO_ROOT)

import argparse
import sys
from datetime import datetime

from speculators_b200.train.benchmark import (  # noqa: F401  (re-exported: the harness is importable as this script)
    ProfileCapture, collect_provenance, compare_benchmarks, compute_statistics, create_synthetic_batch, run_benchmark,
)
from speculators_b200.train.synthetic import SyntheticLoader
from speculators_b200.train.config import TrainConfig

_MetricCapture = ProfileCapture  # the reference script's private names for the same two helpers
_SyntheticLoader = SyntheticLoader


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Training benchmark harness.", formatter_class=argparse.RawDescriptionHelpFormatter,
                                 epilog="Pass train.py flags after '--'.")
    sub = ap.add_subparsers(dest="command", required=True)
    run = sub.add_parser("run", help="run a training benchmark")
    run.add_argument("--synthetic", action="store_true", help="random data instead of a dataset")
    run.add_argument("--warmup-steps", type=int, default=10)
    run.add_argument("--measured-steps", type=int, default=50)
    run.add_argument("--output", default=None, help="default: benchmark_<timestamp>.json")
    run.add_argument("--no-per-step", action="store_true", help="leave per-step timings out of the JSON")
    cmp_ = sub.add_parser("compare", help="compare two result files")
    cmp_.add_argument("baseline")
    cmp_.add_argument("candidate")
    return ap


def main(argv: list[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    train_argv: list[str] = []
    if "--" in argv:
        cut = argv.index("--")
        argv, train_argv = argv[:cut], argv[cut + 1:]
    bench_args = build_parser().parse_args(argv)
    if bench_args.command == "compare":
        compare_benchmarks(bench_args.baseline, bench_args.candidate)
        return 0
    if bench_args.output is None:
        bench_args.output = f"benchmark_{datetime.now():%Y%m%d_%H%M%S}.json"
    run_benchmark(bench_args, argparse.Namespace(**TrainConfig.resolve(train_argv).flatten()))
    return 0


if __name__ == "__main__":
    sys.exit(main())
