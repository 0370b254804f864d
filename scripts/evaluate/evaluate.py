#!/usr/bin/env python3
"""Serving-side evaluation of a speculator: acceptance rates and latency/throughput
curves of a running server, measured with guidellm and the server's Prometheus counters.

    python evaluate.py --target http://localhost:8000/v1 throughput      # acceptance rates at max rate
    python evaluate.py --target http://localhost:8000/v1 sweep           # gen-len probe, rate sweep, CSVs
    python evaluate.py --target http://localhost:8000/v1 sweep --subsets "HumanEval,qa" --gen-kwargs '{"temperature":0.6}'
    python evaluate.py --target http://localhost:8000/v1 throughput --dataset speedbench/qualitative/coding \\
        --speedbench-data-dir ./speedbench_data                          # after prepare_speedbench.py

Outputs in ``--output-dir``: ``acceptance.csv``, ``perf_results.csv`` and
``max_tokens.json`` (sweep), ``eval_command.txt``, raw guidellm JSON under ``artifacts/``.
CLI parity: scripts/evaluate/evaluate.py:364 of the reference.
"""

from __future__ import annotations

import os as _os
import sys as _sys

_REPO_ROOT = _os.path.dirname(_os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))
if _REPO_ROOT not in _sys.path:  # run from a checkout without installing the package
    _sys.path.insert(0, _REPO_ROOT)

import argparse
import json
import logging
import shlex
import sys
from dataclasses import dataclass
from datetime import datetime, timezone
from pathlib import Path
from urllib.error import URLError
from urllib.request import urlopen

sys.path.insert(0, str(Path(__file__).resolve().parent))
import perf_utils as pu  # noqa: E402

logger = logging.getLogger("evaluate")

DEFAULT_DATASET = "RedHatAI/speculator_benchmarks"
DEFAULT_SUBSETS = "HumanEval,math_reasoning,qa,question,rag,summarization,tool_call,translation,writing"
PROMPT_MAPPER = "kind=generative_column_mapper,column_mappings.text_column=prompt"
SPEEDBENCH_MAPPER = "kind=generative_column_mapper,column_mappings.text_column=turns"


@dataclass
class RunItem:
    label: str  # names output files and the CSV row
    dataset: str  # hub dataset id, or a local JSONL file
    mapper: str

    @property
    def hub_subset(self) -> str | None:
        return None if Path(self.dataset).exists() else self.label

    @property
    def safe(self) -> str:
        return self.label.replace("/", "_").replace(" ", "_")


def served_model_name(target: str) -> str | None:
    base = target.rstrip("/")
    base = base if base.endswith("/v1") else base + "/v1"
    try:
        with urlopen(f"{base}/models", timeout=10) as resp:  # noqa: S310
            models = json.loads(resp.read()).get("data", [])
        return models[0].get("id") if models else None
    except (URLError, json.JSONDecodeError, OSError) as err:
        logger.warning("Could not fetch model name from %s/models: %s", base, err)
        return None


def save_eval_provenance(output_dir: Path) -> None:
    """``eval_command.txt``: time, git revision, package versions, command line (best effort)."""
    try:
        from speculators_b200.provenance import atomic_write, git_sha, package_versions

        head = [f"# Timestamp: {datetime.now(timezone.utc).isoformat()}", f"# Git SHA: {git_sha()}"]
        head += package_versions()
        atomic_write(output_dir / "eval_command.txt", "\n".join(head) + f"\n{shlex.join(sys.argv)}\n")
    except Exception:  # noqa: BLE001
        logger.warning("Failed to save eval_command.txt", exc_info=True)


def resolve_speedbench(spec: str, data_dir: Path) -> list[RunItem]:
    """``speedbench/<config>[/<category>[/<subcategory>]]`` -> the matching files written
    by ``prepare_speedbench.py`` (``<config>_<category>[__<subcategory>].jsonl``)."""
    config, *rest = spec.removeprefix("speedbench/").split("/")
    suffix = "" if not rest else rest[0] if len(rest) == 1 else rest[0] + "__" + "_".join(rest[1:])
    pattern = f"{config}_{suffix}*.jsonl"
    files = sorted(data_dir.glob(pattern))
    if not files:
        raise FileNotFoundError(f"--speedbench-data-dir='{data_dir}': no files matching '{pattern}'. Run prepare_speedbench.py first.")
    return [RunItem(f"speedbench/{config}/{p.stem.removeprefix(config + '_').replace('__', '/')}", str(p), SPEEDBENCH_MAPPER) for p in files]


def plan_runs(args: argparse.Namespace) -> list[RunItem]:
    if args.dataset.startswith("speedbench/"):
        if not args.speedbench_data_dir:
            raise ValueError("--speedbench-data-dir is required for speedbench/ datasets (run prepare_speedbench.py first).")
        return resolve_speedbench(args.dataset, Path(args.speedbench_data_dir))
    return [RunItem(s.strip(), args.dataset, args.data_column_mapper) for s in args.subsets.split(",") if s.strip()]


class Evaluation:
    def __init__(self, args: argparse.Namespace):
        self.args = args
        self.sweep = args.mode == "sweep"
        self.metrics_url = args.target.rstrip("/").removesuffix("/v1") + "/metrics"
        self.out = Path(args.output_dir)
        self.artifacts = self.out / "artifacts"
        self.acceptance_csv: pu.CsvWriter | None = None
        self.perf_csv: pu.CsvWriter | None = None
        self.max_tokens: dict[str, int] = {}

    def _scrape(self) -> pu.SpecDecodeCounters:
        text = pu.fetch_metrics(self.metrics_url)
        if text is None:
            raise RuntimeError(f"Failed to fetch metrics from {self.metrics_url}")
        return pu.parse_prometheus_metrics(text)

    def _guidellm(self, item: RunItem, **kw) -> None:
        pu.run_guidellm(target=self.args.target, dataset=item.dataset, subset=item.hub_subset, data_column_mapper=item.mapper,
                        max_concurrency=self.args.max_concurrency, gen_kwargs=pu.parse_gen_kwargs(self.args.gen_kwargs), **kw)

    def run_item(self, item: RunItem) -> None:
        logger.info("[%s] Starting", item.label)
        a = self.args
        max_tokens = 4096
        if self.sweep:  # probe output lengths first, cap the sweep's max_tokens by the median
            probe_dir = self.artifacts / "gen_len"
            probe_dir.mkdir(parents=True, exist_ok=True)
            probe = probe_dir / f"gen_len_{item.safe}.json"
            self._guidellm(item, profile="throughput", rate=a.gen_len_rate, max_requests=None, output_path=probe, max_tokens=4096)
            mapping = pu.parse_gen_len_results([probe], probe_dir / f"max_tokens_{item.safe}.json")
            max_tokens = mapping.get(item.hub_subset or item.safe, max_tokens)
            self.max_tokens[item.label] = max_tokens
            logger.info("[%s] max_tokens=%d", item.label, max_tokens)
        before = self._scrape()
        run_json = self.artifacts / f"run_{item.safe}.json"
        self._guidellm(item, profile="sweep" if self.sweep else "throughput", rate=a.sweep_rate if self.sweep else a.gen_len_rate,
                       max_requests=a.max_requests, output_path=run_json, max_tokens=max_tokens)
        spec = pu.extract_spec_decode_metrics(self._scrape(), baseline_metrics=before)
        has_spec = spec.get("num_drafts", 0) > 0
        if has_spec:
            spec["subset"] = item.label
            pu.print_acceptance_report(spec)
            if self.acceptance_csv is None:
                self.acceptance_csv = pu.CsvWriter(self.out / "acceptance.csv", ["subset", *pu.acceptance_csv_columns(spec)])
            self.acceptance_csv.append(spec)
        else:
            logger.warning("[%s] No speculative decoding metrics found", item.label)
        if self.sweep:
            rows = pu.parse_sweep_results(run_json, spec if has_spec else None)
            if rows and self.perf_csv is None:
                self.perf_csv = pu.CsvWriter(self.out / "perf_results.csv", pu.BASE_CSV_COLUMNS + (pu.acceptance_csv_columns(spec) if has_spec else []))
            if rows:
                self.perf_csv.append_rows(rows)
        logger.info("[%s] Complete", item.label)

    def run(self) -> int:
        pu.check_dependencies()
        self.artifacts.mkdir(parents=True, exist_ok=True)
        save_eval_provenance(self.out)
        items = plan_runs(self.args)
        logger.info("Mode: %s | %d subsets | Output: %s", self.args.mode, len(items), self.out)
        for item in items:
            self.run_item(item)
        if self.acceptance_csv is None:
            logger.error("No acceptance metrics collected from any subset")
            return 1
        if self.sweep and self.max_tokens:
            (self.out / "max_tokens.json").write_text(json.dumps(self.max_tokens, indent=2))
        logger.info("Benchmarking complete! Results: %s", self.out)
        return 0


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="evaluate", description="Speculative decoding performance evaluation toolkit.")
    ap.add_argument("mode", choices=["throughput", "sweep"], help="throughput: max-rate run for acceptance rates; sweep: full pipeline")
    ap.add_argument("--target", required=True, help="server endpoint, e.g. http://localhost:8000/v1")
    ap.add_argument("--dataset", default=DEFAULT_DATASET, help="hub dataset id, local directory, or speedbench/<config>[/...]")
    ap.add_argument("--subsets", default=DEFAULT_SUBSETS, help="comma-separated subset names")
    ap.add_argument("--output-dir", default=None, help="default: <served model>_<timestamp>")
    ap.add_argument("--max-concurrency", type=int, default=128)
    ap.add_argument("--max-requests", type=int, default=200, help="requests per sweep point")
    ap.add_argument("--gen-len-rate", type=int, default=128, help="request rate of the output-length probe")
    ap.add_argument("--sweep-rate", type=int, default=10, help="number of rate points in the sweep")
    ap.add_argument("--gen-kwargs", default="", help='flat JSON of generation parameters, e.g. \'{"temperature":0.6}\'')
    ap.add_argument("--data-column-mapper", default=PROMPT_MAPPER)
    ap.add_argument("--speedbench-data-dir", default=None, help="directory prepared by prepare_speedbench.py")
    return ap


def main(argv: list[str] | None = None) -> int:
    logging.basicConfig(level=logging.INFO, format="[%(levelname)s] %(message)s", stream=sys.stderr)
    args = build_parser().parse_args(argv)
    if args.output_dir is None:
        name = served_model_name(args.target)
        stamp = datetime.now().strftime("%Y%m%d_%H%M%S")
        args.output_dir = f"{name.replace('/', '_').replace(' ', '_')}_{stamp}" if name else f"perf_results_{stamp}"
    try:
        return Evaluation(args).run()
    except (ValueError, FileNotFoundError, RuntimeError) as err:
        logger.error("%s", err)
        return 1


if __name__ == "__main__":
    sys.exit(main())
