"""Shared pieces of the serving-side evaluation tools: Prometheus scraping of the
server's speculative-decoding counters, guidellm invocation and result parsing, CSV
output, curve smoothing for the plots.

Reference surface: scripts/evaluate/perf_utils.py (parse_prometheus_metrics:271,
extract_spec_decode_metrics:326, parse_sweep_file:363, run_guidellm:548).
"""

from __future__ import annotations

import csv
import json
import logging
import math
import re
import shutil
import statistics
import subprocess
import sys
import time
from collections import defaultdict
from dataclasses import dataclass, field
from pathlib import Path
from urllib.error import URLError
from urllib.request import urlopen

logger = logging.getLogger("evaluate")

# plot metric -> (CSV column, guidellm JSON key, statistic, axis label, larger-is-worse)
METRICS: dict[str, dict] = {
    "latency": {"csv_col": "latency_median_s", "json_key": "request_latency", "stat": "median", "label": "Median Latency (s)", "increasing": True},
    "itl": {"csv_col": "itl_median_ms", "json_key": "inter_token_latency_ms", "stat": "median", "label": "Median ITL (ms)", "increasing": True},
    "ttft": {"csv_col": "ttft_median_ms", "json_key": "time_to_first_token_ms", "stat": "median", "label": "Median TTFT (ms)", "increasing": True},
    "output_tps": {"csv_col": "output_tps_median", "json_key": "output_tokens_per_second", "stat": "median", "label": "Output Tokens/s", "increasing": False},
}
PRETTY_SUBSET_NAMES = {
    "HumanEval": "HumanEval", "math_reasoning": "Math Reasoning", "qa": "QA", "question": "Question", "rag": "RAG",
    "summarization": "Summarization", "tool_call": "Tool Call", "translation": "Translation", "writing": "Writing",
}
SWEEP_FIELDS = (
    ("requests_per_second", "rps_median"), ("request_latency", "latency_median_s"), ("inter_token_latency_ms", "itl_median_ms"),
    ("time_to_first_token_ms", "ttft_median_ms"), ("output_tokens_per_second", "output_tps_median"),
)
SKIP_STRATEGIES = frozenset({"throughput"})
BASE_CSV_COLUMNS = ["subset", "strategy", "target_rate", *[c for _, c in SWEEP_FIELDS], "total_output_tokens"]
_SPEC_PREFIX = "vllm:spec_decode"
_LINE = re.compile(r"^([a-zA-Z_:][a-zA-Z0-9_:]*)(?:\{([^}]*)\})?\s+([0-9.eE+-]+|NaN|[+-]?Inf)$")
_POSITION = re.compile(r'position="(\d+)"')


# ----------------------------------------------------------------------------- prometheus
@dataclass
class SpecDecodeCounters:
    """Totals of the server's speculative-decoding counters at one scrape."""

    num_drafts: float = 0.0
    num_draft_tokens: float = 0.0
    num_accepted_tokens: float = 0.0
    accepted_per_pos: list[float] = field(default_factory=list)

    def minus(self, other: "SpecDecodeCounters") -> "SpecDecodeCounters":
        n = max(len(self.accepted_per_pos), len(other.accepted_per_pos))
        pad = lambda xs: xs + [0.0] * (n - len(xs))  # noqa: E731
        return SpecDecodeCounters(
            self.num_drafts - other.num_drafts, self.num_draft_tokens - other.num_draft_tokens,
            self.num_accepted_tokens - other.num_accepted_tokens,
            [a - b for a, b in zip(pad(self.accepted_per_pos), pad(other.accepted_per_pos))],
        )


def parse_prometheus_metrics(raw_text: str) -> SpecDecodeCounters:
    """Sum the ``vllm:spec_decode_*`` series of a ``/metrics`` page (over engines /
    label sets); ``*_per_pos`` series are gathered by their ``position`` label."""
    out = SpecDecodeCounters()
    per_pos: dict[int, float] = defaultdict(float)
    for raw in (raw_text or "").splitlines():
        line = raw.strip()
        if not line or line.startswith("#"):
            continue
        m = _LINE.match(line)
        if not m or _SPEC_PREFIX not in m.group(1):
            continue
        name, labels, value = m.group(1).replace("_total", ""), m.group(2) or "", float(m.group(3))
        if "per_pos" in name:
            pos = _POSITION.search(labels)
            if pos:
                per_pos[int(pos.group(1))] += value
        elif name.endswith("num_drafts"):
            out.num_drafts += value
        elif name.endswith("num_draft_tokens"):
            out.num_draft_tokens += value
        elif name.endswith("num_accepted_tokens"):
            out.num_accepted_tokens += value
    if per_pos:
        out.accepted_per_pos = [per_pos.get(i, 0.0) for i in range(max(per_pos) + 1)]
    return out


def extract_spec_decode_metrics(current: SpecDecodeCounters, baseline_metrics: SpecDecodeCounters | None = None) -> dict[str, float]:
    """Acceptance length (1 + accepted / drafts) and per-position acceptance rates of
    the interval between two scrapes."""
    c = current.minus(baseline_metrics) if baseline_metrics is not None else current
    d = c.num_drafts
    result = {
        "num_drafts": d, "num_draft_tokens": c.num_draft_tokens, "num_accepted_tokens": c.num_accepted_tokens,
        "acceptance_length": 1 + c.num_accepted_tokens / d if d > 0 else 0,
    }
    for i, count in enumerate(c.accepted_per_pos):
        result[f"acceptance_at_pos_{i}"] = count / d if d > 0 else 0
    return result


def load_prometheus_file(path: Path | None) -> SpecDecodeCounters:
    return parse_prometheus_metrics(path.read_text()) if path and path.exists() else SpecDecodeCounters()


def fetch_metrics(metrics_url: str, retries: int = 3, delay: float = 2.0) -> str | None:
    for attempt in range(1, retries + 1):
        try:
            with urlopen(metrics_url, timeout=30) as resp:  # noqa: S310
                return resp.read().decode()
        except (URLError, OSError) as err:
            logger.warning("Failed to fetch metrics from %s (attempt %d/%d): %s", metrics_url, attempt, retries, err)
            if attempt < retries:
                time.sleep(delay)
    return None


def acceptance_csv_columns(spec: dict[str, float]) -> list[str]:
    cols = ["num_drafts", "num_draft_tokens", "num_accepted_tokens", "acceptance_length"]
    pos = 0
    while f"acceptance_at_pos_{pos}" in spec:
        cols.append(f"acceptance_at_pos_{pos}")
        pos += 1
    return cols


def format_acceptance_report(spec: dict[str, float]) -> str:
    lines = ["", "=== Speculative Decoding Acceptance Report ===", ""]
    for label, key, fmt in (("Num drafts", "num_drafts", ".0f"), ("Num draft tokens", "num_draft_tokens", ".0f"),
                            ("Num accepted tokens", "num_accepted_tokens", ".0f"), ("Acceptance length", "acceptance_length", ".4f")):
        lines.append(f"  {label:<25} {format(spec.get(key, 0), fmt):>12}")
    cols = [c for c in acceptance_csv_columns(spec) if c.startswith("acceptance_at_pos_")]
    if cols:
        lines += ["", f"  {'Position':<25} {'Acceptance Rate':>12}", f"  {'-' * 25} {'-' * 12}"]
        lines += [f"  {'Position ' + c.rsplit('_', 1)[1]:<25} {spec[c]:>12.4f}" for c in cols]
    lines.append("")
    return "\n".join(lines)


def print_acceptance_report(spec: dict[str, float]) -> None:
    print(format_acceptance_report(spec))


# ----------------------------------------------------------------------------- guidellm results
def _subset_of(path: Path) -> str:
    m = re.search(r"(?:gen_len|sweeps?|run)_(.+)\.json$", path.name)
    return m.group(1) if m else path.stem


def parse_gen_len_file(path: Path) -> dict:
    """Output-length statistics of a throughput run; ``max_tokens`` = median rounded up
    to a power of two (the cap used for the sweep that follows)."""
    data = json.loads(path.read_text())
    benches = data.get("benchmarks") or []
    if not benches:
        raise ValueError(f"No benchmarks found in {path}")
    done = benches[0].get("requests", {}).get("successful") or []
    if not done:
        raise ValueError(f"No successful requests found in {path}")
    lens = [r["output_metrics"]["text_tokens"] for r in done]
    med = statistics.median(lens)
    return {"count": len(lens), "median": med, "min": min(lens), "max": max(lens), "max_tokens": 2 ** math.ceil(math.log2(max(med, 1)))}


def parse_gen_len_results(files: list[Path], output: Path) -> dict[str, int]:
    print(f"{'Subset':<20} {'Count':>6} {'Median':>8} {'Min':>8} {'Max':>8} {'max_tokens':>12}")
    print("-" * 70)
    mapping: dict[str, int] = {}
    for path in files:
        try:
            s = parse_gen_len_file(path)
        except (FileNotFoundError, ValueError, KeyError, json.JSONDecodeError) as err:
            logger.warning("Skipping %s: %s", path, err)
            continue
        mapping[_subset_of(path)] = s["max_tokens"]
        print(f"{_subset_of(path):<20} {s['count']:>6} {s['median']:>8.0f} {s['min']:>8} {s['max']:>8} {s['max_tokens']:>12}")
    if not mapping:
        logger.error("No files were successfully parsed")
        sys.exit(1)
    output.parent.mkdir(parents=True, exist_ok=True)
    output.write_text(json.dumps(mapping, indent=2))
    return mapping


def parse_sweep_file(path: Path) -> list[dict]:
    data = json.loads(path.read_text())
    benches = data.get("benchmarks") or []
    if not benches:
        raise ValueError(f"No benchmarks found in {path}")
    rows = []
    for bench in benches:
        strategy = bench.get("config", {}).get("strategy", {})
        kind = strategy.get("type_", "unknown")
        if kind in SKIP_STRATEGIES:
            continue
        metrics = bench.get("metrics", {})
        row = {"subset": _subset_of(path), "strategy": kind, "target_rate": strategy.get("rate", "")}
        for key, col in SWEEP_FIELDS:
            row[col] = metrics.get(key, {}).get("successful", {}).get("median", "")
        row["total_output_tokens"] = metrics.get("output_tokens", {}).get("successful", {}).get("sum", "")
        rows.append(row)
    return rows


def parse_sweep_results(path: Path, spec_decode_metrics: dict[str, float] | None = None) -> list[dict]:
    rows = parse_sweep_file(path)
    for row in rows:
        row.update(spec_decode_metrics or {})
    return rows


class CsvWriter:
    """Appends rows to a CSV file; the header goes out with the first row."""

    def __init__(self, path: Path, columns: list[str]):
        self.path, self.columns = Path(path), columns
        self._started = self.path.exists()

    def append(self, row: dict) -> None:
        self.append_rows([row])

    def append_rows(self, rows: list[dict]) -> None:
        if not rows:
            return
        self.path.parent.mkdir(parents=True, exist_ok=True)
        with self.path.open("a" if self._started else "w", newline="") as fh:
            writer = csv.DictWriter(fh, fieldnames=self.columns, extrasaction="ignore")
            if not self._started:
                writer.writeheader()
                self._started = True
            writer.writerows(rows)


# ----------------------------------------------------------------------------- guidellm runs
def check_dependencies() -> None:
    if not shutil.which("guidellm"):
        logger.error("Missing required dependency: guidellm (pip install -r scripts/evaluate/requirements.txt)")
        sys.exit(1)


def parse_gen_kwargs(text: str) -> dict:
    if not text:
        return {}
    try:
        return json.loads(text)
    except json.JSONDecodeError as err:
        raise ValueError(f"Invalid JSON in --gen-kwargs: {text!r}: {err}") from err


def guidellm_command(target: str, dataset: str, subset: str | None, data_column_mapper: str, profile: str, rate: int | str,
                     max_requests: int | None, max_concurrency: int, output_path: Path, max_tokens: int,
                     gen_kwargs: dict | None = None) -> list[str]:
    """``guidellm run`` argv.  ``subset`` set: ``dataset`` is a hub dataset and the
    subset its ``<subset>.jsonl`` file; ``subset`` None: ``dataset`` is a local JSONL."""
    backend = f"kind=openai_http,target={target},max_tokens={max_tokens}" + "".join(
        f",extras.body.{k}={v}" for k, v in (gen_kwargs or {}).items()
    )
    data = (f"kind=huggingface,source={dataset},load_kwargs.data_files={subset}.jsonl,load_kwargs.split=train"
            if subset is not None else f"kind=json_file,path={dataset}")
    prof = f"kind={profile},max_concurrency={max_concurrency}" + (f",sweep_size={rate}" if profile == "sweep" else "")
    cmd = ["guidellm", "run", "--backend", backend, "--data", data, "--data-column-mapper", data_column_mapper, "--profile", prof]
    if max_requests is not None:
        cmd += ["--constraint", f"kind=max_requests,count={max_requests}"]
    return [*cmd, "--output", f"kind=json,path={output_path}"]


def run_guidellm(**kwargs) -> None:
    subprocess.run(guidellm_command(**kwargs), check=True)  # noqa: S603


# ----------------------------------------------------------------------------- plot inputs
def _points_from_csv(path: Path, metric: str) -> dict[str, list[tuple[float, float]]]:
    col = METRICS[metric]["csv_col"]
    out: dict[str, list[tuple[float, float]]] = defaultdict(list)
    with path.open(newline="") as fh:
        for row in csv.DictReader(fh):
            if row.get("strategy") != "constant":
                continue
            try:
                out[re.sub(r"^run_", "", row.get("subset", "unknown"))].append((float(row["rps_median"]), float(row[col])))
            except (ValueError, KeyError):
                continue
    return dict(out)


def _points_from_json(path: Path, metric: str) -> dict[str, list[tuple[float, float]]]:
    cfg = METRICS[metric]
    data = json.loads(path.read_text())
    subset = Path(data["config"]["spec"]["data"][0]["load_kwargs"]["data_files"]).stem
    pts = []
    for bench in data.get("benchmarks", []):
        if bench.get("config", {}).get("strategy", {}).get("type_") != "constant":
            continue
        try:
            pts.append((bench["metrics"]["requests_per_second"]["successful"]["mean"],
                        bench["metrics"][cfg["json_key"]]["successful"][cfg["stat"]]))
        except (KeyError, TypeError):
            continue
    return {subset: sorted(pts)} if pts else {}


def load_data(path: Path, metric: str) -> dict[str, list[tuple[float, float]]]:
    """``{subset: [(requests/s, metric value), ...]}`` of the constant-rate points."""
    if path.suffix == ".csv":
        return _points_from_csv(path, metric)
    if path.suffix == ".json":
        return _points_from_json(path, metric)
    raise ValueError(f"Unsupported file type: {path.suffix} (expected .csv or .json)")


def parse_source_args(source_args: list[str]) -> dict[str, list[Path]]:
    """``LABEL=PATH`` (repeatable; equal labels pool repetitions) -> ``{label: [paths]}``."""
    out: dict[str, list[Path]] = defaultdict(list)
    for arg in source_args:
        if "=" not in arg:
            raise ValueError(f"Invalid source format: '{arg}'. Expected 'LABEL=PATH'.")
        label, path = arg.rsplit("=", 1)
        if not Path(path.strip()).exists():
            raise FileNotFoundError(f"File not found: {path.strip()}")
        out[label.strip()].append(Path(path.strip()))
    return dict(out)


def smooth_curve(x, y, n_dense: int = 300):
    """Smoothing spline through noisy (x, y); falls back to linear interpolation
    when scipy is missing."""
    import numpy as np

    x, y = np.asarray(x, dtype=float), np.asarray(y, dtype=float)
    order = np.argsort(x)
    x, y = x[order], y[order]
    if len(x) < 2:
        return x, y
    dense = np.linspace(x.min(), x.max(), n_dense)
    try:
        from scipy.interpolate import UnivariateSpline

        return dense, UnivariateSpline(x, y, k=min(3, len(x) - 1), s=len(x) * np.var(y))(dense)
    except ImportError:
        return dense, np.interp(dense, x, y)


def pretty_subset(name: str) -> str:
    return PRETTY_SUBSET_NAMES.get(name, name)
