"""Serving-side evaluation helpers: Prometheus parsing, guidellm result parsing, CSV
writer, SPEED-Bench splitting, run planning (no server, no guidellm)."""

import importlib.util
import json
import sys
from pathlib import Path

import pytest

EVAL_DIR = Path(__file__).resolve().parent.parent / "scripts" / "evaluate"


def _load(name):
    sys.path.insert(0, str(EVAL_DIR))
    try:
        spec = importlib.util.spec_from_file_location(f"evaltool_{name}", EVAL_DIR / f"{name}.py")
        mod = importlib.util.module_from_spec(spec)
        sys.modules[spec.name] = mod
        spec.loader.exec_module(mod)
        return mod
    finally:
        sys.path.remove(str(EVAL_DIR))


PAGE_A = """
# HELP vllm:spec_decode_num_drafts_total drafts
vllm:spec_decode_num_drafts_total{engine="0"} 100
vllm:spec_decode_num_draft_tokens_total{engine="0"} 300
vllm:spec_decode_num_accepted_tokens_total{engine="0"} 150
vllm:spec_decode_num_accepted_tokens_per_pos_total{engine="0",position="0"} 80
vllm:spec_decode_num_accepted_tokens_per_pos_total{engine="0",position="1"} 50
vllm:spec_decode_num_accepted_tokens_per_pos_total{engine="0",position="2"} 20
vllm:other_metric 7
"""
PAGE_B = """
vllm:spec_decode_num_drafts_total{engine="0"} 300
vllm:spec_decode_num_draft_tokens_total{engine="0"} 900
vllm:spec_decode_num_accepted_tokens_total{engine="0"} 510
vllm:spec_decode_num_accepted_tokens_per_pos_total{engine="0",position="0"} 260
vllm:spec_decode_num_accepted_tokens_per_pos_total{engine="0",position="1"} 170
vllm:spec_decode_num_accepted_tokens_per_pos_total{engine="0",position="2"} 80
"""

def test_prometheus_delta_and_report():
    pu = _load("perf_utils")
    a, b = pu.parse_prometheus_metrics(PAGE_A), pu.parse_prometheus_metrics(PAGE_B)
    assert (a.num_drafts, a.num_draft_tokens, a.num_accepted_tokens, a.accepted_per_pos) == (100, 300, 150, [80, 50, 20])
    spec = pu.extract_spec_decode_metrics(b, baseline_metrics=a)
    assert spec["num_drafts"] == 200 and spec["acceptance_length"] == pytest.approx(1 + 360 / 200)
    assert spec["acceptance_at_pos_0"] == pytest.approx(0.9) and spec["acceptance_at_pos_2"] == pytest.approx(0.3)
    assert pu.acceptance_csv_columns(spec)[-1] == "acceptance_at_pos_2"
    report = pu.format_acceptance_report(spec)
    assert "Acceptance length" in report and "Position 1" in report
    assert pu.extract_spec_decode_metrics(pu.parse_prometheus_metrics(""))["acceptance_length"] == 0


def _bench(kind, rate, rps, lat):
    stat = lambda v: {"successful": {"median": v, "mean": v, "sum": v * 10}}  # noqa: E731
    return {"config": {"strategy": {"type_": kind, "rate": rate}},
            "metrics": {"requests_per_second": stat(rps), "request_latency": stat(lat), "inter_token_latency_ms": stat(lat * 10),
                        "time_to_first_token_ms": stat(lat * 100), "output_tokens_per_second": stat(1000 / lat), "output_tokens": stat(50)}}


def test_guidellm_parsing_and_csv(tmp_path):
    pu = _load("perf_utils")
    sweep = tmp_path / "run_qa.json"
    sweep.write_text(json.dumps({"benchmarks": [_bench("throughput", "", 9, 3.0), _bench("constant", 2, 2, 1.0), _bench("constant", 4, 4, 1.5)]}))
    rows = pu.parse_sweep_results(sweep, {"acceptance_length": 2.5})
    assert [r["strategy"] for r in rows] == ["constant", "constant"] and rows[0]["subset"] == "qa" and rows[1]["acceptance_length"] == 2.5
    csv_path = tmp_path / "perf.csv"
    writer = pu.CsvWriter(csv_path, pu.BASE_CSV_COLUMNS + ["acceptance_length"])
    writer.append_rows(rows[:1])
    pu.CsvWriter(csv_path, pu.BASE_CSV_COLUMNS + ["acceptance_length"]).append(rows[1])  # resumes without a second header
    assert csv_path.read_text().count("subset,strategy") == 1
    pts = pu.load_data(csv_path, "latency")
    assert pts == {"qa": [(2.0, 1.0), (4.0, 1.5)]}
    gl = tmp_path / "gen_len_qa.json"
    gl.write_text(json.dumps({"benchmarks": [{"requests": {"successful": [{"output_metrics": {"text_tokens": n}} for n in (100, 300, 700)]}}]}))
    assert pu.parse_gen_len_file(gl)["max_tokens"] == 512
    assert pu.parse_gen_len_results([gl, tmp_path / "missing.json"], tmp_path / "mt.json") == {"qa": 512}
    cmd = pu.guidellm_command(target="http://h/v1", dataset="org/ds", subset="qa", data_column_mapper="m", profile="sweep", rate=10,
                              max_requests=200, max_concurrency=64, output_path=tmp_path / "o.json", max_tokens=512, gen_kwargs={"temperature": 0.6})
    assert "kind=sweep,max_concurrency=64,sweep_size=10" in cmd and "extras.body.temperature=0.6" in cmd[cmd.index("--backend") + 1]
    assert "load_kwargs.data_files=qa.jsonl" in cmd[cmd.index("--data") + 1]
    local = pu.guidellm_command(target="t", dataset="/x/f.jsonl", subset=None, data_column_mapper="m", profile="throughput", rate=1,
                                max_requests=None, max_concurrency=1, output_path=tmp_path / "o.json", max_tokens=1)
    assert local[local.index("--data") + 1] == "kind=json_file,path=/x/f.jsonl" and "--constraint" not in local
    with pytest.raises(ValueError):
        pu.parse_gen_kwargs("{bad")
    with pytest.raises(ValueError, match="LABEL=PATH"):
        pu.parse_source_args(["nolabel"])
    x, y = pu.smooth_curve([1, 2, 3, 4, 5], [1.0, 2.1, 2.9, 4.2, 5.0])
    assert len(x) == 300 and abs(y[0] - 1.0) < 0.5


def test_speedbench_split_and_plan(tmp_path):
    sb = _load("prepare_speedbench")
    ev = _load("evaluate")
    rows = [{"turns": "write code", "category": "coding", "sub_category": "x"}, {"messages": [{"content": "sum it"}], "category": "summ ary"},
            {"turns": "", "category": "coding"}]
    (tmp_path / "qualitative.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    (tmp_path / "throughput_1k.jsonl").write_text(json.dumps({"turns": "t", "category": "high_entropy", "sub_category": "code completion"}))
    assert sb.main(["--data-dir", str(tmp_path), "--configs", "qualitative,throughput_1k,throughput_2k"]) == 0
    assert (tmp_path / "qualitative_coding.jsonl").read_text() == json.dumps({"turns": "write code"}) + "\n"
    assert (tmp_path / "qualitative_summ_ary.jsonl").exists() and (tmp_path / "throughput_1k_high_entropy__code_completion.jsonl").exists()
    items = ev.resolve_speedbench("speedbench/qualitative", tmp_path)
    assert [i.label for i in items] == ["speedbench/qualitative/coding", "speedbench/qualitative/summ_ary"] and items[0].hub_subset is None
    items = ev.resolve_speedbench("speedbench/throughput_1k/high_entropy/code_completion", tmp_path)
    assert [i.label for i in items] == ["speedbench/throughput_1k/high_entropy/code_completion"]
    with pytest.raises(FileNotFoundError):
        ev.resolve_speedbench("speedbench/throughput_8k", tmp_path)
    args = ev.build_parser().parse_args(["throughput", "--target", "http://h:8000/v1", "--subsets", "qa, rag"])
    plan = ev.plan_runs(args)
    assert [(p.label, p.hub_subset) for p in plan] == [("qa", "qa"), ("rag", "rag")]
    assert ev.Evaluation(argparse_with(args, output_dir=str(tmp_path / "o"))).metrics_url == "http://h:8000/metrics"
    (tmp_path / "bad.jsonl").write_text(json.dumps({"turns": "x {article}", "category": "c"}))
    with pytest.raises(sb.PlaceholderError):
        sb.split_config(tmp_path / "bad.jsonl", tmp_path, "qualitative")


def argparse_with(ns, **kw):
    for k, v in kw.items():
        setattr(ns, k, v)
    return ns


def test_plot_speedup_curves():
    plot = _load("plot")
    base = [(1, 2.0), (2, 2.4), (3, 3.0), (4, 4.0)]
    fast = [(1, 1.0), (2, 1.2), (3, 1.5), (4, 2.0)]
    x, yb, yt, ratio = plot.speedup_curves(base, fast, increasing=True)
    assert len(x) == 200 and ratio.mean() == pytest.approx(2.0, rel=0.1)
    assert plot.speedup_curves(base, [(10, 1.0), (11, 1.0)], increasing=True) is None
