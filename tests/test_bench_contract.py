"""The benchmark's two arms must be independent: the reference arm may not load this
package (its inputs come from files written by a plain-PyTorch module), and both arms
must describe the measured configuration with the same record."""

import argparse
import json
import os
import re
import subprocess
import sys

import torch

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_bench_inputs_is_plain_torch():
    src = open(os.path.join(REPO, "bench_inputs.py")).read()
    imported = set(re.findall(r"^\s*(?:from|import)\s+([\w\.]+)", src, flags=re.M))
    assert not any(name.split(".")[0] in ("speculators_b200", "speculators", "hs_connectors") for name in imported), imported


def test_reference_arm_never_imports_the_package():
    code = (
        "import sys, bench\n"
        "sys.argv = ['bench.py', '--impl', 'reference', '--model', 'tiny']\n"
        "bench.run_reference(bench.parse_args())\n"
        "leaked = [m for m in sys.modules if m.split('.')[0] == 'speculators_b200']\n"
        "assert not leaked, leaked\n"
    )
    out = subprocess.run([sys.executable, "-c", code], cwd=REPO, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1]
    rec = json.loads(line)
    assert rec["impl"] == "reference"
    # no GPU here: the arm says why it cannot run (or, on a GPU box, prints its record)
    assert "unavailable" in rec or "value" in rec


def test_both_arms_print_the_same_config_record():
    sys.path.insert(0, REPO)
    import bench

    args = argparse.Namespace(model="llama31_8b", config=None, seq_len=None, ttt_steps=None, regions=5, draft_vocab=None, no_verifier_forward=False, scale="full")
    c = bench.resolve_config(args)
    assert c["name"] == "eagle3" and c["seq_len"] == 2048 and c["draft_vocab"] == 32000 and c["metric"] == bench.METRIC
    a = bench.config_record(c, 8, 5)
    assert a["parallelism"] == "dp8-sharded" and a["global_batch"] == 8 and a["algorithm"] == "eagle3"
    src = open(os.path.join(REPO, "bench.py")).read()
    assert src.count('"config": config_record(c, world, args.regions)') == 2  # one expression, both arms
    for name in ("dflash", "dspark", "peagle"):
        args.config = name
        assert bench.resolve_config(args)["algo"] == name


def test_seeded_init_depends_on_names_only():
    sys.path.insert(0, REPO)
    import bench_inputs

    shapes = {"fc.weight": (8, 24), "layers.0.mlp.up_proj.weight": (16, 8), "norm.weight": (8,), "lm_head.weight": (32, 8), "d2t": (32,)}
    a = bench_inputs.seeded_draft_init(shapes)
    b = bench_inputs.seeded_draft_init(dict(reversed(list(shapes.items()))))
    assert set(a) == {"fc.weight", "layers.0.mlp.up_proj.weight", "norm.weight"}
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert torch.equal(a["norm.weight"], torch.ones(8))


def test_loss_parity_rule():
    sys.path.insert(0, REPO)
    import bench

    assert bench.loss_parity([1.0, 0.9], None)["loss_parity"] is None
    assert bench.loss_parity([1.0, 0.9], [1.01, 0.905])["loss_parity"] is True
    assert bench.loss_parity([1.0, 0.9], [1.2, 0.9])["loss_parity"] is False
