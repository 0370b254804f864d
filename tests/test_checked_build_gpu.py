"""Debug flavour of the extension (-DSB200_CHECK_BOUNDS): a bad data-dependent row index is
recorded and its access skipped instead of reaching memory.  Runs in a child process that
loads ``_sb200_checked.so`` and verifies that before it passes any bad index."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

from speculators_b200.ops import _build

pytestmark = pytest.mark.gpu

CHILD = r"""
import json, torch
from speculators_b200 import ops
nat = ops.native()
assert nat.checked_build(), "the debug flavour must be the one loaded"
x = torch.randn(16, 64, device="cuda").bfloat16()
w = torch.ones(64, device="cuda").bfloat16()
idx = torch.tensor([0, 3, 99, 5], device="cuda")  # 99 is outside the 16 rows of x
y = torch.zeros(4, 64, device="cuda").bfloat16()
nat.rmsnorm_fwd(x, w, idx, y, None, 1e-6)
torch.cuda.synchronize()
first = nat.bounds_report().tolist()
second = nat.bounds_report().tolist()
ok_rows = bool((y[[0, 1, 3]].float().abs().sum(-1) > 0).all())
print(json.dumps({"first": first, "second": second, "skipped_row_untouched": bool((y[2] == 0).all()), "other_rows_written": ok_rows}))
"""


def test_bad_gather_index_is_recorded_and_skipped():
    if not _build.LIB_CHECKED.exists():
        pytest.skip("debug flavour not built: python -m speculators_b200.ops._build --checked")
    env = dict(os.environ, SB200_CHECKED_BUILD="1", PYTHONPATH=str(Path(__file__).resolve().parents[1]))
    proc = subprocess.run([sys.executable, "-c", CHILD], capture_output=True, text=True, env=env, timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    res = json.loads(proc.stdout.strip().splitlines()[-1])
    assert res["first"][0] == [1, 99, 16]  # site 1 = rmsnorm gather row, index 99, limit 16
    assert res["second"][0] == [0, 0, 0]  # reading clears the record
    assert res["skipped_row_untouched"] and res["other_rows_written"]
