"""The device-side timeline: kernels compiled with TESSWEAVE_TIMELINE=1 record every block's start, the end of
its wait for the kernel before it, and its end.  Run in a child process, since the switch must be set before the
first kernel library is loaded; only the two small libraries the script touches are compiled with the recorder."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

SCRIPT = r"""
import torch
from tessweave_engine_b200.csrc import ops
from tessweave_engine_b200.engine.timeline import Timeline, format_launches
tl = Timeline(capacity=4096)
logits = torch.randn(5, 1000, device="cuda")
ids = torch.zeros(5, dtype=torch.int32, device="cuda")
ops.sample(ids, logits, 5)
assert ids.tolist() == logits.argmax(-1).tolist()
tl.reset()
ops.sample(ids, logits, 5)
x = torch.randn(3, 256, device="cuda", dtype=torch.bfloat16)
w = torch.randn(64, 256, device="cuda", dtype=torch.bfloat16)
out = torch.empty(3, 64, device="cuda", dtype=torch.bfloat16)
ops.gemm_small_m(out, x, w, 3)
rows = tl.launches()
print(format_launches(rows))
assert [(r["kernel"], r["blocks"], r["seen"]) for r in rows] == [("sample", 5, 5), ("gemm_smallm", 1, 1)], rows
assert all(r["end"] > r["start"] >= 0 and r["first_end"] <= r["end"] for r in rows)
assert rows[1]["gap"] is not None and rows[1]["start"] >= rows[0]["start"]
tl.close()
ops.sample(ids, logits, 5)             # without a buffer the recorder writes nothing and the kernels still run
torch.cuda.synchronize()
assert ids.tolist() == logits.argmax(-1).tolist()
print("timeline ok")
"""


def test_timeline_records_the_blocks_of_each_launch():
    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, TESSWEAVE_TIMELINE="1", PYTHONPATH=str(root) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    done = subprocess.run([sys.executable, "-c", SCRIPT], env=env, cwd=root, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stdout + done.stderr
    assert "timeline ok" in done.stdout


def test_timeline_needs_the_switch():
    from tessweave_engine_b200.engine.timeline import Timeline
    if os.environ.get("TESSWEAVE_TIMELINE") == "1":
        pytest.skip("the switch is on in this process")
    with pytest.raises(RuntimeError, match="TESSWEAVE_TIMELINE"):
        Timeline()
