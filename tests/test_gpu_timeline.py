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
assert [(r["kernel"], r["blocks"], r["seen"]) for r in rows] == [("sample", 40, 40), ("gemm_smallm", 1, 1)], rows      # eight blocks share a greedy row
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


def test_kernel_table_runs_the_parts_own_routes():
    """The per-operation table is made by calling the parts of a model's spec, and names the kernels from the
    launch log: at four rows the products run on the small-batch kernel, the attention of a decode step on the
    kernel fed by TMA (head size 64), and every row carries a positive time and a roofline fraction."""
    import tessweave_engine_b200 as tw
    from tessweave_engine_b200.engine.kernel_bench import format_table, kernel_table
    config = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "vocab_size": 2048, "hidden_size": 512,
              "intermediate_size": 1408, "num_hidden_layers": 1, "num_attention_heads": 8, "num_key_value_heads": 2,
              "head_dim": 64, "rope_theta": 1e4, "rms_norm_eps": 1e-6, "max_position_embeddings": 4096,
              "tie_word_embeddings": False, "use_sliding_window": False, "hidden_act": "silu"}
    _, spec = tw.resolve(config)
    rows = kernel_table(spec, 4, 320, 192, 6456.5, 1657.4, page_size=16)
    by_op = {r["op"]: r for r in rows}
    assert len(rows) == 2 * 6 + 2 and all(r["us"] > 0 and r["frac"] > 0 for r in rows)
    assert by_op["decode: gate/up product + SiLU.mul"]["kernel"] == "gemm_smallm"
    assert "attn_decode_tma" in by_op["decode: bias + RoPE + cache write + attention over 320 keys"]["kernel"]
    assert "attn_prefill_tc5" in by_op["prefill: bias + RoPE + cache write + causal attention, 192 tokens"]["kernel"]
    assert "library product" in by_op["prefill: down product"]["kernel"]
    assert format_table(rows).count("\n") == len(rows) + 1
    only = kernel_table(spec, 4, 320, 192, 6456.5, 1657.4, page_size=16, only=("gate/up",))
    assert [r["op"] for r in only] == ["decode: gate/up product + SiLU.mul", "prefill: gate/up product + SiLU.mul"]
