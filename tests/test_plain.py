"""The plain implementation against the reference's own outputs, and its parts (no GPU)."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2
import tessweave_engine_b200 as tw

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_plain_equals_reference_logits(name, tmp_path):
    """Golden logits come from flow_engine.model.CausalLM (tests/golden/make_golden.py)."""
    meta = json.loads((GOLDEN / f"qwen2_tiny_{name}.json").read_text())
    want = np.load(GOLDEN / f"qwen2_tiny_{name}.npy")
    folder = tw.write_random_model(tmp_path, meta["config"], seed=meta["seed"], store_dtype=meta["store_dtype"])
    config, weights = plain_qwen2.read_folder(folder)
    got = plain_qwen2.logits_of(config, weights, meta["tokens"]).numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= 5e-6


def test_rope_is_a_rotation_and_identity_at_position_zero():
    x = torch.randn(5, 3, 32)
    y = plain_qwen2.rope(x, [0, 1, 2, 3, 1000], 1e6)
    assert torch.equal(y[0], x[0])
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-5)
    # relative property: <rope(q, m), rope(k, n)> depends on m - n only
    q, k = torch.randn(1, 1, 32), torch.randn(1, 1, 32)
    a = (plain_qwen2.rope(q, [7], 1e4) * plain_qwen2.rope(k, [3], 1e4)).sum()
    b = (plain_qwen2.rope(q, [104], 1e4) * plain_qwen2.rope(k, [100], 1e4)).sum()
    assert abs(float(a - b)) < 1e-4


def test_attention_is_causal_and_grouped():
    torch.manual_seed(0)
    q, k, v = torch.randn(6, 4, 8), torch.randn(6, 2, 8), torch.randn(6, 2, 8)
    out = plain_qwen2.attention(q, k, v)
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 9.0, 9.0                              # the future must not matter
    assert torch.allclose(plain_qwen2.attention(q, k2, v2)[:4], out[:4])
    assert torch.allclose(out[0], v[0].repeat_interleave(2, dim=0))     # first token sees itself only
    # heads 0,1 use kv head 0; heads 2,3 use kv head 1
    v3 = v.clone(); v3[:, 1] += 1
    out3 = plain_qwen2.attention(q, k, v3)
    assert torch.allclose(out3[:, :2], out[:, :2]) and torch.allclose(out3[:, 2:], out[:, 2:] + 1, atol=1e-5)
    win = plain_qwen2.attention(q, k, v, window=2)
    two = plain_qwen2.attention(q[4:6], k[4:6], v[4:6])
    assert torch.allclose(win[5], two[1], atol=1e-6)


def test_rms_norm_and_swiglu_formulas():
    x = torch.tensor([[3.0, 4.0]])
    assert torch.allclose(plain_qwen2.rms_norm(x, torch.tensor([1.0, 2.0]), 0.0),
                          torch.tensor([[3 / 12.5 ** .5, 8 / 12.5 ** .5]]))
    w = {"m.gate_proj.weight": torch.tensor([[1.0]]), "m.up_proj.weight": torch.tensor([[2.0]]),
         "m.down_proj.weight": torch.tensor([[3.0]])}
    z = torch.tensor([[0.5]])
    assert torch.allclose(plain_qwen2.swiglu(w, "m", z), 3 * (0.5 / (1 + np.exp(-0.5))) * 1.0 * torch.ones(1, 1))


def test_sampler_definition():
    us = [plain_qwen2.uniform(5, i) for i in range(2000)]
    assert 0 <= min(us) and max(us) < 1 and abs(np.mean(us) - 0.5) < 0.03
    assert plain_qwen2.uniform(5, 3) != plain_qwen2.uniform(6, 3)
    from tessweave_engine_b200.sampling import uniform
    assert [uniform(9, i) for i in range(50)] == [plain_qwen2.uniform(9, i) for i in range(50)]
    logits = torch.tensor([0.0, 5.0, 5.0, 1.0])
    assert plain_qwen2.choose(logits, 0.0) == 1            # lowest index at a tie
    counts = np.bincount([plain_qwen2.choose(torch.tensor([0.0, 1.0, 2.0]), 1.0, 1, i) for i in range(4000)], minlength=3)
    want = np.exp([0, 1, 2]) / np.exp([0, 1, 2]).sum()
    assert np.abs(counts / 4000 - want).max() < 0.03
