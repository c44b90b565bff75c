"""The command line as a user starts it: ``bin/flow-inference`` in a process of its own.
``doctor``, ``inspect``, ``init`` and ``replay`` need no GPU; ``generate`` does and is compared
with the plain implementation (reference: flow_engine/cli.py:48-120)."""
import json
import subprocess
import sys

import pytest

from helpers import CONFIGS, ROOT, make_folder
import plain_qwen2

CLI = [sys.executable, str(ROOT / "bin" / "flow-inference")]


def run_cli(*words, **kw):
    return subprocess.run(CLI + [str(w) for w in words], capture_output=True, text=True, timeout=900, **kw)


def test_doctor_reports_the_runtime():
    proc = run_cli("doctor")
    assert proc.returncode == 0, proc.stderr
    report = json.loads(proc.stdout)
    assert {"python", "platform", "torch", "cuda", "nvcc", "architectures"} <= set(report)
    assert "Qwen2ForCausalLM" in report["architectures"]


@pytest.mark.parametrize("name", ["A", "B"])
def test_inspect_explains_the_cache(name, tmp_path):
    folder = make_folder(tmp_path, name)
    c = CONFIGS[name]
    proc = run_cli("inspect", folder, "--kv-blocks", 10, "--block-size", 8)
    assert proc.returncode == 0, proc.stderr
    out = json.loads(proc.stdout)
    per_token = 2 * c["num_hidden_layers"] * c["num_key_value_heads"] * c["head_dim"]       # K and V, every layer
    assert out["kv_bf16_bytes"] == per_token * 2 * 10 * 8 and out["kv_fp32_bytes"] == per_token * 4 * 10 * 8
    assert out["architecture"]["hidden_size"] == c["hidden_size"] and out["layers_in_schedule"] == c["num_hidden_layers"]
    assert out["state_bytes_per_request"] == 0
    params = sum(t.numel() for t in plain_qwen2.read_folder(folder)[1].values())
    assert 2 * params <= out["weight_bf16_bytes"] <= 2 * params + 2 * 64 * 1024      # matrices in 16 bits, vectors stay in 32
    assert run_cli("inspect", folder, "--kv-blocks", 0).returncode != 0


def test_inspect_refuses_what_the_gate_refuses(tmp_path):
    folder = tmp_path / "m"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps({**CONFIGS["A"], "use_sliding_window": True}))
    proc = run_cli("inspect", folder)
    assert proc.returncode != 0 and "sliding_window" in proc.stderr


def test_init_writes_a_folder_and_replay_filters_events(tmp_path):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(CONFIGS["B"]))
    proc = run_cli("init", tmp_path / "model", "--config", config, "--seed", 3)
    assert proc.returncode == 0, proc.stderr
    assert (tmp_path / "model" / "config.json").exists() and (tmp_path / "model" / "model.safetensors").exists()
    log = tmp_path / "log.jsonl"
    rows = [{"event": "launch", "argv": []}, {"event": "step", "tokens": 3}, {"event": "submit"},
            {"event": "finish", "finish_reason": "length"}]
    log.write_text("".join(json.dumps(r) + "\n" for r in rows))
    proc = run_cli("replay", log)
    assert proc.returncode == 0
    assert [json.loads(l)["event"] for l in proc.stdout.splitlines()] == ["step", "finish"]


def test_the_prompt_never_reaches_the_audit_log():
    from tessweave_engine_b200.engine.cli import argv_without_prompt
    assert argv_without_prompt(["x", "generate", "m", "--prompt", "secret words", "--max-tokens", "3"]) == \
        ["x", "generate", "m", "--prompt", "[REDACTED]", "--max-tokens", "3"]
    assert argv_without_prompt(["x", "--prompt=secret", "--prompt-ids", "1,2"]) == ["x", "--prompt=[REDACTED]", "--prompt-ids", "1,2"]


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["A", "B"])
def test_generate_as_a_user_starts_it(name, tmp_path):
    """init -> generate --prompt-ids in float32 -> the ids on standard output are the plain implementation's
    greedy continuation; the audit log holds the run's events and ``replay`` prints them."""
    config = tmp_path / "config.json"
    config.write_text(json.dumps(CONFIGS[name]))
    folder = tmp_path / "model"
    assert run_cli("init", folder, "--config", config, "--seed", 11).returncode == 0
    prompt = [5, 17, 3, 200, 41, 7, 99, 100, 23]
    log = tmp_path / "runs" / "engine.jsonl"
    proc = run_cli("generate", folder, "--prompt-ids", ",".join(map(str, prompt)), "--dtype", "float32", "--max-tokens", 8,
                   "--ignore-eos", "--log", log, "--block-size", 8, "--kv-blocks", 32, "--prefill-chunk", 4, "--max-context", 256)
    assert proc.returncode == 0, proc.stderr[-3000:]
    got = [int(t) for t in proc.stdout.strip().split(",")]
    cfg, weights = plain_qwen2.read_folder(folder)
    assert got == plain_qwen2.generate(cfg, weights, prompt, 8)
    done = json.loads(proc.stderr.strip().splitlines()[-1])
    assert done["finish_reason"] == "length" and done["usage"] == {"prompt_tokens": 9, "completion_tokens": 8, "total_tokens": 17}
    events = [json.loads(l)["event"] for l in log.read_text().splitlines()]
    assert events[0] == "launch" and "loaded" in events and "admit" in events and events.count("finish") == 1
    assert "--prompt-ids" in json.loads(log.read_text().splitlines()[0])["argv"]
    replayed = run_cli("replay", log)
    assert replayed.returncode == 0 and {json.loads(l)["event"] for l in replayed.stdout.splitlines()} <= \
        {"step", "admit", "finish", "first_token", "fatal"}
    assert sum(json.loads(l)["event"] == "step" for l in replayed.stdout.splitlines()) >= 3 + 7     # 9 prompt tokens in portions of 4, then 7 single tokens
