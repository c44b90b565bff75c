"""Helpers shared by the tests: tiny model folders, replay through the engine, schedules."""
from __future__ import annotations

import io
import json
import sys
from argparse import Namespace
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))

import plain_qwen2  # noqa: E402
from tiny_configs import CONFIGS, PAGE_SIZE, SEEDS  # noqa: E402


def note_error(test: str, case: str, error: float, scale: float) -> None:
    """With TESSWEAVE_ERROR_LOG=<file> every comparison appends what it saw (worst difference, and the
    size of the logits it was measured against): the bounds in the tests are set from such a record."""
    import os
    path = os.environ.get("TESSWEAVE_ERROR_LOG")
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"test": test, "case": case, "error": error, "scale": scale,
                                "relative": error / max(scale, 1e-30)}) + "\n")


def make_folder(tmp, name: str, store_dtype: str = "bfloat16", **overrides) -> Path:
    """Write the tiny model ``name`` ("A" or "B") into ``tmp`` with random weights."""
    from tessweave_engine_b200 import write_random_model
    config = {**CONFIGS[name], **overrides}
    return write_random_model(Path(tmp) / f"tiny_{name}_{store_dtype}", config, seed=SEEDS[name],
                              store_dtype=store_dtype)


def random_tokens(vocab: int, length: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def plain_logits(folder, tokens) -> np.ndarray:
    config, weights = plain_qwen2.read_folder(folder)
    return plain_qwen2.logits_of(config, weights, tokens).numpy()


# ---------------------------------------------------------------------------
# schedules: lists of step records as trace_run reads them
# ---------------------------------------------------------------------------
def schedule_whole(requests: dict[str, list[int]]) -> list[dict]:
    """Each request alone and whole, one after the other."""
    return [{"step": i, "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]}
            for i, (rid, toks) in enumerate(requests.items())]


def schedule_tail(requests: dict[str, list[int]], tail: int = 32) -> list[dict]:
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}],
                          "end": [rid] if p == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def schedule_portions(requests: dict[str, list[int]], sizes=(7, 2, 13, 3, 2, 16, 1, 17, 5, 2, 31)) -> list[dict]:
    """Portions of changing size, down to two tokens (and one), one request after the other."""
    steps = []
    for rid, toks in requests.items():
        p, k = 0, 0
        while p < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - p)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[p:p + n], "want": list(range(n))}],
                          "end": [rid] if p + n == len(toks) else []})
            p += n
    return steps


def schedule_mixed(requests: dict[str, list[int]], live: int = 4, seed: int = 0, prefill=(5, 2, 9, 3, 12, 2),
                   decode_from: float = 0.6) -> list[dict]:
    """Up to ``live`` requests at a time; in every step each live request brings either a
    portion of its prompt part or, past ``decode_from`` of its length, a single token; requests
    that finish are ended and the next waiting one starts, so pages are used again."""
    rng = np.random.default_rng(seed)
    waiting = list(requests.items())
    active: dict[str, list] = {}
    steps = []
    while waiting or active:
        while waiting and len(active) < live:
            rid, toks = waiting.pop(0)
            active[rid] = [toks, 0]
        entries, ended = [], []
        for rid, (toks, p) in list(active.items()):
            if len(active) > 1 and rng.random() < 0.2:
                continue                    # a request may sit a step out
            if p >= int(decode_from * len(toks)):
                n = 1
            else:
                n = int(prefill[int(rng.integers(len(prefill)))])
            n = min(n, len(toks) - p)
            entries.append({"id": rid, "tokens": toks[p:p + n], "want": list(range(n))})
            active[rid][1] = p + n
            if p + n == len(toks):
                ended.append(rid)
        for rid in ended:
            del active[rid]
        if entries:
            steps.append({"step": len(steps), "entries": entries, "end": ended})
    return steps


def max_live_tokens(steps: list[dict]) -> int:
    """Most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held: dict[str, int] = {}
    worst = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        worst = max(worst, sum(-(-n // 64) * 64 for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return worst


# ---------------------------------------------------------------------------
# running a schedule
# ---------------------------------------------------------------------------
def collect(steps: list[dict], out_dir: Path, vocab: int) -> dict[tuple[str, int], np.ndarray]:
    """(request, position) -> logits row, from the files a replay wrote."""
    pos: dict[str, int] = {}
    rows: dict[tuple[str, int], np.ndarray] = {}
    for s in steps:
        wanted = [(e["id"], pos.get(e["id"], 0) + w) for e in s["entries"] for w in e["want"]]
        for e in s["entries"]:
            pos[e["id"]] = pos.get(e["id"], 0) + len(e["tokens"])
        path = out_dir / f"{s['step']}.f32"
        if wanted:
            data = np.fromfile(path, dtype="<f4").reshape(len(wanted), vocab)
            for key, row in zip(wanted, data):
                rows[key] = row
    return rows


def replay_in_process(folder, dtype: str, steps: list[dict], out_dir, max_tokens: int | None = None,
                      block_size: int = 16, poison: bool = True, prefix_cache: bool = False) -> dict:
    """Run ``steps`` through the engine's replay program inside this process."""
    from tessweave_engine_b200.engine import replay
    out_dir = Path(out_dir)
    args = Namespace(model=str(folder), dtype=dtype, out=str(out_dir), block_size=block_size, max_active=8,
                     max_tokens=max_tokens or max_live_tokens(steps), poison_freed_pages=poison,
                     prefix_cache=prefix_cache)
    stdin = io.StringIO("".join(json.dumps(s) + "\n" for s in steps))
    stdout = io.StringIO()
    code = replay.run(args, stdin=stdin, stdout=stdout)
    assert code == 0, f"replay exited with {code}"
    done = [line for line in stdout.getvalue().splitlines() if line.startswith("done ")]
    assert len(done) == len(steps), "replay did not report every step"
    vocab = json.loads((Path(folder) / "config.json").read_text())["vocab_size"]
    return collect(steps, out_dir, vocab)
