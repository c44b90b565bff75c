"""Trace replay: feed given token ids through the model step by step and write logits.

Nothing is sampled.  The program drives the engine's own model, step function,
cache manager and kernels -- the ones generation uses; it has no forward pass,
cache or loader of its own.  The reference's ``replay`` only prints recorded
scheduler events (flow_engine/cli.py:94-98); a replay of logits is this engine's.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input carries one JSON object per line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step are one batch.  For a step in which something is wanted the
logits at the wanted places are written to ``DIR/<step>.f32`` as little-endian
fp32 ``[wanted, vocab]``, in the order of the entries and of ``want``.  After every
step ``done <step>`` is printed and flushed.  ``end`` names requests whose pages are
given back after the step.  ``--max-tokens`` sizes the page pool, so pages are used
again.
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

import torch


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    p.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    p.add_argument("--out", required=True, help="folder for <step>.f32 files")
    p.add_argument("--max-tokens", type=int, required=True,
                   help="most tokens live requests hold at any time (each rounded up to a multiple of 64)")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--max-active", type=int, default=8, help="request slots")
    p.add_argument("--poison-freed-pages", action="store_true",
                   help="fill pages with NaN when they are given back, so a stale read shows")
    return p


def run(args, stdin=None, stdout=None) -> int:
    from ..cache.manager import CacheManager
    from ..weights.loader import load_model
    from .runner import ModelRunner, StepEntry

    stdin = stdin or sys.stdin
    stdout = stdout or sys.stdout
    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; this engine has no CPU path", file=sys.stderr)
        return 3
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)
    page = args.block_size
    if page <= 0 or args.max_tokens <= 0:
        print("trace_run: --block-size and --max-tokens must be positive", file=sys.stderr)
        return 2
    model = load_model(args.model, args.dtype, "cuda")
    num_pages = math.ceil(args.max_tokens / page)
    cache = CacheManager(model.cache_needs(), page, num_pages, args.max_active, args.max_tokens,
                         model.runtime.dtype, model.runtime.device, prefix_cache=False,
                         poison_freed=args.poison_freed_pages)
    runner = ModelRunner(model, cache, max_step_tokens=args.max_tokens, max_step_seqs=args.max_active,
                         cuda_graphs=False)
    live: dict[str, tuple] = {}     # id -> (lease, tokens so far)
    for line in stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        step = record["step"]
        entries, seen = [], set()
        for item in record.get("entries", []):
            rid = str(item["id"])
            if rid in seen:
                raise ValueError(f"step {step}: request {rid!r} appears twice")
            seen.add(rid)
            tokens = [int(t) for t in item["tokens"]]
            if rid not in live:
                live[rid] = [cache.admit(None), 0]
            lease, held = live[rid]
            cache.ensure(lease, held + len(tokens))
            entries.append(StepEntry(lease.slot, tokens, held, [int(w) for w in item.get("want", [])]))
            live[rid][1] = held + len(tokens)
        if entries:
            logits = runner.step(entries)
            if logits.shape[0]:
                host = logits.to("cpu", torch.float32).contiguous()
                runner.check_status()
                (out_dir / f"{step}.f32").write_bytes(host.numpy().astype("<f4", copy=False).tobytes())
            else:
                runner.check_status()
            for item in record.get("entries", []):
                lease, held = live[str(item["id"])]
                cache.advance(lease, None, held)
        for rid in record.get("end", []):
            rid = str(rid)
            if rid in live:
                cache.release(live.pop(rid)[0])
        print(f"done {step}", file=stdout, flush=True)
    return 0


def main(argv=None) -> int:
    return run(build_parser().parse_args(argv))


if __name__ == "__main__":
    sys.exit(main())
