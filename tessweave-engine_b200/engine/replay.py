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

With ``--prefix-cache`` full pages are shared between requests as in generation: a request's
first entry is looked up in the prefix index, and the tokens its hit covers (whole pages,
never the entry's last token) are not run again: the request starts at ``computed = shared``
and only places behind the hit may be wanted.  The hit is reported on standard error.
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
    p.add_argument("--prefix-cache", action="store_true",
                   help="share full pages between requests with a common prefix, as generation does")
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
                         model.runtime.dtype, model.runtime.device, prefix_cache=bool(getattr(args, "prefix_cache", False)),
                         poison_freed=args.poison_freed_pages)
    runner = ModelRunner(model, cache, max_step_tokens=args.max_tokens, max_step_seqs=args.max_active,
                         cuda_graphs=False)
    vocab = model.spec.vocab_size
    live: dict[str, list] = {}      # id -> [lease, tokens held, all tokens so far]
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
            if not tokens or min(tokens) < 0 or max(tokens) >= vocab:
                raise ValueError(f"step {step}: request {rid!r} brings no tokens or a token id outside 0..{vocab - 1}")
            want = [int(w) for w in item.get("want", [])]
            if rid not in live:
                lease = cache.admit(tokens if cache.prefix_cache else None)
                live[rid] = [lease, lease.cached_tokens, []]
                if lease.cached_tokens:
                    print(f"trace_run: request {rid} reuses {lease.cached_tokens} cached tokens", file=sys.stderr, flush=True)
                    if want and min(want) < lease.cached_tokens:
                        raise ValueError(f"step {step}: request {rid!r} wants place {min(want)}, which lies inside "
                                         f"the {lease.cached_tokens} tokens taken from shared pages")
                    want = [w - lease.cached_tokens for w in want]
                    live[rid][2].extend(tokens[:lease.cached_tokens])
                    tokens = tokens[lease.cached_tokens:]
            lease, held, history = live[rid]
            cache.ensure(lease, held + len(tokens))
            entries.append(StepEntry(lease.slot, tokens, held, want))
            history.extend(tokens)
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
                lease, held, history = live[str(item["id"])]
                cache.advance(lease, history, held)
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
