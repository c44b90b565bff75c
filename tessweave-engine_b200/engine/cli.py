"""Command line in the manner of the reference's ``flow-inference`` (flow_engine/cli.py:48-120).

    flow-inference doctor
    flow-inference inspect MODEL [--kv-blocks N --block-size P]
    flow-inference replay LOG
    flow-inference generate MODEL (--prompt TEXT | --prompt-ids 1,2,3 | --prompt-len N) [options]
    flow-inference init FOLDER --config CONFIG.json [--seed S --init-std STD]
    flow-inference bench MODEL [--batch B --prompt-len N --max-tokens T]

Options of ``generate`` keep the reference's names and meanings where it has them:
--dtype, --max-context, --kv-blocks, --block-size, --max-active, --prefill-chunk,
--target-step-ms, --no-prefix-cache, --log, --prompt, --max-tokens.  Not carried over:
--attention, --draft-tokens, --draft-window, --unfused (one attention path, no speculative
decoding, projections always packed) and ``serve`` (no HTTP server).  New: token ids as
input (random weights have no tokenizer), --temperature, --seed, --ignore-eos, ``init``,
which writes a model folder with random weights, and ``bench``, which times generation
through the engine on the model it is given.

Every command is a function ``(args) -> exit code`` in the table at the end of this file; the
parser only describes options.
"""
from __future__ import annotations

import argparse
import json
import platform
import sys
import time
from dataclasses import asdict, is_dataclass
from pathlib import Path

import torch

REPLAYED_EVENTS = frozenset({"step", "admit", "finish", "first_token", "fatal"})
HIDDEN = "[REDACTED]"


# ---------------------------------------------------------------------------
# helpers
# ---------------------------------------------------------------------------
def argv_without_prompt(argv: list[str]) -> list[str]:
    """The command line as the audit log may keep it: the text after --prompt never reaches a file."""
    out, hide_next = [], False
    for word in argv:
        if hide_next:
            out.append(HIDDEN)
            hide_next = False
        elif word == "--prompt":
            out.append(word)
            hide_next = True
        elif word.startswith("--prompt="):
            out.append("--prompt=" + HIDDEN)
        else:
            out.append(word)
    return out


def config_as_dict(cfg) -> dict:
    if cfg is None:
        return {}
    if is_dataclass(cfg):
        return asdict(cfg)
    return {k: v for k, v in vars(cfg).items() if not k.startswith("_")}


def need_cuda(command: str) -> None:
    if not torch.cuda.is_available():
        raise SystemExit(f"flow-inference {command}: no CUDA device is visible; this engine runs on sm_100a only")


def engine_config_from(args):
    from ..config.engine_config import EngineConfig
    return EngineConfig(block_size=args.block_size, kv_blocks=args.kv_blocks, max_context=args.max_context,
                        max_active=args.max_active, prefill_chunk=args.prefill_chunk,
                        min_prefill_chunk=min(16, args.prefill_chunk), target_step_ms=args.target_step_ms,
                        adaptive_chunk=args.adaptive_chunk, prefix_cache=not args.no_prefix_cache)


def open_engine(args, command: str):
    """Model folder and options -> a running-ready ``Engine`` with its audit log."""
    from ..weights.loader import load_model
    from .scheduler import Engine
    from .trace import Trace

    need_cuda(command)
    dtype = "bfloat16" if args.dtype == "auto" else args.dtype
    trace = Trace(args.log)
    trace.emit("launch", argv=argv_without_prompt(sys.argv), python=sys.version, torch=torch.__version__,
               device="cuda", dtype=dtype)
    print(f"Loading local weights: {args.model} (cuda, {dtype})", file=sys.stderr, flush=True)
    model = load_model(args.model, dtype, "cuda")
    config = engine_config_from(args)
    engine = Engine(model, config, trace)
    trace.emit("loaded", engine=asdict(config), model=config_as_dict(model.config),
               kv_bytes=engine.cache.allocated_bytes)
    return engine


def read_prompt(args, vocab: int):
    """(token ids, tokenizer or None).  Text needs the folder's tokenizer files and its chat template
    (flow_engine/cli.py:39-42,108); ids and random prompts need neither."""
    if args.prompt_ids:
        return [int(word) for word in args.prompt_ids.split(",") if word.strip()], None
    if args.prompt_len:
        draw = torch.Generator().manual_seed(args.seed)
        return torch.randint(0, vocab, (args.prompt_len,), generator=draw).tolist(), None
    if args.prompt is None:
        raise SystemExit("flow-inference generate: give --prompt, --prompt-ids or --prompt-len")
    from transformers import AutoTokenizer      # tokenizer files and chat template only; no model code
    tokenizer = AutoTokenizer.from_pretrained(args.model, local_files_only=True, trust_remote_code=False)
    if not tokenizer.chat_template:
        raise ValueError("A tokenizer chat_template is required; no template will be guessed")
    ids = tokenizer.apply_chat_template([{"role": "user", "content": args.prompt}], tokenize=True,
                                        add_generation_prompt=True)
    return list(ids), tokenizer


def wait_for_end(request) -> dict:
    """Consume a request's events until the terminal one; raise if it ended with an error."""
    while True:
        event = request.events.get()
        if event["type"] == "done":
            if event["error"]:
                raise RuntimeError(event["error"])
            return event


# ---------------------------------------------------------------------------
# commands
# ---------------------------------------------------------------------------
def cmd_doctor(args) -> int:
    report = {"python": sys.version, "platform": platform.platform(), "torch": torch.__version__,
              "cuda": torch.cuda.is_available()}
    if report["cuda"]:
        prop = torch.cuda.get_device_properties(0)
        report.update(device=prop.name, capability=f"{prop.major}.{prop.minor}", memory_bytes=prop.total_memory,
                      multiprocessors=prop.multi_processor_count)
    from ..csrc.build import _nvcc
    try:
        report["nvcc"] = _nvcc()
    except Exception as exc:    # noqa: BLE001  (a report, not a failure)
        report["nvcc"] = f"missing: {exc}"
    from ..config.registry import architectures
    report["architectures"] = architectures()
    print(json.dumps(report, indent=2))
    return 0


def cmd_inspect(args) -> int:
    """The gate on config.json, then what the cache would take: asked of the model's own parts (built
    without memory), so an architecture with other cache needs is described as it is."""
    from ..config.registry import resolve_folder
    from ..models.model import Model
    from ..parts.base import Runtime
    if min(args.kv_blocks, args.block_size) < 1:
        raise SystemExit("flow-inference inspect: Positive block count/size required")
    cfg, spec = resolve_folder(args.model)
    model = Model(spec, Runtime(torch.device("meta"), torch.bfloat16), config=cfg)
    tokens = args.kv_blocks * args.block_size
    print(json.dumps({
        "architecture": config_as_dict(cfg), "layers_in_schedule": len(spec.schedule),
        "kv_formula": "2 * layers * KV_heads * head_dim * bytes_per_element * blocks * block_size",
        "kv_bf16_bytes": model.cache_bytes_per_token(2) * tokens,
        "kv_fp32_bytes": model.cache_bytes_per_token(4) * tokens,
        "state_bytes_per_request": model.state_bytes_per_request(),
        "weight_bf16_bytes": model.weight_bytes(),
        "excludes": ["weights", "step workspace", "runtime/allocator"]}, indent=2))
    return 0


def cmd_replay(args) -> int:
    with open(args.log, encoding="utf-8") as log:
        for line in log:
            if line.strip() and json.loads(line).get("event") in REPLAYED_EVENTS:
                print(line.rstrip("\n"))
    return 0


def cmd_init(args) -> int:
    from ..weights.random_init import write_random_model
    folder = write_random_model(args.folder, json.loads(Path(args.config).read_text()), seed=args.seed,
                                std=args.init_std, store_dtype=args.store_dtype)
    print(f"wrote {folder}/config.json and model.safetensors", file=sys.stderr)
    return 0


def cmd_generate(args) -> int:
    engine = open_engine(args, "generate")
    try:
        ids, tokenizer = read_prompt(args, engine.model.spec.vocab_size)
        request = engine.submit(ids, args.max_tokens, temperature=args.temperature, seed=args.seed,
                                ignore_eos=args.ignore_eos)
        engine.start()
        end = wait_for_end(request)
        if tokenizer is None:
            print(",".join(map(str, request.output)))
        else:
            print(tokenizer.decode(request.output, skip_special_tokens=True))
        print(json.dumps(end), file=sys.stderr)
    finally:
        engine.close()
    return 0


def cmd_bench(args) -> int:
    """``--batch`` random prompts of ``--prompt-len`` tokens, ``--max-tokens`` generated each, through the
    engine (host tokens in and out): wall time from the first submit to the last token."""
    args.kv_blocks = max(args.kv_blocks, args.batch * -(-(args.prompt_len + args.max_tokens) // args.block_size) + 1)
    args.max_context = max(args.max_context, args.prompt_len + args.max_tokens)
    args.max_active = max(args.max_active, args.batch)
    engine = open_engine(args, "bench")
    try:
        vocab = engine.model.spec.vocab_size
        draw = torch.Generator().manual_seed(args.seed)
        prompts = [torch.randint(0, vocab, (args.prompt_len,), generator=draw).tolist() for _ in range(args.batch)]
        warm = engine.submit(prompts[0][:max(2, args.prompt_len // 2)], 4, ignore_eos=True, namespace="warm-up")
        engine.run_until_done()             # compiles, captures; not timed
        del warm
        torch.cuda.synchronize()
        start = time.perf_counter()
        requests = [engine.submit(p, args.max_tokens, temperature=args.temperature, seed=args.seed + i, ignore_eos=True)
                    for i, p in enumerate(prompts)]
        engine.run_until_done()
        torch.cuda.synchronize()
        seconds = time.perf_counter() - start
        generated = sum(len(r.output) for r in requests)
        first = [r.first_token - r.created for r in requests if r.first_token]
        print(json.dumps({"batch": args.batch, "prompt_tokens": args.prompt_len, "generated_tokens": generated,
                          "seconds": round(seconds, 4), "tokens_per_s": round(generated / seconds, 1),
                          "mean_ttft_ms": round(1000 * sum(first) / max(1, len(first)), 2), **engine.stats()}))
    finally:
        engine.close()
    return 0


# ---------------------------------------------------------------------------
# parser
# ---------------------------------------------------------------------------
def add_engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("model", help="Local safetensors directory; no automatic downloads")
    p.add_argument("--device", choices=["auto", "cuda"], default="auto")
    p.add_argument("--dtype", choices=["auto", "float32", "bfloat16"], default="auto")
    p.add_argument("--max-context", type=int, default=2048)
    p.add_argument("--kv-blocks", type=int, default=256)
    p.add_argument("--block-size", type=int, default=16)
    p.add_argument("--max-active", type=int, default=4)
    p.add_argument("--prefill-chunk", type=int, default=256)
    p.add_argument("--target-step-ms", type=float, default=50)
    p.add_argument("--adaptive-chunk", action="store_true", help="steer the portion size towards --target-step-ms")
    p.add_argument("--no-prefix-cache", action="store_true")
    p.add_argument("--log", default="runs/engine.jsonl")
    p.add_argument("--max-tokens", type=int, default=128)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=0)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="flow-inference",
                                     description="Single-GPU inference engine for the Qwen2 dense decoder on B200")
    sub = parser.add_subparsers(dest="command", required=True)
    sub.add_parser("doctor", help="Read-only runtime and accelerator report")
    inspect = sub.add_parser("inspect", help="Validate architecture and explain KV allocation")
    inspect.add_argument("model")
    inspect.add_argument("--kv-blocks", type=int, default=256)
    inspect.add_argument("--block-size", type=int, default=16)
    replay = sub.add_parser("replay", help="Summarize JSONL scheduler events (no inference)")
    replay.add_argument("log")
    init = sub.add_parser("init", help="Write a model folder with random weights from a config.json")
    init.add_argument("folder")
    init.add_argument("--config", required=True, help="config.json of the architecture")
    init.add_argument("--seed", type=int, default=0)
    init.add_argument("--init-std", type=float, default=None, help="default: the config's initializer_range")
    init.add_argument("--store-dtype", choices=["bfloat16", "float32"], default="bfloat16")
    generate = sub.add_parser("generate", help="Generate from one prompt")
    add_engine_options(generate)
    generate.add_argument("--prompt", default=None)
    generate.add_argument("--prompt-ids", default=None, help="comma-separated token ids instead of text")
    generate.add_argument("--prompt-len", type=int, default=0, help="a random prompt of this many tokens (from --seed)")
    generate.add_argument("--ignore-eos", action="store_true")
    bench = sub.add_parser("bench", help="Time generation of random prompts through the engine")
    add_engine_options(bench)
    bench.add_argument("--batch", type=int, default=8)
    bench.add_argument("--prompt-len", type=int, default=512)
    return parser


COMMANDS = {"doctor": cmd_doctor, "inspect": cmd_inspect, "replay": cmd_replay, "init": cmd_init,
            "generate": cmd_generate, "bench": cmd_bench}


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return COMMANDS[args.command](args)


if __name__ == "__main__":
    sys.exit(main())
