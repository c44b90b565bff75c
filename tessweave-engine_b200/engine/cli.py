"""Command line in the manner of the reference's ``flow-inference`` (flow_engine/cli.py:48-120).

    flow-inference doctor
    flow-inference inspect MODEL [--kv-blocks N --block-size P]
    flow-inference replay LOG
    flow-inference generate MODEL (--prompt TEXT | --prompt-ids 1,2,3 | --prompt-len N) [options]
    flow-inference init FOLDER --config CONFIG.json [--seed S --init-std STD]

Options of ``generate`` keep the reference's names and meanings where it has them:
--dtype, --max-context, --kv-blocks, --block-size, --max-active, --prefill-chunk,
--target-step-ms, --no-prefix-cache, --log, --prompt, --max-tokens.  Not carried over:
--attention, --draft-tokens, --draft-window, --unfused (one attention path, no speculative
decoding, projections always packed) and ``serve`` (no HTTP server).  New: token ids as
input (random weights have no tokenizer), --temperature, --seed, --ignore-eos, and ``init``,
which writes a model folder with random weights.
"""
from __future__ import annotations

import argparse
import json
import platform
import sys
from dataclasses import asdict
from pathlib import Path

import torch


def make_engine(args):
    """Load the model and build the engine (flow_engine/cli.py:14-45)."""
    from ..config.engine_config import EngineConfig
    from ..weights.loader import load_model
    from .scheduler import Engine
    from .trace import Trace

    if not torch.cuda.is_available():
        raise SystemExit("flow-inference: no CUDA device is visible; this engine runs on sm_100a only")
    dtype = "bfloat16" if args.dtype == "auto" else args.dtype
    trace = Trace(args.log)
    argv = list(sys.argv)
    for i, a in enumerate(argv):        # the prompt never reaches the audit log
        if a == "--prompt" and i + 1 < len(argv):
            argv[i + 1] = "[REDACTED]"
        elif a.startswith("--prompt="):
            argv[i] = "--prompt=[REDACTED]"
    trace.emit("launch", argv=argv, python=sys.version, torch=torch.__version__, device="cuda", dtype=dtype)
    print(f"Loading local weights: {args.model} (cuda, {dtype})", file=sys.stderr, flush=True)
    model = load_model(args.model, dtype, "cuda")
    config = EngineConfig(block_size=args.block_size, kv_blocks=args.kv_blocks, max_context=args.max_context,
                          max_active=args.max_active, prefill_chunk=args.prefill_chunk,
                          min_prefill_chunk=min(16, args.prefill_chunk), target_step_ms=args.target_step_ms,
                          adaptive_chunk=args.adaptive_chunk, prefix_cache=not args.no_prefix_cache)
    engine = Engine(model, config, trace)
    trace.emit("loaded", engine=asdict(config), model=model.config.as_dict() if model.config else {},
               kv_bytes=engine.cache.allocated_bytes)
    return engine


def prompt_ids(args, vocab: int) -> tuple[list[int], object]:
    """Token ids of the prompt, and the tokenizer if text was given."""
    if args.prompt_ids:
        return [int(t) for t in args.prompt_ids.split(",") if t.strip()], None
    if args.prompt_len:
        g = torch.Generator().manual_seed(args.seed)
        return torch.randint(0, vocab, (args.prompt_len,), generator=g).tolist(), None
    if args.prompt is None:
        raise SystemExit("flow-inference generate: give --prompt, --prompt-ids or --prompt-len")
    from transformers import AutoTokenizer      # tokenizer and chat template only (flow_engine/cli.py:39-42)
    tokenizer = AutoTokenizer.from_pretrained(args.model, local_files_only=True, trust_remote_code=False)
    if not tokenizer.chat_template:
        raise ValueError("A tokenizer chat_template is required; no template will be guessed")
    ids = tokenizer.apply_chat_template([{"role": "user", "content": args.prompt}], tokenize=True,
                                        add_generation_prompt=True)
    return list(ids), tokenizer


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
    p = sub.add_parser("generate")
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
    p.add_argument("--prompt", default=None)
    p.add_argument("--prompt-ids", default=None, help="comma-separated token ids instead of text")
    p.add_argument("--prompt-len", type=int, default=0, help="a random prompt of this many tokens (from --seed)")
    p.add_argument("--max-tokens", type=int, default=128)
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--ignore-eos", action="store_true")
    return parser


def main(argv=None) -> int:
    parser = build_parser()
    args = parser.parse_args(argv)
    if args.command == "doctor":
        report = {"python": sys.version, "platform": platform.platform(), "torch": torch.__version__,
                  "cuda": torch.cuda.is_available()}
        if torch.cuda.is_available():
            prop = torch.cuda.get_device_properties(0)
            report.update(device=prop.name, capability=f"{prop.major}.{prop.minor}",
                          memory_bytes=prop.total_memory, multiprocessors=prop.multi_processor_count)
        from ..csrc.build import _nvcc
        try:
            report["nvcc"] = _nvcc()
        except Exception as exc:    # noqa: BLE001  (a report, not a failure)
            report["nvcc"] = f"missing: {exc}"
        print(json.dumps(report, indent=2))
    elif args.command == "inspect":
        from ..config.registry import resolve_folder
        cfg, spec = resolve_folder(args.model)
        if min(args.kv_blocks, args.block_size) < 1:
            parser.error("Positive block count/size required")
        tokens = args.kv_blocks * args.block_size
        print(json.dumps({"architecture": cfg.as_dict(), "layers_in_schedule": len(spec.schedule),
                          "kv_formula": "2 * layers * KV_heads * head_dim * bytes_per_element * blocks * block_size",
                          "kv_bf16_bytes": cfg.kv_bytes_per_token(2) * tokens,
                          "kv_fp32_bytes": cfg.kv_bytes_per_token(4) * tokens,
                          "excludes": ["weights", "step workspace", "runtime/allocator"]}, indent=2))
    elif args.command == "replay":
        for line in Path(args.log).read_text().splitlines():
            event = json.loads(line)
            if event["event"] in {"step", "admit", "finish", "first_token", "fatal"}:
                print(json.dumps(event, ensure_ascii=False))
    elif args.command == "init":
        from ..weights.random_init import write_random_model
        config = json.loads(Path(args.config).read_text())
        folder = write_random_model(args.folder, config, seed=args.seed, std=args.init_std,
                                    store_dtype=args.store_dtype)
        print(f"wrote {folder}/config.json and model.safetensors", file=sys.stderr)
    else:
        engine = make_engine(args)
        try:
            ids, tokenizer = prompt_ids(args, engine.model.spec.vocab_size)
            r = engine.submit(ids, args.max_tokens, temperature=args.temperature, seed=args.seed,
                              ignore_eos=args.ignore_eos)
            engine.start()
            while True:
                event = r.events.get()
                if event["type"] == "done":
                    if event["error"]:
                        raise RuntimeError(event["error"])
                    break
            if tokenizer is not None:
                print(tokenizer.decode(r.output, skip_special_tokens=True))
            else:
                print(",".join(str(t) for t in r.output))
            print(json.dumps(event), file=sys.stderr)
        finally:
            engine.close()
    return 0


if __name__ == "__main__":
    sys.exit(main())
