"""Benchmark of the engine on one B200: decode tokens per second (the headline), end-to-end
decode through the Python entry point, prefill of 2,048 tokens, and decode at batch 1 and 64.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--context C]
    python bench.py --impl reference ...      # the unmodified reference, if it is installed
    python bench.py --kernels                 # every operation of a layer alone, with its roofline

The default run has the layer sizes of the Qwen2.5-7B-sized benchmark configuration with
random weights (N(0, 0.02), drawn on the device), a batch of 8 and a context of 4,096 tokens.
A "step" is one decode step.  One JSON line is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# Layer sizes of the benchmark configuration (Qwen2.5-7B-sized).
BENCH_CONFIG = {
    "architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2",
    "vocab_size": 152064, "hidden_size": 3584, "intermediate_size": 18944, "num_hidden_layers": 28,
    "num_attention_heads": 28, "num_key_value_heads": 4, "head_dim": 128,
    "rope_theta": 1000000.0, "rms_norm_eps": 1e-6, "max_position_embeddings": 32768,
    "tie_word_embeddings": False, "use_sliding_window": False, "hidden_act": "silu", "initializer_range": 0.02,
}
PAGE_SIZE = 16
PREFILL_TOKENS = 2048
SHORT_CONTEXT = 512             # the benchmark configuration's prompts: generation starts here and runs to the context length
LONG_CONTEXT = 16384            # a further point: four times the benchmark's context
LONG_PREFILL_TOKENS = 8192
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
            out = dict(FALLBACK_PEAKS)
            for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                if isinstance(raw.get(key), (int, float)):
                    out[key] = float(raw[key])
            return out, "measured"
        except Exception:   # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region is timed."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def mark(self) -> int:
        return len(self.rows)

    def stop(self):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, begin: int = 0, end: int | None = None) -> dict:
        rows = self.rows[begin:end] or self.rows
        mhz, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                mhz.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ---------------------------------------------------------------------------
def build_model(layers: int):
    import torch
    import tessweave_engine_b200 as tw
    from tessweave_engine_b200.parts.base import Runtime
    config = dict(BENCH_CONFIG, num_hidden_layers=layers)
    cfg, spec = tw.resolve(config)
    model = tw.Model(spec, Runtime(torch.device("cuda:0"), torch.bfloat16), config=cfg)
    tw.fill_random(model, seed=0)
    return model, cfg


def decode_run(model, cfg, batch: int, context: int, steps: int, warmup: int, graphs: bool = True, max_context: int = 0):
    """Device-timed decode: ``batch`` requests that already hold ``context - steps - warmup``
    tokens each (cache filled with random keys and values) decode one token per step.  ``max_context``: the
    longest request the engine is configured for (block tables and the choices frozen into the captured graphs
    are made for it); by default the context itself."""
    import torch
    import tessweave_engine_b200 as tw
    from tessweave_engine_b200.engine.runner import ModelRunner, StepEntry
    total = warmup + steps
    start = max(1, context - total)
    pages = batch * (-(-(start + total) // PAGE_SIZE))
    cache = tw.CacheManager(model.cache_needs(), PAGE_SIZE, pages, batch, max(start + total, max_context), model.runtime.dtype,
                            model.runtime.device, prefix_cache=False)
    for g in cache.groups:
        g.k.normal_(0, 0.5)
        g.v.normal_(0, 0.5)
    runner = ModelRunner(model, cache, max_step_tokens=batch, max_step_seqs=batch, cuda_graphs=graphs)
    leases = [cache.admit(None) for _ in range(batch)]
    for lease in leases:
        cache.ensure(lease, start + total)
    gen = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, cfg.vocab_size, (total, batch), generator=gen).tolist()

    def one(i):
        entries = [StepEntry(leases[b].slot, [tokens[i][b]], start + i, [0]) for b in range(batch)]
        return runner.step(entries)

    from tessweave_engine_b200.csrc import ops
    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    eager_before = ops.LAUNCHES[0]
    begin.record()
    for i in range(warmup, total):
        one(i)
    end.record()
    torch.cuda.synchronize()
    eager = ops.LAUNCHES[0] - eager_before
    runner.check_status()
    ms = begin.elapsed_time(end)
    bucket = next((b for b in sorted(runner.graph_kernels) if b >= batch), None)
    kernels_per_step = runner.graph_kernels.get(bucket)
    del runner, cache
    torch.cuda.empty_cache()
    ctx_mid = start + warmup + steps / 2
    return {"ms_per_step": ms / steps, "tok_s": batch * steps / (ms / 1e3), "context": ctx_mid,
            "kernels_per_step": kernels_per_step, "eager_launches": eager}


def decode_bytes(model, cfg, batch: int, context: float) -> float:
    """Bytes a decode step has to read: every weight it uses once (all blocks, final norm,
    output matrix; of the embedding only ``batch`` rows) and the cache of the live requests."""
    element = 2 if model.runtime.dtype == __import__("torch").bfloat16 else 4
    return model.step_weight_bytes(batch) + batch * context * model.cache_bytes_per_token(element)


def prefill_run(model, cfg, tokens: int, reps: int, warmup: int):
    import torch
    import tessweave_engine_b200 as tw
    from tessweave_engine_b200.engine.runner import ModelRunner, StepEntry
    pages = -(-tokens // PAGE_SIZE)
    cache = tw.CacheManager(model.cache_needs(), PAGE_SIZE, pages, 1, tokens, model.runtime.dtype,
                            model.runtime.device, prefix_cache=False)
    runner = ModelRunner(model, cache, max_step_tokens=tokens, max_step_seqs=1, max_logit_rows=1, cuda_graphs=False)
    lease = cache.admit(None)
    cache.ensure(lease, tokens)
    gen = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (tokens,), generator=gen).tolist()
    entry = [StepEntry(lease.slot, ids, 0, [tokens - 1])]
    for _ in range(warmup):
        runner.step(entry)
    torch.cuda.synchronize()
    # every repetition is timed by itself and the median is reported: a 25 ms burst of tensor-core work is
    # sensitive to where the power management happens to be
    times = []
    for _ in range(reps):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        runner.step(entry)
        end.record()
        torch.cuda.synchronize()
        times.append(begin.elapsed_time(end))
    runner.check_status()
    ms = statistics.median(times)
    L, H, I, V = cfg.num_hidden_layers, cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    qkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
    linear = 2.0 * tokens * L * (H * qkv + cfg.num_attention_heads * cfg.head_dim * H + 3 * H * I)
    attn = L * 4.0 * cfg.num_attention_heads * cfg.head_dim * tokens * (tokens + 1) / 2
    flops = linear + attn + 2.0 * H * V
    del runner, cache
    torch.cuda.empty_cache()
    return {"ms": ms, "tok_s": tokens / (ms / 1e3), "flops": flops}


def e2e_run(model, cfg, batch: int, context: int, steps: int, warmup: int):
    """The same decode through the public entry point: ``Engine.submit`` / ``Engine.step``,
    host token ids in (pinned staging buffer, one H2D copy per step) and sampled ids out (one
    D2H copy per step).  The prompts are read by the engine first (not timed)."""
    import torch
    import tessweave_engine_b200 as tw
    total = warmup + steps + 8          # head-room: no request reaches its length budget inside the timed steps
    prompt_len = max(1, context - total)
    pages = batch * (-(-(prompt_len + total) // PAGE_SIZE)) + 1
    engine = tw.Engine(model, tw.EngineConfig(block_size=PAGE_SIZE, kv_blocks=pages, max_context=prompt_len + total,
                                              max_active=batch, max_queue=batch, prefill_chunk=2048,
                                              max_step_tokens=2048 + batch, prefix_cache=False))
    gen = torch.Generator().manual_seed(3)
    for b in range(batch):
        prompt = torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen).tolist()
        engine.submit(prompt, max_tokens=total, ignore_eos=True)
    while any(r.computed < len(r.prompt) for r in list(engine.requests.values())) or engine.waiting:
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        engine.step()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    h2d = engine.runner._host.numel() * 4
    d2h = (batch + 1) * 4
    generated = engine.counters["generated_tokens"]
    engine.close()
    del engine
    torch.cuda.empty_cache()
    return {"tok_s": batch * steps / seconds, "ms_per_step": seconds / steps * 1e3, "h2d": h2d, "d2h": d2h,
            "generated": generated}


def generation_run(model, cfg, batch: int, prompt_len: int, context: int):
    """The workload the benchmark configuration names, end to end through ``Engine.submit`` / ``Engine.step``:
    ``batch`` random prompts of ``prompt_len`` tokens, each generating up to ``context`` tokens in all.  Decode
    tokens per second averaged over the whole run (the prompts' steps are left out of the time)."""
    import torch
    import tessweave_engine_b200 as tw
    pages = batch * (-(-context // PAGE_SIZE)) + 1
    engine = tw.Engine(model, tw.EngineConfig(block_size=PAGE_SIZE, kv_blocks=pages, max_context=context, max_active=batch,
                                              max_queue=batch, prefill_chunk=2048, max_step_tokens=2048 + batch,
                                              prefix_cache=False))
    gen = torch.Generator().manual_seed(5)
    reqs = [engine.submit(torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen).tolist(),
                          max_tokens=context - prompt_len, ignore_eos=True) for _ in range(batch)]
    while any(r.computed < len(r.prompt) for r in reqs) or engine.waiting:
        engine.step()
    for _ in range(4):
        engine.step()
    torch.cuda.synchronize()
    before = sum(len(r.output) for r in reqs)
    t0 = time.perf_counter()
    engine.run_until_done()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    generated = sum(len(r.output) for r in reqs) - before
    engine.close()
    del engine
    torch.cuda.empty_cache()
    return {"tok_s": generated / seconds, "seconds": seconds, "generated": generated}


WORKLOAD_SIZES = {
    # layer sizes of the Qwen2.5-14B-sized and -32B-sized configurations
    "continuous14b": dict(num_hidden_layers=48, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                          head_dim=128, intermediate_size=13824),
    "prefix32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=40, num_key_value_heads=8,
                      head_dim=128, intermediate_size=27648),
}


def workload_run(name: str, layers: int | None) -> dict:
    """Two whole-engine workloads through ``Engine.submit`` / ``Engine.step`` with random weights:
    continuous14b -- 32 requests, prompts of 128..2048 tokens, 64..512 generated tokens each, prompt
                     portions of 512, continuous batching;
    prefix32b     -- 16 requests with prompts of 8192 tokens that share their first 4096, 256 generated
                     tokens each; the shared pages are computed once."""
    import torch
    import tessweave_engine_b200 as tw
    from tessweave_engine_b200.parts.base import Runtime
    sizes = dict(WORKLOAD_SIZES[name])
    full_layers = sizes["num_hidden_layers"]
    if layers:
        sizes["num_hidden_layers"] = layers
    config = dict(BENCH_CONFIG, **sizes)
    cfg, spec = tw.resolve(config)
    model = tw.Model(spec, Runtime(torch.device("cuda:0"), torch.bfloat16), config=cfg)
    tw.fill_random(model, seed=0)
    # An untimed request first: whatever has to be compiled or captured (kernels of this head size, prompt
    # portions long enough for the tcgen05 kernels, decode graphs) is compiled and captured here.
    warm = tw.Engine(model, tw.EngineConfig(block_size=PAGE_SIZE, kv_blocks=64, max_context=800, max_active=2, max_queue=2,
                                            prefill_chunk=640, max_step_tokens=642, prefix_cache=False))
    warm.submit(torch.randint(0, cfg.vocab_size, (700,)).tolist(), max_tokens=3, ignore_eos=True)
    warm.run_until_done()
    warm.close()
    del warm
    gen = torch.Generator().manual_seed(11)
    rand = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=gen))
    toks = lambda n: torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()
    if name == "continuous14b":
        jobs = [(toks(rand(128, 2048)), rand(64, 512)) for _ in range(32)]
        pages = sum(-(-(len(p) + m) // PAGE_SIZE) for p, m in jobs) + 8
        engine = tw.Engine(model, tw.EngineConfig(block_size=PAGE_SIZE, kv_blocks=pages, max_context=2560, max_active=32,
                                                  max_queue=32, prefill_chunk=512, max_step_tokens=512))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        reqs = [engine.submit(p, max_tokens=m, ignore_eos=True) for p, m in jobs]
        engine.run_until_done()
    else:
        shared = toks(4096)
        jobs = [(shared + toks(4096), 256) for _ in range(16)]
        pages = 4096 // PAGE_SIZE + 16 * (-(-(4096 + 256) // PAGE_SIZE)) + 8
        engine = tw.Engine(model, tw.EngineConfig(block_size=PAGE_SIZE, kv_blocks=pages, max_context=8192 + 256,
                                                  max_active=16, max_queue=16, prefill_chunk=2048,
                                                  max_step_tokens=2048 + 16))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        reqs = [engine.submit(jobs[0][0], max_tokens=256, ignore_eos=True)]
        while reqs[0].computed < 4096:           # the owner of the prefix computes it first
            engine.step()
        reqs += [engine.submit(p, max_tokens=m, ignore_eos=True) for p, m in jobs[1:]]
        engine.run_until_done()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    stats = engine.stats()
    engine.close()
    generated = sum(len(r.output) for r in reqs)
    return {"workload": name, "impl": "ours", "layers": sizes["num_hidden_layers"], "layers_full": full_layers,
            "requests": len(reqs), "prompt_tokens": sum(len(p) for p, _ in jobs), "generated_tokens": generated,
            "prefill_tokens_computed": stats["prefill_tokens"], "prefix_hit_tokens": stats["prefix_hit_tokens"],
            "steps": stats["steps"], "seconds": round(seconds, 3), "generated_tok_s": round(generated / seconds, 1),
            "total_tok_s": round((generated + stats["prefill_tokens"]) / seconds, 1),
            "finished": stats["finished"], "weights_gb": round(model.weight_bytes() / 1e9, 2)}


def config_record(args, peaks_source: str) -> dict:
    """What both arms measure on (flat, every size named): the same record in the line of either arm."""
    c = BENCH_CONFIG
    return {"model": "Qwen2.5-7B-sized (random weights)", "layers": args.layers, "layers_full": c["num_hidden_layers"],
            "hidden": c["hidden_size"], "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"],
            "head_dim": c["head_dim"], "intermediate": c["intermediate_size"], "vocab": c["vocab_size"],
            "global_batch": args.batch, "seq_len": args.context, "page_size": PAGE_SIZE, "prefill_tokens": PREFILL_TOKENS,
            "parallelism": "single GPU", "l2": "inputs larger than L2 (weights >> 126 MB)", "peaks": peaks_source}


def reference_arm(args) -> int:
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "flow_engine").exists():
        print(json.dumps({"impl": "reference", "unavailable": "the reference is not installed under baseline/_ref "
                          "(pip install --no-index --no-deps --target baseline/_ref <reference>)"}))
        return 0
    try:
        from baseline.run_reference import run
        print(json.dumps(run(args, BENCH_CONFIG, config_record(args, peaks()[1]))))
    except Exception as exc:    # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:160]}"}))
    return 0


def timeline_run(args) -> int:
    """One decode step of ``--layers`` layers recorded on the device: every launch with its start, the gap to
    the launch before, how long its blocks took to start and waited, and when its first and last block ended."""
    import torch
    import tessweave_engine_b200 as tw
    from tessweave_engine_b200.engine.runner import ModelRunner, StepEntry
    from tessweave_engine_b200.engine.timeline import Timeline, format_launches
    timeline = Timeline()
    model, cfg = build_model(args.layers)
    batch, total = args.batch, max(4, args.warmup) + 1
    start = max(1, args.context - total)
    pages = batch * (-(-(start + total) // PAGE_SIZE))
    cache = tw.CacheManager(model.cache_needs(), PAGE_SIZE, pages, batch, start + total, model.runtime.dtype,
                            model.runtime.device, prefix_cache=False)
    for g in cache.groups:
        g.k.normal_(0, 0.5)
        g.v.normal_(0, 0.5)
    runner = ModelRunner(model, cache, max_step_tokens=batch, max_step_seqs=batch, cuda_graphs=not args.no_graphs)
    leases = [cache.admit(None) for _ in range(batch)]
    for lease in leases:
        cache.ensure(lease, start + total)

    def one(i):
        runner.step([StepEntry(leases[b].slot, [(7 * i + b) % cfg.vocab_size], start + i, [0]) for b in range(batch)])

    for i in range(total - 1):
        one(i)
    timeline.reset()
    one(total - 1)
    rows = timeline.launches()
    runner.check_status()
    print(format_launches(rows), file=sys.stderr)
    by_kernel: dict[str, list[float]] = {}
    for r in rows:
        by_kernel.setdefault(f"{r['kernel']} x{r['blocks']}", []).append(r["end"] - r["start"] - r["waited"])
    # per kernel and grid size: launches, and the median time from the end of its blocks' wait to its last block's end
    summary = {k: {"launches": len(v), "median_us": round(sorted(v)[len(v) // 2], 2)} for k, v in by_kernel.items()}
    print(json.dumps({"timeline": "one decode step", "layers": args.layers, "batch": batch, "context": args.context,
                      "launches": len(rows), "step_us": round(rows[-1]["end"], 1) if rows else None, "kernels": summary}))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=BENCH_CONFIG["num_hidden_layers"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--skip-extras", action="store_true", help="only the headline decode measurement")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one small measurement and print its figures (for profiling a kernel on a small case)")
    ap.add_argument("--no-graphs", action="store_true", help="launch decode steps kernel by kernel")
    ap.add_argument("--kernels", action="store_true",
                    help="time every operation of a layer and the output head alone and print each with its roofline")
    ap.add_argument("--timeline", action="store_true",
                    help="record one decode step block by block on the device (kernels compiled with their recorder) "
                         "and print its launches in time order; for looking at, not a measurement")
    ap.add_argument("--workload", choices=sorted(WORKLOAD_SIZES), default=None,
                    help="run a whole-engine workload at 14B / 32B layer sizes instead of the headline measurement")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported by this single-GPU engine")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(3, args.warmup)

    import torch
    if not torch.cuda.is_available():
        print("bench.py needs a CUDA device", file=sys.stderr)
        return 1
    if args.workload:
        print(json.dumps(workload_run(args.workload, args.layers if args.layers != BENCH_CONFIG["num_hidden_layers"] else None)))
        return 0
    pk, pk_source = peaks()
    if args.kernels:
        import tessweave_engine_b200 as tw
        from tessweave_engine_b200.engine.kernel_bench import format_table, kernel_table
        _, spec = tw.resolve(BENCH_CONFIG)
        rows = kernel_table(spec, args.batch, args.context, PREFILL_TOKENS, pk["hbm_gbs"], pk["bf16_tflops"], PAGE_SIZE)
        print(format_table(rows), file=sys.stderr)
        print(json.dumps({"kernels": rows, "peaks": pk, "peaks_source": pk_source, "batch": args.batch,
                          "context": args.context, "prefill_tokens": PREFILL_TOKENS}))
        return 0
    if args.timeline:
        os.environ["TESSWEAVE_TIMELINE"] = "1"       # before the first kernel library is loaded
        return timeline_run(args)
    model, cfg = build_model(args.layers)
    if args.only == "prefill":
        print(json.dumps({"only": "prefill", "layers": args.layers, **prefill_run(model, cfg, PREFILL_TOKENS, args.steps, args.warmup)}))
        return 0
    if args.only == "decode":
        print(json.dumps({"only": "decode", "layers": args.layers,
                          **decode_run(model, cfg, args.batch, args.context, args.steps, args.warmup, not args.no_graphs)}))
        return 0
    sampler = ClockSampler()
    sampler.start()
    mark0 = sampler.mark()
    main_run = decode_run(model, cfg, args.batch, args.context, args.steps, args.warmup)
    mark1 = sampler.mark()
    clocks = sampler.summary(mark0, mark1)
    record = {
        "metric": "decode tokens/s, Qwen2.5-7B-sized bf16, batch 8, context 4096", "value": round(main_run["tok_s"], 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main_run["ms_per_step"], 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), uniform random token ids",
        "impl": "ours",
        "config": config_record(args, pk_source),
    }
    nbytes = decode_bytes(model, cfg, args.batch, main_run["context"])
    achieved = nbytes / (main_run["ms_per_step"] / 1e3) / 1e9
    record["roofline"] = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                          "frac": round(achieved / pk["hbm_gbs"], 4), "of": pk_source}
    kernels = main_run["kernels_per_step"]
    record["gpu_launches"] = int(kernels * args.steps) if kernels else int(main_run["eager_launches"])
    if not args.skip_extras:
        pre = prefill_run(model, cfg, PREFILL_TOKENS, reps=7, warmup=3)
        peak_flops = pk.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]) * 1e12
        record["prefill"] = {"value": round(pre["tok_s"], 1), "tokens": PREFILL_TOKENS, "ms": round(pre["ms"], 3),
                             "frac": round(pre["flops"] / (pre["ms"] / 1e3) / peak_flops, 4)}
        points = {}
        for b in (1, 64):
            r = decode_run(model, cfg, b, args.context, max(8, args.steps // 2), 3)
            points[f"decode_b{b}"] = round(r["tok_s"], 1)
        # the other end of the workload: requests of about 512 tokens inside an engine set up for 4,096
        for b in (1, 8, 64):
            r = decode_run(model, cfg, b, SHORT_CONTEXT, max(8, args.steps // 2), 3, max_context=args.context)
            points[f"decode_b{b}_ctx{SHORT_CONTEXT}"] = round(r["tok_s"], 1)
        # a longer context: 16,384 keys a request (the cache of the live requests is then half of what a step reads)
        r = decode_run(model, cfg, args.batch, LONG_CONTEXT, max(8, args.steps // 2), 3)
        points[f"decode_b{args.batch}_ctx{LONG_CONTEXT}"] = round(r["tok_s"], 1)
        points[f"decode_b{args.batch}_ctx{LONG_CONTEXT}_hbm_frac"] = round(
            decode_bytes(model, cfg, args.batch, r["context"]) / (r["ms_per_step"] / 1e3) / 1e9 / pk["hbm_gbs"], 4)
        # and the whole of it: prompts of 512 tokens generating to 4,096, end to end, averaged over the run
        run = generation_run(model, cfg, args.batch, SHORT_CONTEXT, args.context)
        points[f"decode_b{args.batch}_avg_{SHORT_CONTEXT}_to_{args.context}_e2e"] = round(run["tok_s"], 1)
        long_pre = prefill_run(model, cfg, LONG_PREFILL_TOKENS, reps=3, warmup=2)
        points[f"prefill_{LONG_PREFILL_TOKENS}"] = round(long_pre["tok_s"], 1)
        points[f"prefill_{LONG_PREFILL_TOKENS}_frac"] = round(long_pre["flops"] / (long_pre["ms"] / 1e3) / peak_flops, 4)
        record["points"] = points
        e2e = e2e_run(model, cfg, args.batch, args.context, args.steps, args.warmup)
        record["e2e"] = {"value": round(e2e["tok_s"], 1), "unit": "tokens/s", "ms_per_step": round(e2e["ms_per_step"], 4),
                         "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"]}
        # the dominant kernel of both regimes (the gate/up product) alone, against its own roofline
        from tessweave_engine_b200.engine.kernel_bench import kernel_table
        rows = kernel_table(model.spec, args.batch, args.context, PREFILL_TOKENS, pk["hbm_gbs"], pk["bf16_tflops"], PAGE_SIZE,
                            only=("gate/up",))
        record["dominant_kernel"] = {r["op"]: {"kernel": r["kernel"], "us": r["us"], "frac": r["frac"], "bound": r["bound"]}
                                     for r in rows}
    sampler.stop()
    record["clocks"] = clocks
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
