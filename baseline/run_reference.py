"""The reference arm of bench.py: the unmodified reference package (installed under
``baseline/_ref`` with pip, without its dependencies) driven through its own public API --
``flow_engine.model.CausalLM``, ``flow_engine.engine.Engine.submit/step`` -- on its stock code
path (its default ``attention="sdpa"``).  Nothing of this repository's engine, kernels or models
is on that path.  The reference has no random-weights mode; its model class is constructed on
the GPU in bfloat16 and its parameters are filled with N(0, 0.02) in place, then packed with
its own ``pack_projections()`` as its loader does.

The headline value is the reference's default path.  Its opt-in ``attention="triton"`` decode path
(flow_engine/kernels/paged_decode.py) is measured as a second, separately named point where Triton
imports and the kernel compiles on the box; otherwise the record says why it is missing.
"""
from __future__ import annotations

import sys
import time
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def run(args, bench_config: dict, config_record: dict) -> dict:
    import torch
    sys.path.insert(0, str(REF))
    from flow_engine.config import EngineConfig, ModelConfig
    from flow_engine.engine import Engine
    from flow_engine.model import CausalLM

    if not torch.cuda.is_available():
        return {"impl": "reference", "unavailable": "no CUDA device is visible"}
    torch.backends.cuda.matmul.allow_tf32 = False
    batch, context = args.batch, args.context
    steps, warmup = args.steps, max(3, args.warmup)
    cfg = ModelConfig.from_dict(dict(bench_config, num_hidden_layers=args.layers))
    old = torch.get_default_dtype()
    torch.set_default_dtype(torch.bfloat16)
    try:
        with torch.device("cuda"):
            model = CausalLM(cfg)
    finally:
        torch.set_default_dtype(old)
    g = torch.Generator(device="cuda").manual_seed(0)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if name.endswith("norm.weight") or "layernorm" in name:
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=g, device="cuda", dtype=torch.float32))
            else:
                p.normal_(0.0, 0.02, generator=g)
    model.pack_projections().eval()

    total = warmup + steps + 1
    prompt_len = max(1, context - total)
    pages = batch * (-(-(prompt_len + total) // 16)) + 1

    def measure(attention: str):
        engine = Engine(model, EngineConfig(block_size=16, kv_blocks=pages, max_context=prompt_len + total,
                                            max_active=batch, max_queue=batch, prefill_chunk=2048, min_prefill_chunk=2048,
                                            target_step_ms=1e9, prefix_cache=False, attention=attention))
        try:
            gen = torch.Generator().manual_seed(3)
            for _ in range(batch):
                engine.submit(torch.randint(0, cfg.vocab_size, (prompt_len,), generator=gen).tolist(), max_tokens=total,
                              ignore_eos=True)
            t_prefill = time.perf_counter()
            while engine.waiting or any(r.computed < len(r.prompt) for r in engine.active):
                engine.step()
            torch.cuda.synchronize()
            prefill_s = time.perf_counter() - t_prefill
            for _ in range(warmup):
                engine.step()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(steps):
                engine.step()
            torch.cuda.synchronize()
            return time.perf_counter() - t0, prefill_s
        finally:
            engine.close()

    seconds, prefill_s = measure("sdpa")
    value = batch * steps / seconds
    points = {}
    try:
        import triton  # noqa: F401
        triton_seconds, _ = measure("triton")
        points["decode_triton_attention"] = round(batch * steps / triton_seconds, 1)
    except Exception as exc:       # noqa: BLE001  (an optional path of the reference; its absence is a note, not a failure)
        points["decode_triton_attention"] = None
        points["decode_triton_attention_unavailable"] = f"{type(exc).__name__}: {str(exc)[:120]}"
    return {
        "metric": "decode tokens/s, Qwen2.5-7B-sized bf16, batch 8, context 4096", "value": round(value, 1),
        "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": round(seconds / steps * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), uniform random token ids", "impl": "reference",
        "config": config_record, "attention": "sdpa (the reference's default)", "points": points,
        "e2e": {"value": round(value, 1), "unit": "tokens/s", "note": "the reference's step is host-driven; one number"},
        "prefill": {"value": round(batch * prompt_len / prefill_s, 1), "tokens": batch * prompt_len,
                    "ms": round(prefill_s * 1e3, 1), "note": "all prompts through Engine.step, chunk 2048"},
    }
