"""Live anchors on the reference's own code, where it can be imported (a checkout beside this one, or the
installed copy under ``baseline/_ref``); skipped elsewhere.  No GPU.

1. greedy token ids of the plain implementation equal those of the reference's ``Engine`` on the same tiny
   models and prompts (flow_engine/engine.py, driven as tests/test_engine.py:34-38 drives it);
2. the number of tokens a request takes from shared prefix pages equals what the reference's ``KVPool``
   and ``Engine`` report for the same sequence of requests (tests/test_engine.py:113-137), through this
   engine's scheduler with a stand-in step function.
The GPU tests then compare the engine with the plain implementation, which these tests tie to the reference.
"""
import importlib
import os
import sys
from pathlib import Path

import pytest
import torch

import plain_qwen2
from helpers import CONFIGS, PAGE_SIZE, SEEDS, random_tokens
import tessweave_engine_b200 as tw

ROOT = Path(__file__).resolve().parent.parent


def reference():
    """The reference's package, or None."""
    for place in (os.environ.get("TESSWEAVE_REFERENCE"), str(ROOT / "baseline" / "_ref")):
        if place and (Path(place) / "flow_engine" / "engine.py").exists():
            if place not in sys.path:
                sys.path.insert(0, place)
            try:
                return importlib.import_module("flow_engine")
            except Exception:       # noqa: BLE001  (an unimportable copy is the same as none)
                continue
    return None


needs_reference = pytest.mark.skipif(reference() is None, reason="the reference project cannot be imported here")


def run_reference_engine(folder, prompts, max_tokens, page, chunk, blocks=64):
    from flow_engine.config import EngineConfig
    from flow_engine.engine import Engine
    from flow_engine.model import CausalLM
    model = CausalLM.load(str(folder), "cpu", torch.float32)
    engine = Engine(model, EngineConfig(block_size=page, kv_blocks=blocks, max_context=128, max_active=4,
                                        prefill_chunk=chunk, min_prefill_chunk=min(chunk, 16)))
    requests = [engine.submit(list(p), max_tokens, ignore_eos=True) for p in prompts]
    for _ in range(10_000):
        if not engine.step():
            break
    outputs, cached = [r.output for r in requests], [r.cached for r in requests]
    engine.close()
    return outputs, cached


@needs_reference
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_plain_generation_equals_the_reference_engine(name, tmp_path):
    config = CONFIGS[name]
    folder = tw.write_random_model(tmp_path, config, seed=SEEDS[name], store_dtype="float32")
    prompts = [random_tokens(config["vocab_size"], n, 40 + n) for n in (5, 17, 33)]
    outputs, _ = run_reference_engine(folder, prompts, 8, PAGE_SIZE[name] if PAGE_SIZE[name] >= 8 else 8, 7)
    cfg, weights = plain_qwen2.read_folder(folder)
    assert outputs == [plain_qwen2.generate(cfg, weights, p, 8) for p in prompts]


class CountingRunner:
    """Stand-in step function: the scheduler's decisions are what is compared, not logits."""

    def stage_sampling(self, temperature, seed, counter):
        pass

    def step(self, entries):
        self.rows = sum(1 for e in entries if e.want)
        return torch.zeros(self.rows, 1)

    def sample(self, logits, greedy_only=False):
        return [1] * self.rows


@needs_reference
def test_prefix_hits_equal_the_reference_pool(tmp_path):
    """The same requests one after the other through the reference's engine and through this one: each
    request's ``cached`` count (tokens taken from shared pages) is the same.  Full pages only, never the last
    prompt token, the namespace part of the key, a diverging tail."""
    name, page = "A", 16
    config = CONFIGS[name]
    folder = tw.write_random_model(tmp_path, config, seed=SEEDS[name], store_dtype="float32")
    base = random_tokens(config["vocab_size"], 50, 3)
    prompts = [base, base, base[:32], base[:33], base[:20] + random_tokens(config["vocab_size"], 20, 4), base[:48] + [7]]
    from flow_engine.config import EngineConfig
    from flow_engine.engine import Engine
    from flow_engine.model import CausalLM
    ref_engine = Engine(CausalLM.load(str(folder), "cpu", torch.float32),
                        EngineConfig(block_size=page, kv_blocks=64, max_context=128, max_active=1, prefill_chunk=64))
    ours = tw.Engine(tw.load_model(folder, "float32", "cpu"),
                     tw.EngineConfig(block_size=page, kv_blocks=64, max_context=128, max_active=1, prefill_chunk=64),
                     runner=CountingRunner())
    want, got = [], []
    for p in prompts:                       # one after the other: the reference publishes a prefix when its owner ends
        for engine, record in ((ref_engine, want), (ours, got)):
            r = engine.submit(list(p), 2, ignore_eos=True)
            for _ in range(1000):
                if not engine.step():
                    break
            record.append(r.cached)
    other = [e.submit(list(base), 2, namespace="elsewhere", ignore_eos=True) for e in (ref_engine, ours)]
    for engine in (ref_engine, ours):
        while engine.step():
            pass
    assert want == got == [0, 48, 16, 32, 16, 48]
    assert other[0].cached == other[1].cached == 0
    assert ref_engine.stats()["prefix_hit_tokens"] == ours.stats()["prefix_hit_tokens"]
    ref_engine.close(); ours.close()
