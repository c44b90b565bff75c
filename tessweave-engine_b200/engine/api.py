"""Python entry point, shaped like the reference's use of its engine
(tools/validate_model.py:87-105): load a model, build an ``Engine``, ``submit`` token ids,
``step`` until done, read ``request.output``.  ``generate`` does that in one call."""
from __future__ import annotations

from ..config.engine_config import EngineConfig
from ..models.model import Model
from ..weights.loader import load_model
from .scheduler import Engine


def generate(model, prompts: list[list[int]], max_tokens: int = 128, temperature: float = 0.0, seed: int = 0,
             ignore_eos: bool = False, engine_config: EngineConfig | None = None, dtype: str = "bfloat16") -> list[list[int]]:
    """Generated token ids for each prompt (lists of token ids in, lists of token ids out).

    ``model`` is a loaded ``Model`` or the path of a model folder.  Requests run together
    under continuous batching; request ``i`` samples with ``seed + i``.
    """
    if not isinstance(model, Model):
        model = load_model(model, dtype, "cuda")
    if engine_config is None:
        longest = max(len(p) for p in prompts) + max_tokens
        block = 16
        engine_config = EngineConfig(block_size=block, max_context=min(model.spec.max_position_embeddings, longest),
                                     max_active=min(len(prompts), 64), max_queue=max(32, len(prompts)),
                                     kv_blocks=min(len(prompts), 64) * (-(-longest // block)) + 1)
    engine = Engine(model, engine_config)
    try:
        requests = [engine.submit(list(p), max_tokens, temperature=temperature, seed=seed + i, ignore_eos=ignore_eos)
                    for i, p in enumerate(prompts)]
        engine.run_until_done()
        return [r.output for r in requests]
    finally:
        engine.close()
