"""Engine knobs, with the reference's names where it has them.

``block_size, kv_blocks, max_context, max_active, max_queue, prefill_chunk,
min_prefill_chunk, target_step_ms, prefix_cache`` carry the meaning and the
defaults of flow_engine/config.py:68-81.  The reference's ``attention`` and
``draft_*`` knobs have no counterpart (one attention path; no speculative
decoding).  ``max_step_tokens`` is new: the token budget of one mixed step.
"""
from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class EngineConfig:
    block_size: int = 16          # tokens per cache page
    kv_blocks: int = 256          # pages in each group's pool
    max_context: int = 2048       # prompt + generated tokens of one request
    max_active: int = 4           # requests that hold pages at the same time
    max_queue: int = 32           # waiting requests before submit() refuses
    prefill_chunk: int = 256      # largest portion of one prompt in a step
    min_prefill_chunk: int = 16   # floor for the adaptive portion size
    target_step_ms: float = 50.0  # step time the adaptive portion size aims at
    adaptive_chunk: bool = False  # follow the reference's EMA controller (engine.py:261-268)
    prefix_cache: bool = True     # share full pages between requests with a common prefix
    max_step_tokens: int = 0      # token budget of a step; 0 = max_active + prefill_chunk
    cuda_graphs: bool = True      # replay captured graphs for decode-only steps
    lookahead: bool = True        # launch the next step before the current one's tokens have reached the host

    def __post_init__(self):
        for key in ("block_size", "kv_blocks", "max_context", "max_active", "max_queue",
                    "prefill_chunk", "min_prefill_chunk"):
            if getattr(self, key) <= 0:
                raise ValueError(f"{key} must be positive")
        if self.prefill_chunk < self.min_prefill_chunk or self.target_step_ms <= 0:
            raise ValueError("Invalid prefill control bounds")
        if self.max_step_tokens < 0:
            raise ValueError("max_step_tokens must not be negative")
        if self.max_step_tokens and self.max_step_tokens < 2:
            raise ValueError("max_step_tokens must leave room for at least two tokens")

    @property
    def step_token_budget(self) -> int:
        return self.max_step_tokens or (self.max_active + self.prefill_chunk)
