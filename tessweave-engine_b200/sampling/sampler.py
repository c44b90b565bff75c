"""Greedy and temperature sampling.

The reference offers exactly these two (flow_engine/engine.py:154-158; top-p, top-k
and penalties are not offered).  Greedy takes the largest logit, the lowest index at a
tie.  Temperature sampling draws from softmax(logits / T) by inverse CDF with a
uniform that depends only on the request's seed and on how many tokens the request has
drawn so far -- the reference's property that a seeded request is independent of its
neighbours (tests/test_engine.py:251-260) -- but not its CPU generator's stream, which a
device kernel cannot reproduce.  The kernel is csrc/sampling.cu.
"""
from __future__ import annotations

import torch

from ..csrc import ops

_MASK = (1 << 64) - 1


def uniform(seed: int, counter: int) -> float:
    """Host copy of the kernel's uniform in [0, 1): splitmix64, top 24 bits."""
    z = (seed + (counter + 1) * 0x9E3779B97F4A7C15) & _MASK
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def select_tokens(out: torch.Tensor, logits: torch.Tensor, n_rows: int, temperature: torch.Tensor | None = None,
                  seed: torch.Tensor | None = None, counter: torch.Tensor | None = None) -> None:
    """out[r] = the token of row r of fp32 ``logits``, for the first ``n_rows`` rows; everything stays on the device and
    nothing is allocated, so the call can be captured and can follow a step without a round trip to the host.  Rows
    whose ``temperature`` is 0 -- all of them without the three tensors (fp32, int64, int64 per row) -- are greedy.
    This is what the step function calls after every forward pass."""
    if temperature is None:
        ops.sample(out, logits, n_rows)
    else:
        ops.sample(out, logits, n_rows, temperature, seed, counter)


@torch.inference_mode()
def choose_tokens(logits: torch.Tensor, temperature=None, seed=None, counter=None) -> torch.Tensor:
    """One token id per row of fp32 ``logits`` (on the device).  ``temperature``, ``seed`` and
    ``counter`` are per-row sequences; without them every row is greedy."""
    m = logits.shape[0]
    out = torch.empty(m, dtype=torch.int32, device=logits.device)
    if temperature is None:
        select_tokens(out, logits, m)
    else:
        t = torch.as_tensor(temperature, dtype=torch.float32).to(logits.device)
        s = torch.as_tensor(seed if seed is not None else [0] * m, dtype=torch.int64).to(logits.device)
        c = torch.as_tensor(counter if counter is not None else [0] * m, dtype=torch.int64).to(logits.device)
        select_tokens(out, logits, m, t, s, c)
    return out
