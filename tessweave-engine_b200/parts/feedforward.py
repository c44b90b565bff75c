"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, Runtime, StepContext, WeightDecl, register_part
from .linear import linear


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """delta = (silu(h @ Wg.T) * (h @ Wu.T)) @ Wd.T, no biases.

    gate and up are one product with rows packed [Wg; Wu]; the activation runs in
    fp32.  Reference: flow_engine/model.py:68-85.
    """

    def __init__(self, runtime: Runtime, hidden: int, intermediate: int):
        super().__init__(runtime)
        if min(hidden, intermediate) <= 0:
            raise ValueError("swiglu needs positive sizes")
        self.hidden, self.intermediate = hidden, intermediate
        self.w_gate_up = runtime.empty(2 * intermediate, hidden)
        self.w_down = runtime.empty(hidden, intermediate)

    def weights(self) -> list[WeightDecl]:
        i = self.intermediate
        return [WeightDecl("gate_proj.weight", (i, self.hidden), dest=self.w_gate_up[:i]),
                WeightDecl("up_proj.weight", (i, self.hidden), dest=self.w_gate_up[i:]),
                WeightDecl("down_proj.weight", (self.hidden, i), dest=self.w_down)]

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        n, ws, dt = ctx.n_tokens, ctx.workspace, self.runtime.dtype
        gate_up = linear(ctx, "ffn.gate_up", h, self.w_gate_up)
        act = ws.get("ffn.act", (n, self.intermediate), dt)
        ops.silu_mul(act, gate_up, n)
        return linear(ctx, "ffn.delta", act, self.w_down, allow_split=ctx.split_ok)
