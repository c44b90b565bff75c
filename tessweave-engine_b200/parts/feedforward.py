"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import FeedForward, Runtime, StepContext, WeightDecl, register_part
from .linear import linear


@register_part("feed_forward", "swiglu")
class SwiGLU(FeedForward):
    """delta = (silu(h @ Wg.T) * (h @ Wu.T)) @ Wd.T, no biases.

    gate and up are one product.  The reference packs the rows [Wg; Wu]
    (flow_engine/model.py:82-85); here, when the intermediate size is a multiple of 8, the rows
    alternate between eight gate rows and their eight up rows -- an exact permutation -- so
    that a tensor-core tile of the small-batch kernel holds a gate and its up in one thread and
    writes silu(gate) * up directly.  The activation runs in fp32.
    Reference: flow_engine/model.py:68-85.
    """

    def __init__(self, runtime: Runtime, hidden: int, intermediate: int):
        super().__init__(runtime)
        if min(hidden, intermediate) <= 0:
            raise ValueError("swiglu needs positive sizes")
        self.hidden, self.intermediate = hidden, intermediate
        self.w_gate_up = runtime.empty(2 * intermediate, hidden)
        self.w_down = runtime.empty(hidden, intermediate)
        self.interleaved = intermediate % 8 == 0

    def weights(self) -> list[WeightDecl]:
        i = self.intermediate
        if self.interleaved:
            groups = self.w_gate_up.view(i // 8, 2, 8, self.hidden)
            gate, up = groups[:, 0], groups[:, 1]          # [i / 8, 8, hidden] views; the loader reshapes the source
        else:
            gate, up = self.w_gate_up[:i], self.w_gate_up[i:]
        return [WeightDecl("gate_proj.weight", (i, self.hidden), dest=gate),
                WeightDecl("up_proj.weight", (i, self.hidden), dest=up),
                WeightDecl("down_proj.weight", (self.hidden, i), dest=self.w_down)]

    def forward(self, ctx: StepContext, h: torch.Tensor):
        return self.down(ctx, self.gate_up(ctx, h))

    def streamed_first(self) -> torch.Tensor:
        return self.w_gate_up

    def down(self, ctx: StepContext, act: torch.Tensor):
        """delta = act @ Wd.T (a tensor, or the slices of the product for the next norm to add)."""
        return linear(ctx, "ffn.delta", act, self.w_down, allow_split=True, consumer_early=True)

    def gate_up(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        """act = silu(h @ Wg.T) * (h @ Wu.T), by whichever kernel takes the step's number of rows."""
        n, ws, dt = ctx.n_tokens, ctx.workspace, self.runtime.dtype
        act = ws.get("ffn.act", (n, self.intermediate), dt)
        if self.interleaved and ops.small_m_supported(h, self.w_gate_up, n):
            ops.gemm_small_m(act, h, self.w_gate_up, n, silu_mul_pairs=True,
                             prefetch=ops.weight_head(self.w_down, ops.product_prefetch_bytes()))
        elif (self.interleaved and ops.stream_product_preferred(h, self.w_gate_up, n)
              and (ops.stream_whole_k_balanced(2 * self.intermediate) or ops.stream_split_gate_up_enabled())):
            # decode steps of 9 to 64 requests: persistent tcgen05 kernel, weights as the 128-row operand
            if ops.stream_whole_k_balanced(2 * self.intermediate):
                ops.gemm_tcgen05_stream(act, h, self.w_gate_up, n, ctx.status, silu_mul_pairs=True,    # SiLU.mul in its epilogue
                                        prefetch=ops.weight_head(self.w_down, ops.product_prefetch_bytes()))
            else:
                # the row tiles alone would leave half of the blocks with half of the work: slices over k, added
                # by the SiLU.mul kernel
                split, kper = ops.stream_split(2 * self.intermediate, self.hidden)
                slices = ws.get("ffn.gate_up.slices", (split, n, 2 * self.intermediate), torch.float32)
                ops.gemm_tcgen05_stream(slices if split > 1 else slices[0], h, self.w_gate_up, n, ctx.status, kper=kper)
                ops.silu_mul(act, ops.SplitSum(slices), n, True)
        elif self.interleaved and ops.pair_product_preferred(h, self.w_gate_up, n):
            # prompt steps: 256 x 256 tiles on pairs of thread blocks (tcgen05.mma.cta_group::2), SiLU.mul in the
            # epilogue, so the [tokens, 2 * intermediate] product never reaches memory
            ops.gemm_tcgen05_pair(act, h, self.w_gate_up, n, ctx.status, silu_mul_pairs=True)
        else:
            gate_up = linear(ctx, "ffn.gate_up", h, self.w_gate_up)
            ops.silu_mul(act, gate_up, n, self.interleaved)
        return act
