"""Normalisation parts."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, Runtime, StepContext, WeightDecl, register_part


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """y = x / sqrt(mean(x^2) + eps) * weight, statistics in fp32.

    Reference: flow_engine/model.py:15-23.  The pending delta of the previous
    sub-layer is added to the residual stream in the same kernel.
    """
    accepts_split_sum = True

    def __init__(self, runtime: Runtime, size: int, eps: float, weight_name: str = "weight"):
        super().__init__(runtime)
        if size <= 0 or not eps > 0:
            raise ValueError("rmsnorm needs a positive size and eps")
        self.size, self.eps, self.weight_name = int(size), float(eps), weight_name
        self.weight = runtime.empty(self.size, dtype=torch.float32)

    def weights(self) -> list[WeightDecl]:
        return [WeightDecl(self.weight_name, (self.size,), role="vector", init="one_plus_normal", dest=self.weight)]

    def forward(self, ctx: StepContext, out, resid, delta, n_rows, rows=None) -> None:
        ops.add_rmsnorm(out, resid, delta, self.weight, self.eps, n_rows, rows)
