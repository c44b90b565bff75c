"""Output heads: normalised rows in, fp32 logits out."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Head, Runtime, StepContext, WeightDecl, register_part
from .linear import matmul_nt


@register_part("head", "linear_head")
class LinearHead(Head):
    """logits = y @ weight.T, accumulated and stored in fp32, no bias (reference: flow_engine/model.py:204).

    With ``tied`` the matrix is the embedding's: one buffer, two users, and the checkpoint brings no
    tensor for the head (flow_engine/model.py:110-112).  Steps with few rows stream the matrix once
    through the hand-written kernels; the rest is a library product.
    """

    def __init__(self, runtime: Runtime, vocab: int, hidden: int, tied: torch.Tensor | None = None):
        super().__init__(runtime)
        if min(vocab, hidden) <= 0:
            raise ValueError("head needs a positive vocabulary and width")
        self.vocab, self.hidden = int(vocab), int(hidden)
        if tied is not None and tuple(tied.shape) != (self.vocab, self.hidden):
            raise ValueError(f"a tied head needs a [{vocab}, {hidden}] matrix, got {tuple(tied.shape)}")
        self.tied = tied is not None
        self.weight = tied if tied is not None else runtime.empty(self.vocab, self.hidden)

    def weights(self) -> list[WeightDecl]:
        return [] if self.tied else [WeightDecl("weight", (self.vocab, self.hidden), dest=self.weight)]

    def redundant_names(self) -> list[str]:
        return ["weight"] if self.tied else []

    def forward(self, ctx: StepContext, logits: torch.Tensor, y: torch.Tensor, n_rows: int) -> None:
        out = logits[:n_rows]
        if ops.stream_product_preferred(y, self.weight, n_rows):
            ops.gemm_tcgen05_stream(out, y, self.weight, n_rows, ctx.status)
        elif ops.small_m_supported(y, self.weight, n_rows):
            ops.gemm_small_m(out, y, self.weight, n_rows)
        else:
            matmul_nt(out, y[:n_rows], self.weight)
