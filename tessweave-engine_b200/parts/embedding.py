"""Embedding parts: token ids in, rows of the residual stream out."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Embedding, ResidualStream, Runtime, StepContext, WeightDecl, register_part


@register_part("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    """resid[n] = float(weight[token_ids[n]]), no scaling (reference: flow_engine/model.py:176).

    The residual stream this part creates is fp32 in both run types.  A token id ``-(i + 1)`` names the
    i-th token the step before chose, which is still on the device (``ctx.device_tokens``); the kernel
    looks it up itself.  A token id outside the vocabulary sets an error bit and gives a row of zeros.
    """

    def __init__(self, runtime: Runtime, vocab: int, hidden: int):
        super().__init__(runtime)
        if min(vocab, hidden) <= 0:
            raise ValueError("embedding needs a positive vocabulary and width")
        self.vocab, self.hidden = int(vocab), int(hidden)
        self.weight = runtime.empty(self.vocab, self.hidden)

    def weights(self) -> list[WeightDecl]:
        return [WeightDecl("weight", (self.vocab, self.hidden), dest=self.weight)]

    def shared_matrix(self) -> torch.Tensor:
        return self.weight

    def forward(self, ctx: StepContext) -> ResidualStream:
        resid = ctx.workspace.get("model.resid", (ctx.n_tokens, self.hidden), torch.float32)
        ops.embed(resid, self.weight, ctx.token_ids, ctx.n_tokens, ctx.status, ctx.device_tokens)
        return ResidualStream(resid)
