"""Arrangements of parts around the residual stream."""
from __future__ import annotations

from .base import Block, PartSpec, ResidualStream, Runtime, StepContext, WeightDecl, build_part, register_part


@register_part("block", "pre_norm")
class PreNormBlock(Block):
    """x = x + mixer(norm1(x));  x = x + feed_forward(norm2(x)).

    Reference: flow_engine/model.py:179-202.  The residual stream is fp32; each
    sub-layer's output is handed to the next norm as a pending delta, so the add
    and the norm are one kernel.  ``names`` gives the checkpoint's prefix of each
    sub-part inside the layer.
    """

    def __init__(self, runtime: Runtime, hidden: int, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec,
                 feed_forward: PartSpec, names: dict[str, str] | None = None):
        super().__init__(runtime)
        self.hidden = hidden
        self.names = {"norm1": "norm1", "mixer": "mixer", "norm2": "norm2", "feed_forward": "feed_forward",
                      **(names or {})}
        self.norm1 = build_part("norm", norm1, runtime)
        self.mixer = build_part("mixer", mixer, runtime)
        self.norm2 = build_part("norm", norm2, runtime)
        self.feed_forward = build_part("feed_forward", feed_forward, runtime)
        self.graph_safe = all(p.graph_safe for p in self.parts().values())

    def parts(self):
        return {"norm1": self.norm1, "mixer": self.mixer, "norm2": self.norm2, "feed_forward": self.feed_forward}

    def weights(self) -> list[WeightDecl]:
        decls = []
        for role, part in self.parts().items():
            prefix = self.names[role]
            for w in part.weights():
                decls.append(WeightDecl(f"{prefix}.{w.name}" if prefix else w.name, w.shape, w.role, w.init, w.dest))
        return decls

    def redundant_names(self) -> list[str]:
        return [f"{self.names[role]}.{name}" if self.names[role] else name
                for role, part in self.parts().items() for name in part.redundant_names()]

    def finalize(self) -> None:
        for part in self.parts().values():
            part.finalize()

    def cache_need(self):
        return self.mixer.cache_need()

    def forward(self, ctx: StepContext, stream: ResidualStream, cache, write_cache: bool) -> None:
        n = ctx.n_tokens
        h = ctx.workspace.get("block.h", (n, self.hidden), self.runtime.dtype)
        self.norm1.apply(ctx, h, stream.resid, stream.pending, n)
        ctx.upcoming_weights = self.feed_forward.streamed_first()
        delta = self.mixer.forward(ctx, h, cache, write_cache)
        ctx.upcoming_weights = None
        self.norm2.apply(ctx, h, stream.resid, delta, n)
        stream.pending = self.feed_forward.forward(ctx, h)      # whoever normalises next adds it
