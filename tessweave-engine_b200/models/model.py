"""A model assembled from a ``ModelSpec``: embedding, scheduled blocks, final norm, output head.

Every stage is a part built from the spec; this file only walks them.  What an architecture does to
its embedding rows (a scale, learned positions), to its logits (a bias, a cap) or inside a layer is
the business of the part kinds its spec names.
"""
from __future__ import annotations

import torch

from ..parts.base import FixedState, PagedKV, Runtime, StepContext, WeightDecl, build_part
from .spec import ModelSpec


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime, config=None):
        self.spec, self.runtime, self.config = spec, runtime, config
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = [build_part("block", layer.block, runtime) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        # one matrix, two users, when the output head is tied to the embedding (flow_engine/model.py:110-112)
        tied = self.embedding.shared_matrix() if spec.tie_word_embeddings else None
        if spec.tie_word_embeddings and tied is None:
            raise ValueError(f"embedding kind {spec.embedding.kind!r} has no matrix a head could be tied to")
        self.head = build_part("head", spec.head, runtime, **({"tied": tied} if tied is not None else {}))
        self.graph_safe = all(p.graph_safe for p in (self.embedding, *self.blocks, self.final_norm, self.head))
        self.loaded = False

    # ---- weights --------------------------------------------------------
    def named_parts(self):
        """(checkpoint prefix, part) of every part that may declare weights."""
        spec = self.spec
        yield spec.embedding_prefix, self.embedding
        for layer, block in zip(spec.layers, self.blocks):
            yield layer.prefix, block
        yield spec.final_norm_prefix, self.final_norm
        yield spec.head_prefix, self.head

    def weight_decls(self) -> dict[str, WeightDecl]:
        """Full checkpoint name -> declaration, for the loader and the random-weights writer."""
        decls: dict[str, WeightDecl] = {}
        for prefix, part in self.named_parts():
            for w in part.weights():
                name = f"{prefix}.{w.name}" if prefix else w.name
                if name in decls:
                    raise ValueError(f"two parts declare the weight {name!r}")
                decls[name] = WeightDecl(name, tuple(w.shape), w.role, w.init, w.dest)
        return decls

    def redundant_names(self) -> set[str]:
        """Checkpoint tensors that are skipped without complaint (see ``Part.redundant_names``)."""
        return {f"{prefix}.{name}" if prefix else name for prefix, part in self.named_parts()
                for name in part.redundant_names()}

    def finalize(self) -> None:
        for _, part in self.named_parts():
            part.finalize()
        self.loaded = True

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for d in self.weight_decls().values():
            key = (d.dest.untyped_storage()._cdata, d.dest.storage_offset())     # the storage itself: also right without memory
            if key not in seen:
                seen.add(key)
                total += d.dest.numel() * d.dest.element_size()
        return total

    def step_weight_bytes(self, rows: int = 1) -> int:
        """Bytes of weights a step of ``rows`` tokens has to read: every tensor once, except the
        embedding matrix, of which a step reads one row per token (unless the head shares it)."""
        total = self.weight_bytes()
        table = self.embedding.shared_matrix()
        if table is not None and not self.spec.tie_word_embeddings:
            total -= table.numel() * table.element_size()
            total += rows * table.shape[1] * table.element_size()
        return total

    # ---- cache needs ------------------------------------------------------
    def cache_needs(self):
        """For every schedule entry: (need, cache_of).  Entries that read another entry's cache
        have no need of their own."""
        needs = []
        for e in self.spec.schedule:
            need = self.blocks[e.layer].cache_need() if e.cache_of is None else None
            needs.append((need, e.cache_of))
        return needs

    def cache_bytes_per_token(self, element_bytes: int) -> int:
        """Bytes of keys and values one token adds to the paged groups (all layers; a windowed layer
        counts like any other: the window bounds how many tokens are held, not their size)."""
        return sum(2 * need.kv_heads * need.head_dim * element_bytes
                   for need, _ in self.cache_needs() if isinstance(need, PagedKV))

    def state_bytes_per_request(self) -> int:
        """Bytes of fixed-size state one request holds beside its pages."""
        return sum(need.numel * torch.empty((), dtype=need.dtype).element_size()
                   for need, _ in self.cache_needs() if isinstance(need, FixedState))

    # ---- forward ------------------------------------------------------------
    def forward(self, ctx: StepContext, caches: list, logit_rows: torch.Tensor, n_logit_rows: int,
                logits: torch.Tensor) -> torch.Tensor:
        """Run the rows of one step through every scheduled layer; write fp32 logits of the
        wanted rows into ``logits[:n_logit_rows]``.

        Reference: flow_engine/model.py:167-204.  ``caches[i]`` is the cache view of schedule
        entry i (for an entry with ``cache_of`` the owner's view).
        """
        if not self.loaded:
            raise RuntimeError("the model has no weights yet: load them or write random ones first")
        stream = self.embedding.forward(ctx)
        for i, entry in enumerate(self.spec.schedule):
            self.blocks[entry.layer].forward(ctx, stream, caches[i], write_cache=entry.cache_of is None)
        if n_logit_rows > 0:
            y = ctx.workspace.get("model.final", (n_logit_rows, self.spec.hidden_size), self.runtime.dtype)
            self.final_norm.apply(ctx, y, stream.resid, stream.pending, n_logit_rows, rows=logit_rows)
            self.head.forward(ctx, logits, y, n_logit_rows)
        return logits
