"""A model assembled from a ``ModelSpec``: embedding, scheduled blocks, final norm, output head."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..parts.base import ResidualStream, Runtime, StepContext, WeightDecl, build_part
from ..parts.linear import matmul_nt
from .spec import ModelSpec


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime, config=None):
        self.spec, self.runtime, self.config = spec, runtime, config
        self.blocks = [build_part("block", layer.block, runtime) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.embedding = runtime.empty(spec.vocab_size, spec.hidden_size)
        # one buffer, two views when the output matrix is tied (flow_engine/model.py:110-112)
        self.head = self.embedding if spec.tie_word_embeddings else runtime.empty(spec.vocab_size, spec.hidden_size)
        self.graph_safe = all(b.graph_safe for b in self.blocks) and self.final_norm.graph_safe
        # who consumes each run's output: the first norm of the next run, or the final norm
        self._split_ok = []
        for i, entry in enumerate(spec.schedule):
            nxt = self.blocks[spec.schedule[i + 1].layer] if i + 1 < len(spec.schedule) else None
            consumer = getattr(nxt, "norm1", None) if nxt is not None else self.final_norm
            self._split_ok.append(bool(getattr(consumer, "accepts_split_sum", False)))
        self.loaded = False

    # ---- weights --------------------------------------------------------
    def weight_decls(self) -> dict[str, WeightDecl]:
        """Full checkpoint name -> declaration, for the loader and the random-weights writer."""
        spec = self.spec
        decls: dict[str, WeightDecl] = {}

        def add(name: str, decl: WeightDecl):
            if name in decls:
                raise ValueError(f"two parts declare the weight {name!r}")
            decls[name] = WeightDecl(name, tuple(decl.shape), decl.role, decl.init, decl.dest)

        add(spec.embedding_name, WeightDecl("", (spec.vocab_size, spec.hidden_size), dest=self.embedding))
        for layer, block in zip(spec.layers, self.blocks):
            for w in block.weights():
                add(f"{layer.prefix}.{w.name}", w)
        for w in self.final_norm.weights():
            add(f"{spec.final_norm_prefix}.{w.name}", w)
        if not spec.tie_word_embeddings:
            add(spec.head_name, WeightDecl("", (spec.vocab_size, spec.hidden_size), dest=self.head))
        return decls

    def finalize(self) -> None:
        for b in self.blocks:
            b.finalize()
        self.final_norm.finalize()
        self.loaded = True

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for d in self.weight_decls().values():
            key = (d.dest.untyped_storage().data_ptr(), d.dest.storage_offset())
            if key not in seen:
                seen.add(key)
                total += d.dest.numel() * d.dest.element_size()
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
        spec, n = self.spec, ctx.n_tokens
        resid = ctx.workspace.get("model.resid", (n, spec.hidden_size), torch.float32)
        ops.embed(resid, self.embedding, ctx.token_ids, n, ctx.status, ctx.device_tokens)
        stream = ResidualStream(resid)
        for i, entry in enumerate(spec.schedule):
            block = self.blocks[entry.layer]
            block.next_norm_accepts_split_sum = self._split_ok[i]
            block.forward(ctx, stream, caches[i], write_cache=entry.cache_of is None)
        if n_logit_rows > 0:
            y = ctx.workspace.get("model.final", (n_logit_rows, spec.hidden_size), self.runtime.dtype)
            self.final_norm.forward(ctx, y, resid, stream.pending, n_logit_rows, rows=logit_rows)
            self.head_logits(ctx, logits, y, n_logit_rows)
        return logits

    def head_logits(self, ctx: StepContext, logits: torch.Tensor, y: torch.Tensor, n_rows: int) -> None:
        """logits = y @ head.T in fp32 (reference: flow_engine/model.py:204)."""
        if ops.stream_product_preferred(y, self.head, n_rows):
            ops.gemm_tcgen05_stream(logits[:n_rows], y, self.head, n_rows, ctx.status)
        elif ops.tcgen05_supported(y, self.head, n_rows):
            ops.gemm_tcgen05(logits[:n_rows], y, self.head, n_rows, ctx.status, swap=True)
        elif ops.small_m_supported(y, self.head, n_rows):
            ops.gemm_small_m(logits[:n_rows], y, self.head, n_rows)
        else:
            matmul_nt(logits[:n_rows], y, self.head)
