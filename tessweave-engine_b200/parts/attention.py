"""Grouped-query attention over a paged cache."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import (Mixer, PagedKV, PagedView, PartSpec, Runtime, StepContext, WeightDecl, build_part,
                   register_part)
from .linear import SplitSum, linear


@register_part("mixer", "gqa_attention")
class GQAAttention(Mixer):
    """q/k/v projections (optionally biased), position encoding on q and k, paged causal
    attention with ``n_heads / n_kv_heads`` query heads per key/value head, output projection.

        q, k, v = split(h @ Wqkv.T + b)                 rows packed [Wq; Wk; Wv]
        q, k    = position(q), position(k)
        cache[slot(position)] = k, v
        out_h   = softmax(q_h . k_{h // group} * scale  over keys p <= position [, p > position - window]) @ v
        delta   = out @ Wo.T

    Reference: flow_engine/model.py:36-55 (projections, packing), 183-201 (forward),
    flow_engine/cache.py:93-100 (slots).  Weight names are the checkpoint's.
    """

    def __init__(self, runtime: Runtime, hidden: int, n_heads: int, n_kv_heads: int, head_dim: int,
                 qkv_bias: bool, position: PartSpec, scale: float | None = None, window: int | None = None,
                 out_bias: bool = False):
        super().__init__(runtime)
        if min(hidden, n_heads, n_kv_heads, head_dim) <= 0 or n_heads % n_kv_heads:
            raise ValueError("attention: heads must be positive and n_heads a multiple of n_kv_heads")
        if head_dim % 2 or head_dim > 256:
            raise ValueError(f"attention: head_dim {head_dim} must be even and at most 256")
        if out_bias:
            raise ValueError("attention: a bias on the output projection is not implemented")
        if window is not None and window <= 0:
            raise ValueError("attention: window must be positive or None")
        self.hidden, self.n_heads, self.n_kv_heads, self.head_dim = hidden, n_heads, n_kv_heads, head_dim
        self.scale = float(scale) if scale is not None else head_dim ** -0.5
        self.window = window
        self.q_size, self.kv_size = n_heads * head_dim, n_kv_heads * head_dim
        self.qkv_width = self.q_size + 2 * self.kv_size
        self.position = build_part("position", position, runtime)
        self.w_qkv = runtime.empty(self.qkv_width, hidden)
        self.b_qkv = runtime.empty(self.qkv_width, dtype=torch.float32) if qkv_bias else None
        self.w_o = runtime.empty(hidden, self.q_size)

    def weights(self) -> list[WeightDecl]:
        q, kv = self.q_size, self.kv_size
        spans = (("q_proj", 0, q), ("k_proj", q, q + kv), ("v_proj", q + kv, q + 2 * kv))
        decls = [WeightDecl(f"{n}.weight", (e - b, self.hidden), dest=self.w_qkv[b:e]) for n, b, e in spans]
        if self.b_qkv is not None:
            decls += [WeightDecl(f"{n}.bias", (e - b,), role="vector", dest=self.b_qkv[b:e]) for n, b, e in spans]
        decls.append(WeightDecl("o_proj.weight", (self.hidden, self.q_size), dest=self.w_o))
        return decls

    def cache_need(self) -> PagedKV:
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, ctx: StepContext, h: torch.Tensor, cache, write_cache: bool):
        if not isinstance(cache, PagedView):
            raise TypeError("gqa_attention needs a paged key/value cache")
        return self.project_out(ctx, self.attend(ctx, self.project_qkv(ctx, h, cache), cache, write_cache))

    def _fused_decode(self, ctx: StepContext):
        """The rotation table, if this step's attention kernel adds the bias, rotates, writes the new key and value
        and attends all by itself (decode-only steps in bfloat16 with a rotary encoding); else None."""
        table = self.position.fused_rotary_table(self.head_dim)
        if (table is not None and ctx.decode_only and ops.fused_decode_enabled()
                and ops.tensor_core_attention_supported(self.runtime.dtype, self.head_dim)):
            return table
        return None

    def project_qkv(self, ctx: StepContext, h: torch.Tensor, cache: PagedView | None = None):
        """h @ [Wq; Wk; Wv].T without the bias: a tensor, or the slices of a split product where the kernel
        that follows adds them itself (both rotary kernels do).  With the cache the attention will read, the
        product knows how large that launch will be and lets a small one settle on the SMs while it runs."""
        rotary = self.position.fused_rotary_table(self.head_dim) is not None
        fused = self._fused_decode(ctx) is not None
        early = False
        if fused and cache is not None:
            tma, nsplit, blocks = self._decode_launch(ctx, cache)
            early = tma and ops.decode_attention_resident_early(blocks, nsplit)
        # the decode kernel reads the product once per block: up to four slices are one round trip to L2 for it
        return linear(ctx, "attn.qkv", h, self.w_qkv, allow_split=rotary, max_slices=4 if fused else 12,
                      consumer_early=early)

    def _decode_launch(self, ctx: StepContext, cache: PagedView) -> tuple[bool, int, int]:
        """(fed by TMA?, slices per request, blocks) of the decode attention this step will launch."""
        group = self.n_heads // self.n_kv_heads
        tma = ops.decode_tma_supported(self.runtime.dtype, self.head_dim, cache.page_size)
        splits = ops.decode_tma_splits if tma else ops.decode_splits
        nsplit = splits(ctx.n_seqs, self.n_kv_heads, group, ctx.max_kv_len)
        return tma, nsplit, ctx.n_seqs * self.n_kv_heads * -(-group // 8) * nsplit

    def project_out(self, ctx: StepContext, out: torch.Tensor):
        return linear(ctx, "mixer.delta", out, self.w_o, allow_split=True, consumer_early=True,
                      prefetch=self._prefetch_plan(ctx)[1])

    def _prefetch_plan(self, ctx: StepContext):
        """What a decode-only step asks into L2 ahead of its kernel, of the weights the part after this one
        streams first (``ctx.upcoming_weights``): (the attention kernel's share, the output product's share).
        While the attention's slices merge and while the output product ends, the memory system has little to do.
        Not this part's own output matrix (the product that reads it starts fetching it before the attention has
        ended); and the attention only asks where its keys take longer to read than the output matrix, else the
        two fetches collide."""
        upcoming = ctx.upcoming_weights
        if upcoming is None or self._fused_decode(ctx) is None:
            return None, None
        window = self.window or 0
        keys = min(ctx.max_kv_len, window) if window else ctx.max_kv_len
        cache_bytes = ctx.n_seqs * keys * 2 * self.n_kv_heads * self.head_dim * self.w_qkv.element_size()   # the cache has the weights' type
        first = ops.weight_prefetch_bytes() if cache_bytes >= ops.weight_prefetch_min_cache_bytes() else 0
        return (ops.weight_head(upcoming, first),
                ops.weight_head(upcoming, ops.output_product_prefetch_bytes(), skip_bytes=first))

    def attend(self, ctx: StepContext, qkv, cache: PagedView, write_cache: bool) -> torch.Tensor:
        """Bias, position encoding, cache write and attention for the step's rows; [rows, Hq * D]."""
        n, ws, dt = ctx.n_tokens, ctx.workspace, self.runtime.dtype
        table = self.position.fused_rotary_table(self.head_dim)
        source = None
        if isinstance(qkv, SplitSum):       # the kernels below add the slices themselves
            source, qkv = qkv, ws.get("attn.qkv", (n, self.qkv_width), dt)
        out = ws.get("attn.out", (n, self.q_size), dt)
        if self._fused_decode(ctx) is not None:
            # decode-only step: the attention kernel adds the bias, rotates, writes the new key and value and attends
            self._decode(ctx, out, None, cache, fused=(source if source is not None else qkv, table, write_cache))
            return out
        if table is None:
            # generic path: bias, then the position part's own transformation, then the cache write
            if self.b_qkv is not None:
                ops.rotate_heads(qkv, self.b_qkv, ctx.positions, ctx.seq_of_token, None, n,
                                 self.n_heads + 2 * self.n_kv_heads, self.head_dim)
            self.position.apply(ctx, qkv, self.n_heads + self.n_kv_heads, self.head_dim)
            bias = None
        else:
            bias = self.b_qkv
        ops.rope_kv_write(qkv, bias, ctx.positions, ctx.seq_of_token, ctx.seq_slot, cache.block_table, table,
                          cache.k_pages, cache.v_pages, n, self.n_heads, self.n_kv_heads, self.head_dim,
                          write_cache, ctx.status, source=source)
        self._attend(ctx, out, qkv, cache)
        return out

    def _attend_tensor_cores(self, ctx: StepContext, out: torch.Tensor, q: torch.Tensor, cache: PagedView) -> None:
        """bfloat16: flash attention for requests with several tokens, split-KV attention for
        requests with one; both read the same flat batch and skip the other's requests."""
        window = self.window or 0
        singles = ctx.decode_only or ctx.fixed_shape or any(n == 1 for n in ctx.host_q_len)
        if not ctx.decode_only:
            # long portions: tcgen05 kernel (TMA, accumulators in tensor memory); short ones, and the shapes it
            # does not take, stay on the mma.sync kernel, which starts faster
            prefill = ops.attention_prefill
            if ops.prefer_tcgen05_attention(self.runtime.dtype, self.head_dim, cache.k_pages.shape[2], ctx.max_q_len):
                prefill = ops.attention_prefill_tcgen05
            prefill(out, q, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len, ctx.seq_slot,
                                  cache.block_table, cache.k_pages, cache.v_pages, ctx.n_seqs, ctx.max_q_len,
                                  self.n_heads, self.n_kv_heads, self.head_dim, window, self.scale, singles, ctx.status)
        if singles:
            self._decode(ctx, out, q, cache)

    def _decode(self, ctx: StepContext, out: torch.Tensor, q: torch.Tensor | None, cache: PagedView, fused=None) -> None:
        """Split-KV attention for the requests that bring one token; with ``fused`` = (product, rotation table,
        write_cache) the kernel makes q, k and v of the new token from the product itself.  Head sizes that are
        multiples of 64 take the kernel that is fed by TMA, the others the one that loads keys through registers."""
        group = self.n_heads // self.n_kv_heads
        tma, nsplit, _ = self._decode_launch(ctx, cache)
        scratch = ctx.workspace.get("attn.decode_scratch", (ops.decode_scratch_floats(self.n_heads, self.head_dim),),
                                    torch.float32)
        counters = ctx.workspace.get(
            "attn.decode_counters", (ops.decode_counter_ints(ctx.n_seqs, self.n_kv_heads, group),), torch.int32, zero=True)
        window = self.window or 0
        product, table, write_cache = fused if fused is not None else (None, None, False)
        prefetch = self._prefetch_plan(ctx)[0] if fused is not None else None
        if tma:
            ops.attention_decode_tma(out, q, product, self.b_qkv if fused is not None else None, table, write_cache,
                                     ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len, ctx.seq_slot, cache.block_table,
                                     cache.k_pages, cache.v_pages, ctx.n_seqs, self.n_heads, self.n_kv_heads, self.head_dim,
                                     window, self.scale, nsplit, scratch, counters, ctx.status, prefetch=prefetch)
        elif fused is not None:
            ops.attention_decode_fused(out, product, self.b_qkv, table, write_cache, ctx.seq_q_start, ctx.seq_q_len,
                                       ctx.seq_kv_len, ctx.seq_slot, cache.block_table, cache.k_pages, cache.v_pages,
                                       ctx.n_seqs, self.n_heads, self.n_kv_heads, self.head_dim, window, self.scale,
                                       nsplit, scratch, counters, ctx.status, prefetch=prefetch)
        else:
            ops.attention_decode(out, q, ctx.seq_q_start, ctx.seq_q_len, ctx.seq_kv_len, ctx.seq_slot,
                                 cache.block_table, cache.k_pages, cache.v_pages, ctx.n_seqs, self.n_heads,
                                 self.n_kv_heads, self.head_dim, window, self.scale, nsplit, scratch, counters,
                                 ctx.status)

    def _attend(self, ctx: StepContext, out: torch.Tensor, qkv: torch.Tensor, cache: PagedView) -> None:
        q = qkv[:, : self.q_size]
        if ops.tensor_core_attention_supported(self.runtime.dtype, self.head_dim):
            self._attend_tensor_cores(ctx, out, q, cache)
            return
        ops.attention_generic(out, q, ctx.positions, ctx.seq_of_token, ctx.seq_slot, cache.block_table,
                              cache.k_pages, cache.v_pages, ctx.n_tokens, self.n_heads, self.n_kv_heads,
                              self.head_dim, self.window or 0, self.scale, ctx.status)
