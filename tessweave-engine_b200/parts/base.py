"""Interfaces of the parts a model is put together from, and their registries.

A model is an embedding, a list of blocks, a final norm and an output head; a block
arranges a mixer, a feed-forward and their norms; a mixer may use a position
encoding.  Every part gets its sizes and constants as parameters, declares the
weights it wants by name, says what cache it needs, and runs on the rows of a step.
No part knows which model it is in.

A part kind is registered under a name in its category; a model description
(``ModelSpec``) names kinds and parameters only, so a new embedding, mixer,
feed-forward, norm, position encoding or head is added by registering it: no
framework file changes.

What a sub-layer hands to the residual stream is a *delta*: a tensor ``[rows, width]``
of the activation type, or a ``SplitSum`` -- the fp32 slices of a matrix product that
was split over k, whose sum is the delta.  A producer may return either; a consumer
that cannot add slices itself calls ``dense_delta`` first.  Nobody has to know who
comes next.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from ..csrc.ops import SplitSum


# ---------------------------------------------------------------------------
# what a part is described by
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class PartSpec:
    """Kind name plus keyword parameters of one part."""
    kind: str
    params: dict = field(default_factory=dict)

    def with_params(self, **more) -> "PartSpec":
        return PartSpec(self.kind, {**self.params, **more})


@dataclass
class WeightDecl:
    """One tensor a part expects from the checkpoint.

    ``name`` is relative to the part's prefix.  ``role`` decides how it is kept:
    ``matrix`` in the run's element type, ``vector`` always in fp32 (a tensor stored
    in 32 bits stays so; bf16 widens exactly), ``table_int`` in int32.  ``dest`` is
    the device storage the loader copies into, usually a slice of a packed buffer.
    ``init`` is the random-weights rule: ``normal`` ~ N(0, std), ``one_plus_normal``
    ~ 1 + N(0, 0.1), ``zeros``.
    """
    name: str
    shape: tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    dest: torch.Tensor | None = None


# ---------------------------------------------------------------------------
# what a part may need from the cache manager
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class PagedKV:
    """Keys and values for every token (or the last ``window`` tokens), in pages."""
    kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class FixedState:
    """A state of fixed size per request (``numel`` elements of ``dtype``)."""
    numel: int
    dtype: torch.dtype = torch.float32


# ---------------------------------------------------------------------------
# run-time handles
# ---------------------------------------------------------------------------
@dataclass
class Runtime:
    """Where and in which element type a model lives."""
    device: torch.device
    dtype: torch.dtype

    def empty(self, *shape, dtype=None) -> torch.Tensor:
        return poisoned(torch.empty(*shape, dtype=dtype or self.dtype, device=self.device))


def poison_new_buffers() -> bool:
    """TESSWEAVE_POISON_BUFFERS=1 (the tests set it): every buffer that is allocated without a value --
    workspace, weight storage before loading -- is filled with NaN (integers with a large negative
    number), so that a kernel that reads what nobody wrote gives NaN instead of whatever the memory held.
    Fresh device memory is often zero, or holds the same values an earlier run left there, and hides
    such a read."""
    return os.environ.get("TESSWEAVE_POISON_BUFFERS", "0") == "1"


def poisoned(t: torch.Tensor) -> torch.Tensor:
    if poison_new_buffers():
        t.fill_(float("nan") if t.is_floating_point() else -(2 ** 30))
    return t


class Workspace:
    """Named scratch tensors that only ever grow; shared by all parts of a model.

    A buffer asked for under one name is reused by every layer, so the memory of a
    step does not grow with depth, and addresses stay fixed for CUDA graphs.
    """

    def __init__(self, device: torch.device):
        self.device = device
        self._buffers: dict[str, torch.Tensor] = {}
        self.frozen = False

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype, zero: bool = False) -> torch.Tensor:
        """The buffer ``name`` with at least ``shape`` elements.  ``zero`` fills it with zeros when it
        is (re)allocated -- for state that kernels keep zero between launches, such as counters."""
        numel = 1
        for s in shape:
            numel *= int(s)
        buf = self._buffers.get(name)
        if buf is None or buf.dtype != dtype or buf.numel() < numel:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow while a CUDA graph holds its address")
            if zero:
                buf = torch.zeros(max(numel, 1), dtype=dtype, device=self.device)
            else:
                buf = poisoned(torch.empty(max(numel, 1), dtype=dtype, device=self.device))
            self._buffers[name] = buf
        return buf[:numel].view(*shape)

    def reserve(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> None:
        self.get(name, shape, dtype)

    def bytes(self) -> int:
        return sum(b.numel() * b.element_size() for b in self._buffers.values())


@dataclass
class PagedView:
    """One cache layer of a paged group, as a mixer sees it."""
    k_pages: torch.Tensor          # [pages, kv_heads, page_size, head_dim]
    v_pages: torch.Tensor
    block_table: torch.Tensor      # int32 [request slots, max blocks], -1 where no page is held
    page_size: int
    window: int | None
    host_tables: Any = None        # callable slot -> list[int], for parts that want the table on the host


@dataclass
class StateView:
    """One cache layer of fixed-size per-request state."""
    state: torch.Tensor            # [request slots, numel]


@dataclass
class StepContext:
    """Everything a part may read about the step that is running.

    Device tensors are int32.  ``n_tokens`` rows are live; rows beyond belong to the
    padding of a fixed-size (graph) batch and have ``seq_of_token == -1``.
    """
    runtime: Runtime
    workspace: Workspace
    n_tokens: int                  # rows in this step (including padding rows)
    n_seqs: int
    token_ids: torch.Tensor        # [n_tokens]
    positions: torch.Tensor        # [n_tokens] absolute position of each row in its request
    seq_of_token: torch.Tensor     # [n_tokens] index into the per-sequence arrays, -1 = padding
    seq_slot: torch.Tensor         # [n_seqs] request slot (row of block tables and state)
    seq_q_start: torch.Tensor      # [n_seqs] first row of the sequence in this step
    seq_q_len: torch.Tensor        # [n_seqs] rows of the sequence in this step
    seq_kv_len: torch.Tensor       # [n_seqs] tokens the request holds after this step
    status: torch.Tensor           # int32 [1] error bits written by kernels
    # host copies of the per-sequence arrays, for parts that loop on the host
    host_slot: list[int] = field(default_factory=list)
    host_q_start: list[int] = field(default_factory=list)
    host_q_len: list[int] = field(default_factory=list)
    host_kv_len: list[int] = field(default_factory=list)
    max_q_len: int = 1
    max_kv_len: int = 1
    decode_only: bool = False      # every sequence brings exactly one token
    fixed_shape: bool = False      # the launch is being captured: sizes must not depend on host values of this step
    device_tokens: torch.Tensor | None = None   # int32: token ids the previous step left on the device (id -(i+1) -> [i])
    upcoming_weights: torch.Tensor | None = None  # set by a block: what the part after the running one streams first


# ---------------------------------------------------------------------------
# part base classes
# ---------------------------------------------------------------------------
class Part:
    """Common behaviour: parameters in, weight declarations out."""
    graph_safe = True   # False if forward() syncs with the host or allocates

    def __init__(self, runtime: Runtime):
        self.runtime = runtime

    def weights(self) -> list[WeightDecl]:
        return []

    def redundant_names(self) -> list[str]:
        """Tensors a checkpoint may carry for this part that are not loaded because the part gets them
        another way (a tied head's copy of the embedding matrix).  Relative to the part's prefix."""
        return []

    def finalize(self) -> None:
        """Called once after every declared weight has been filled."""

    def streamed_first(self) -> torch.Tensor | None:
        """The contiguous weight this part's forward reads first and from end to end, or None.  A part that runs
        before it may ask the memory system to bring its head into L2 while its own last blocks finish."""
        return None

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for w in self.weights():
            if w.dest is not None:
                base = w.dest.untyped_storage().data_ptr()
                if (base, w.dest.storage_offset()) not in seen:
                    seen.add((base, w.dest.storage_offset()))
                    total += w.dest.numel() * w.dest.element_size()
        return total


def dense_delta(ctx: "StepContext", delta, dtype: torch.dtype, name: str = "delta.dense"):
    """``delta`` as a tensor: a ``SplitSum`` is added up (in slice order) into a workspace buffer."""
    if isinstance(delta, SplitSum):
        _, rows, width = delta.slices.shape
        return delta.dense(dtype, ctx.workspace.get(name, (rows, width), dtype))
    return delta


class Embedding(Part):
    """Turns the token ids of a step into the rows of the residual stream."""

    def forward(self, ctx: "StepContext") -> "ResidualStream":
        raise NotImplementedError

    def shared_matrix(self) -> torch.Tensor | None:
        """The [vocab, hidden] matrix an output head may share when the model ties the two, or None."""
        return None


class Head(Part):
    """Turns normalised rows into fp32 logits."""

    def forward(self, ctx: "StepContext", logits: torch.Tensor, y: torch.Tensor, n_rows: int) -> None:
        """logits[:n_rows] = head(y[:n_rows]); logits is fp32 [>= n_rows, vocab]."""
        raise NotImplementedError


class Norm(Part):
    """out = norm(resid [+ delta]); updates the fp32 residual stream in place.

    ``delta`` is None, a tensor of the activation type, or a ``SplitSum``.  A norm whose kernel adds
    the slices itself sets ``accepts_split_sum``; callers go through ``apply``, which adds them up
    first for a norm that does not."""
    accepts_split_sum = False

    def apply(self, ctx: "StepContext", out: torch.Tensor, resid: torch.Tensor, delta, n_rows: int,
              rows: torch.Tensor | None = None) -> None:
        if not self.accepts_split_sum:
            delta = dense_delta(ctx, delta, out.dtype)
        self.forward(ctx, out, resid, delta, n_rows, rows)

    def forward(self, ctx: "StepContext", out: torch.Tensor, resid: torch.Tensor, delta, n_rows: int,
                rows: torch.Tensor | None = None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    """Encodes positions into queries and keys.

    ``apply`` rewrites the first ``n_heads`` heads of the packed rows (q heads, then k heads) in
    place; every encoding implements it, and a mixer needs to know nothing else.  An encoding that
    is a rotation by ``position * inv_freq[i]`` of the pairs ``(i, i + head_dim / 2)`` may also give
    that table through ``fused_rotary_table()``: a mixer that has a kernel which rotates while it
    does something else (writes the cache, attends) can then skip ``apply``.  ``None`` means
    "call apply()".
    """

    def apply(self, ctx: StepContext, qk: torch.Tensor, n_heads: int, head_dim: int) -> None:
        raise NotImplementedError

    def fused_rotary_table(self, head_dim: int) -> torch.Tensor | None:
        return None


class Mixer(Part):
    """Mixes information between the tokens of a request (attention here)."""

    def cache_need(self) -> PagedKV | FixedState | None:
        return None

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: PagedView | StateView | None,
                write_cache: bool):
        """h: [n_tokens, hidden] normalised rows.  Returns the delta for the residual stream
        (a tensor or a ``SplitSum``)."""
        raise NotImplementedError


class FeedForward(Part):
    """Token-wise transformation (dense or routed)."""

    def forward(self, ctx: StepContext, h: torch.Tensor):
        """Returns the delta for the residual stream (a tensor or a ``SplitSum``)."""
        raise NotImplementedError


class Block(Part):
    """Arrangement of a mixer and a feed-forward around the residual stream."""

    def forward(self, ctx: StepContext, stream: "ResidualStream", cache, write_cache: bool) -> None:
        raise NotImplementedError

    def parts(self) -> dict[str, Part]:
        raise NotImplementedError


@dataclass
class ResidualStream:
    """The fp32 residual rows plus a delta (tensor or ``SplitSum``) the next norm still has to add."""
    resid: torch.Tensor
    pending: object = None


# ---------------------------------------------------------------------------
# registries
# ---------------------------------------------------------------------------
CATEGORIES = ("embedding", "norm", "position", "mixer", "feed_forward", "block", "head")
_REGISTRY: dict[str, dict[str, Callable[..., Part]]] = {c: {} for c in CATEGORIES}


def register_part(category: str, kind: str):
    """Class decorator: make ``kind`` buildable in ``category``."""
    if category not in _REGISTRY:
        raise KeyError(f"unknown part category {category!r}; one of {CATEGORIES}")

    def deco(cls):
        _REGISTRY[category][kind] = cls
        cls.kind = kind
        return cls
    return deco


def build_part(category: str, spec: PartSpec, runtime: Runtime, **extra) -> Part:
    try:
        cls = _REGISTRY[category][spec.kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(category, {}))) or "none"
        raise KeyError(f"no {category} part of kind {spec.kind!r} is registered (known: {known})") from None
    return cls(runtime, **spec.params, **extra)


def registered(category: str) -> list[str]:
    return sorted(_REGISTRY[category])
