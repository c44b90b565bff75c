"""Matrix products ``out = x @ w.T`` (w stored [out_features, in_features], as nn.Linear).

The reference's engine runs its projections through a library (nn.Linear, i.e.
cuBLAS: flow_engine/model.py:39-43,71-73,108); so does this function where no
hand-written kernel takes the shape.  float32 products run in true fp32: TF32 and
every other reduced-precision matrix mode is switched off before the first call.
bfloat16 products accumulate in fp32 (no reduced-precision split-K sums).
"""
from __future__ import annotations

import torch

from ..csrc import ops
from ..csrc.ops import SplitSum

_configured = False


def configure_matmul_precision() -> None:
    """No TF32 in fp32 products, no bf16 accumulation in bf16 products."""
    global _configured
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")
    torch.backends.cuda.matmul.allow_bf16_reduced_precision_reduction = False
    _configured = True


def verify_true_fp32(device) -> None:
    """Raise unless the library's float32 product is a true 32-bit one on ``device``.

    Every element is 1 + 2**-12: exact in float32, rounded to 1 by any mode that shortens the
    operands (TF32 keeps 10 bits, bfloat16 7).  The sum of 256 squares is 256.125 in 32 bits and
    256 otherwise.  Run once per float32 runner, after the switches above: a reduced mode left on by
    an environment variable or by an earlier user of the process would put errors of 1e-3 into every
    logit, which no later test could tell from a fault of the model."""
    configure_matmul_precision()
    a = torch.full((48, 256), 1.0 + 2.0 ** -12, dtype=torch.float32, device=device)
    got = torch.mm(a, a.t())
    worst = float((got - 256.125).abs().max())
    if not worst < 1e-3:
        raise RuntimeError(f"float32 matrix products are not computed in 32 bits on {device} "
                           f"(256 x (1 + 2**-12)**2 came out {float(got[0, 0])!r}); a reduced-precision matrix mode is on")


def matmul_nt(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """out[n, o] = sum_i x[n, i] * w[o, i].  x and w are of one element type; out is of the
    same type, or fp32 for a bf16 product whose result must not be rounded (the logits)."""
    if not _configured:
        configure_matmul_precision()
    if not x.is_cuda:
        raise RuntimeError("matrix products run on the GPU only; this engine has no CPU path")
    ops.note_call("library product (cuBLAS)")
    if out.dtype != x.dtype:
        torch.mm(x, w.t(), out_dtype=out.dtype, out=out)
    else:
        torch.mm(x, w.t(), out=out)
    return out


def linear(ctx, name: str, x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype | None = None,
           allow_split: bool = False, consumer_early: bool = False, max_slices: int = 12,
           prefetch: torch.Tensor | None = None):
    """``x @ w.T`` into the workspace buffer ``name``.

    Steps with up to 8 rows (decode) in bfloat16 go through the weight-streaming kernel of
    csrc/gemm_smallm.cu; products of 9 to 64 rows with a large matrix (down, logits) through the persistent
    tcgen05 kernel of csrc/gemm_tcgen05_stream.cu.
    When the matrix has too few rows to fill the GPU these kernels split k and, if the caller can take it
    (``allow_split``), the fp32 slices are returned as a ``SplitSum`` for the consuming kernel
    to add.  Everything else is a library product.  ``consumer_early``: the weight-streaming kernel lets the kernel
    that follows become resident while it runs (that kernel waits for the result itself).  It pays where the
    follower is small (a norm, a sampler) or leaves most of the GPU free; the caller knows which.
    ``max_slices``: the most slices the consumer of a ``SplitSum`` wants to add.  ``prefetch``: weights of a
    later kernel that the weight-streaming kernels ask into L2 when their own stream ends (the library ignores it).
    """
    m, n = x.shape[0], w.shape[0]
    dtype = out_dtype or x.dtype
    if ops.stream_product_preferred(x, w, m):
        # decode steps of 9 to 64 requests, large matrices: the weights stream once through the persistent
        # tcgen05 kernel (csrc/gemm_tcgen05_stream.cu); slices only where the consumer adds them itself
        split, kper = ops.stream_split(n, w.shape[1])
        if split > 1 and allow_split:
            slices = ctx.workspace.get(name + ".slices", (split, m, n), torch.float32)
            ops.gemm_tcgen05_stream(slices, x, w, m, ctx.status, kper=kper, early_dependents=consumer_early,
                                    prefetch=prefetch)
            return SplitSum(slices)
        if split == 1:
            out = ctx.workspace.get(name, (m, n), dtype)
            ops.gemm_tcgen05_stream(out, x, w, m, ctx.status, early_dependents=consumer_early, prefetch=prefetch)
            return out
        # slices that nobody would add: the library's product below, which reduces its own split inside the kernel
    if x.is_cuda and ops.small_m_supported(x, w, m):
        split, kper = ops.small_m_split(n, w.shape[1], max_slices if allow_split else 12)
        if split > 1 and allow_split:
            slices = ctx.workspace.get(name + ".slices", (split, m, n), torch.float32)
            ops.gemm_small_m(slices, x, w, m, kper, early_dependents=consumer_early, prefetch=prefetch)
            return SplitSum(slices)
        if split > 1:
            slices = ctx.workspace.get(name + ".slices", (split, m, n), torch.float32)
            ops.gemm_small_m(slices, x, w, m, kper)
            return SplitSum(slices).dense(dtype, ctx.workspace.get(name, (m, n), dtype))
        out = ctx.workspace.get(name, (m, n), dtype)
        ops.gemm_small_m(out, x, w, m, early_dependents=consumer_early, prefetch=prefetch)
        return out
    return matmul_nt(ctx.workspace.get(name, (m, n), dtype), x, w)
