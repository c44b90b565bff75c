"""Per-kernel timings of one decoder layer and the output head, each with its roofline.

Every operation of a decode step (few rows) and of a prompt step (many rows) is run alone, the
way the engine runs it (the same wrappers, the same routing between hand-written kernels and the
library), inside a CUDA graph and with its large operands rotated through more copies than the
L2 cache holds, so that a timing is neither launch-bound nor cache-resident.  A row gives the
bytes the operation has to move, its FLOPs, the time, and

    fraction = max(bytes / HBM peak, FLOPs / tensor peak) / time.

``python bench.py --kernels`` prints the table.
"""
from __future__ import annotations

from types import SimpleNamespace

import torch

from ..csrc import ops
from ..csrc.ops import SplitSum
from ..parts.base import Workspace
from ..parts.linear import linear

L2_BYTES = 126 * 1024 * 1024


def _graph_us(calls, reps: int = 4) -> float:
    """Microseconds per call of ``calls`` (a list of thunks, run round robin) inside a CUDA graph."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        for f in calls:
            f()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(reps):
                for f in calls:
                    f()
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(3):
            graph.replay()
        end.record()
        torch.cuda.synchronize()
    return begin.elapsed_time(end) / (3 * reps * len(calls)) * 1000.0


def _copies(nbytes: int) -> int:
    return max(2, min(16, -(-3 * L2_BYTES // max(1, nbytes))))


def kernel_table(cfg, batch: int, context: int, prefill_tokens: int, hbm_gbs: float, tflops: float,
                 page_size: int = 16, only: tuple[str, ...] | None = None) -> list[dict]:
    """All rows, or with ``only`` the rows whose operation name contains one of the given words."""
    dev = torch.device("cuda")
    bf = torch.bfloat16
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    qkv_w = (Hq + 2 * Hkv) * D
    rows: list[dict] = []
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)   # noqa: E731

    def want(name: str) -> bool:
        return only is None or any(word in name for word in only)

    def add(name, rows_m, us, nbytes, flops, kernel):
        floor = max(nbytes / (hbm_gbs * 1e9), flops / (tflops * 1e12)) * 1e6
        rows.append({"op": name, "rows": rows_m, "kernel": kernel, "us": round(us, 2), "mbytes": round(nbytes / 1e6, 2),
                     "gflop": round(flops / 1e9, 2), "floor_us": round(floor, 2), "frac": round(floor / us, 3),
                     "bound": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / (tflops * 1e12) else "tensor"})

    def product(name, m, n, k, fused_silu=False, out_dtype=None):
        """x[m, k] @ w[n, k].T the way the engine runs it; weights rotated beyond L2.  With ``fused_silu`` the
        weights are gate/up rows and the step's SiLU.mul is part of the row where a kernel fuses it."""
        fused = None
        x = torch.randn(m, k, device=dev, dtype=bf)
        probe = torch.empty(n, k, device=dev, dtype=bf)
        if fused_silu and m <= ops.SMALL_M_LIMIT:
            fused = "small"
        elif fused_silu and ops.stream_product_preferred(x, probe, m) and ops.stream_whole_k_balanced(n):
            fused = "stream"
        elif fused_silu and ops.pair_product_preferred(x, probe, m):
            fused = "pair"
        del probe
        if fused:
            name += " + SiLU.mul"
        if not want(name):
            return
        copies = _copies(n * k * 2)
        ws = [torch.randn(n, k, device=dev, dtype=bf) * 0.02 for _ in range(copies)]
        ctx = SimpleNamespace(workspace=Workspace(dev), status=status)
        out_cols = n
        if fused == "small":
            out_cols = n // 2
            out = torch.empty(m, out_cols, device=dev, dtype=bf)
            calls = [(lambda w=w: ops.gemm_small_m(out, x, w, m, silu_mul_pairs=True)) for w in ws]
            kernel = "gemm_smallm"
        elif fused == "stream":
            out_cols = n // 2
            out = torch.empty(m, out_cols, device=dev, dtype=bf)
            calls = [(lambda w=w: ops.gemm_tcgen05_stream(out, x, w, m, status, silu_mul_pairs=True)) for w in ws]
            kernel = "gemm_tcgen05_stream"
        elif fused == "pair":
            out_cols = n // 2
            out = torch.empty(m, out_cols, device=dev, dtype=bf)
            calls = [(lambda w=w: ops.gemm_tcgen05_pair(out, x, w, m, status, silu_mul_pairs=True)) for w in ws]
            kernel = "gemm_tcgen05_pair (2-CTA)"
        else:
            calls = [(lambda w=w: linear(ctx, "p", x, w, out_dtype=out_dtype, allow_split=True)) for w in ws]
            kernel = ("gemm_smallm" if m <= ops.SMALL_M_LIMIT else
                      "gemm_tcgen05_stream" if ops.stream_product_preferred(x, ws[0], m) else
                      "gemm_tcgen05 (swap-AB)" if ops.tcgen05_supported(x, ws[0], m) else "library (cuBLAS)")
        us = _graph_us(calls)
        out_bytes = m * out_cols * (4 if out_dtype == torch.float32 else 2)
        add(name, m, us, n * k * 2 + m * k * 2 + out_bytes, 2.0 * m * n * k, kernel)
        del ws
        if fused_silu and not fused and want(name.split(":")[0] + ": SiLU.mul"):
            gu = torch.randn(m, n, device=dev, dtype=bf)
            act = torch.empty(m, n // 2, device=dev, dtype=bf)
            us = _graph_us([lambda: ops.silu_mul(act, gu, m, True)], reps=4)
            add(name.split(":")[0] + ": SiLU.mul", m, us, m * (n // 2) * 2 * 3, 0.0, "silu_mul")

    for m, phase in ((batch, "decode"), (prefill_tokens, "prefill")):
        elementwise = only is None or any(want(f"{phase}: {t}") for t in ("residual add + RMSNorm", "bias + RoPE + cache write",
                                                                          "attention"))
        if elementwise:
            resid = torch.randn(m, H, device=dev)
            delta = torch.randn(m, H, device=dev, dtype=bf)
            weight = torch.ones(H, device=dev)
            out = torch.empty(m, H, device=dev, dtype=bf)
            us = _graph_us([lambda: ops.add_rmsnorm(out, resid, delta, weight, cfg.rms_norm_eps, m)], reps=8)
            add(f"{phase}: residual add + RMSNorm", m, us, m * H * (4 + 4 + 2 + 2), 0.0, "add_rmsnorm")
        product(f"{phase}: qkv product", m, qkv_w, H)
        if elementwise:
            # bias + RoPE + cache write, and attention
            pages = -(-context // page_size) * batch if phase == "decode" else -(-m // page_size)
            kp = torch.zeros(pages, Hkv, page_size, D, device=dev, dtype=bf)
            vp = torch.zeros_like(kp)
            qkv = torch.randn(m, qkv_w, device=dev, dtype=bf)
            bias = torch.randn(qkv_w, device=dev)
            inv = (cfg.rope_theta ** (-torch.arange(0, D, 2, dtype=torch.float32) / D)).to(dev)
            if phase == "decode":
                blocks = -(-context // page_size)
                table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(batch, blocks)
                positions, seq_of = i32([context - 1] * m), i32(list(range(m)))
                slots = i32(list(range(batch)))
            else:
                table = torch.arange(pages, dtype=torch.int32, device=dev).reshape(1, pages)
                positions = torch.arange(m, dtype=torch.int32, device=dev)
                seq_of = torch.zeros(m, dtype=torch.int32, device=dev)
                slots = i32([0])
            if phase == "prefill":
                us = _graph_us([lambda: ops.rope_kv_write(qkv, bias, positions, seq_of, slots, table, inv, kp, vp, m, Hq, Hkv, D,
                                                          True, status)], reps=8)
                add(f"{phase}: bias + RoPE + cache write", m, us, m * qkv_w * 2 * 2, 0.0, "rope_kv_write")
                q = torch.randn(m, Hq * D, device=dev, dtype=bf)
                ao = torch.empty_like(q)
                kp.normal_(); vp.normal_()
                args = (i32([0]), i32([m]), i32([m]), slots, table, kp, vp, 1, m, Hq, Hkv, D, 0, D ** -0.5, False, status)
                tc5 = ops.prefer_tcgen05_attention(bf, D, page_size, m)
                fn = ops.attention_prefill_tcgen05 if tc5 else ops.attention_prefill
                us = _graph_us([lambda: fn(ao, q, *args)], reps=4)
                add(f"prefill: causal attention, {m} tokens", m, us, m * (Hq + 2 * Hkv) * D * 2 + m * Hq * D * 2,
                    4.0 * Hq * D * m * (m + 1) / 2, "attn_prefill_tc5 (tcgen05)" if tc5 else "attn_prefill (mma.sync)")
            else:
                # decode-only steps: one kernel adds the bias, rotates, writes the new key and value and attends
                nset = _copies(kp.numel() * 2 * 2)
                sets = [(torch.randn_like(kp), torch.randn_like(vp)) for _ in range(nset)]
                ao = torch.empty(m, Hq * D, device=dev, dtype=bf)
                qs, ql, kl = i32(list(range(m))), i32([1] * m), i32([context] * m)
                ns = ops.decode_splits(m, Hkv, Hq // Hkv, context)
                scratch = torch.empty(ops.decode_scratch_floats(Hq, D), device=dev)
                counters = torch.zeros(ops.decode_counter_ints(m, Hkv, Hq // Hkv), dtype=torch.int32, device=dev)
                nsl, _ = ops.small_m_split(qkv_w, H)
                source = SplitSum(torch.randn(nsl, m, qkv_w, device=dev)) if nsl > 1 else qkv
                calls = [(lambda k=k, v=v: ops.attention_decode_fused(ao, source, bias, inv, True, qs, ql, kl, slots, table, k, v, m,
                                                                      Hq, Hkv, D, 0, D ** -0.5, ns, scratch, counters, status))
                         for k, v in sets]
                us = _graph_us(calls)
                add(f"decode: bias + RoPE + cache write + attention over {context} keys", m, us,
                    m * context * Hkv * D * 2 * 2 + nsl * m * qkv_w * 4, 4.0 * m * Hq * D * context,
                    f"attn_decode fused ({ns} slices)")
                del sets
            del kp, vp
        product(f"{phase}: o_proj product", m, H, Hq * D)
        product(f"{phase}: gate/up product", m, 2 * I, H, fused_silu=True)
        product(f"{phase}: down product", m, H, I)
    product("decode: output matrix (logits, fp32)", batch, V, H, out_dtype=torch.float32)
    if want("decode: greedy sampling"):
        logits = torch.randn(batch, V, device=dev)
        ids = torch.zeros(batch, dtype=torch.int32, device=dev)
        us = _graph_us([lambda: ops.sample(ids, logits, batch)], reps=8)
        add("decode: greedy sampling", batch, us, batch * V * 4, 0.0, "sample")
    if int(status) != 0:
        raise RuntimeError(f"a kernel reported status {int(status)} during the kernel table")
    return rows


def format_table(rows: list[dict]) -> str:
    head = f"{'operation':62s} {'rows':>5s} {'kernel':28s} {'us':>9s} {'MB':>9s} {'GFLOP':>9s} {'floor us':>9s} {'frac':>6s}"
    lines = [head, "-" * len(head)]
    for r in rows:
        lines.append(f"{r['op']:62s} {r['rows']:5d} {r['kernel']:28s} {r['us']:9.2f} {r['mbytes']:9.2f} {r['gflop']:9.2f} "
                     f"{r['floor_us']:9.2f} {r['frac']:6.3f}")
    return "\n".join(lines)
