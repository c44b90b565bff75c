"""Per-operation timings of one decoder layer and the output head, each with its roofline.

Every operation of a decode step (few rows) and of a prompt step (many rows) is run alone by calling the
engine's own parts -- the attention part's ``project_qkv / attend / project_out``, the feed-forward's
``gate_up / down``, the norm, the head, the sampler -- built from the model's own spec, so whatever routing
between hand-written kernels and the library a part does, the table follows it; the name of the kernel that ran
is read from the launch log, not restated here.  Each call sits inside a CUDA graph, and the large operands
(weights, cache pages, activations of prompt steps) exist in more copies than the L2 cache holds and are used
in turn, so that a timing is neither launch-bound nor cache-resident.  A row gives the bytes the operation has
to move, its FLOPs, the time, and

    fraction = max(bytes / HBM peak, FLOPs / tensor peak) / time.

``python bench.py --kernels`` prints the table.
"""
from __future__ import annotations

import torch

from ..cache.manager import CacheManager
from ..csrc import ops
from ..parts.base import Runtime, StepContext, Workspace, build_part

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


def _kernels_of(thunk) -> str:
    """Run ``thunk`` once and name the launchers it called."""
    ops.CALL_LOG = []
    try:
        thunk()
        names = []
        for name in ops.CALL_LOG:
            name = name.removeprefix("tw_")
            if name not in names:
                names.append(name)
    finally:
        ops.CALL_LOG = None
    return " + ".join(names) or "none"


def _context(rt: Runtime, ws: Workspace, status, positions, seq_of_token, slots, q_start, q_len, kv_len) -> StepContext:
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=rt.device)   # noqa: E731
    return StepContext(runtime=rt, workspace=ws, n_tokens=len(positions), n_seqs=len(slots), token_ids=i32([0] * len(positions)),
                       positions=i32(positions), seq_of_token=i32(seq_of_token), seq_slot=i32(slots), seq_q_start=i32(q_start),
                       seq_q_len=i32(q_len), seq_kv_len=i32(kv_len), status=status, host_slot=list(slots),
                       host_q_start=list(q_start), host_q_len=list(q_len), host_kv_len=list(kv_len), max_q_len=max(q_len),
                       max_kv_len=max(kv_len), decode_only=all(c == 1 for c in q_len), fixed_shape=all(c == 1 for c in q_len))


def _fill(part, std: float = 0.02) -> None:
    for decl in part.weights():
        if decl.role == "matrix":
            decl.dest.normal_(0, std)
        elif decl.init == "one_plus_normal":
            decl.dest.fill_(1.0)
        else:
            decl.dest.normal_(0, std)
    part.finalize()


def kernel_table(spec, batch: int, context: int, prefill_tokens: int, hbm_gbs: float, tflops: float,
                 page_size: int = 16, only: tuple[str, ...] | None = None) -> list[dict]:
    """All rows for the first layer of ``spec`` (a ``ModelSpec``) and its head, or with ``only`` the rows whose
    operation name contains one of the given words."""
    dev = torch.device("cuda")
    bf = torch.bfloat16
    rt = Runtime(dev, bf)
    block_spec = spec.layers[0].block
    mixer_spec, ffn_spec, norm_spec = block_spec.params["mixer"], block_spec.params["feed_forward"], block_spec.params["norm1"]
    H, V = spec.hidden_size, spec.vocab_size
    rows: list[dict] = []
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def want(name: str) -> bool:
        return only is None or any(word in name for word in only)

    def add(name, rows_m, us, nbytes, flops, kernel):
        floor = max(nbytes / (hbm_gbs * 1e9), flops / (tflops * 1e12)) * 1e6
        rows.append({"op": name, "rows": rows_m, "kernel": kernel, "us": round(us, 2), "mbytes": round(nbytes / 1e6, 2),
                     "gflop": round(flops / 1e9, 2), "floor_us": round(floor, 2), "frac": round(floor / us, 3),
                     "bound": "hbm" if nbytes / (hbm_gbs * 1e9) >= flops / (tflops * 1e12) else "tensor"})

    def measure(name, m, thunks, nbytes, flops, reps=4):
        kernel = _kernels_of(thunks[0])
        add(name, m, _graph_us(thunks, reps), nbytes, flops, kernel)

    wants_mixer = any(want(f"{ph}: {t}") for ph in ("decode", "prefill") for t in ("qkv product", "attention", "o_proj product"))
    wants_ffn = any(want(f"{ph}: {t}") for ph in ("decode", "prefill") for t in ("gate/up product", "down product"))
    for m, phase in ((batch, "decode"), (prefill_tokens, "prefill")):
        ws = Workspace(dev)
        if phase == "decode":
            ctx = _context(rt, ws, status, [context - 1] * m, list(range(m)), list(range(m)), list(range(m)), [1] * m, [context] * m)
        else:
            ctx = _context(rt, ws, status, list(range(m)), [0] * m, [0], [0], [m], [m])
        act_copies = _copies(m * H * 2) if phase == "prefill" else 1
        hs = [torch.randn(m, H, device=dev, dtype=bf) for _ in range(act_copies)]
        # ---- residual add + norm
        if want(f"{phase}: residual add + RMSNorm"):
            norm = build_part("norm", norm_spec, rt)
            _fill(norm)
            n_sets = _copies(m * H * 12)
            sets = [(torch.randn(m, H, device=dev), torch.randn(m, H, device=dev, dtype=bf), torch.empty(m, H, device=dev, dtype=bf))
                    for _ in range(n_sets)]
            measure(f"{phase}: residual add + RMSNorm", m,
                    [(lambda r=r, d=d, o=o: norm.apply(ctx, o, r, d, m)) for r, d, o in sets], m * H * (4 + 4 + 2 + 2), 0.0, reps=8)
            del sets
        # ---- the mixer in its three stages
        if wants_mixer:
            first = build_part("mixer", mixer_spec, rt)
            weight_bytes = first.w_qkv.numel() * 2
            mixers = [first] + [build_part("mixer", mixer_spec, rt) for _ in range(_copies(weight_bytes) - 1)]
            for mx in mixers:
                _fill(mx)
            Hq, Hkv, D = first.n_heads, first.n_kv_heads, first.head_dim
            qkv_w = first.qkv_width
            if want(f"{phase}: qkv product"):
                measure(f"{phase}: qkv product", m, [(lambda mx=mx, i=i: mx.project_qkv(ctx, hs[i % len(hs)])) for i, mx in enumerate(mixers)],
                        qkv_w * H * 2 + m * H * 2 + m * qkv_w * 2, 2.0 * m * qkv_w * H)
            if want(f"{phase}: attention"):
                requests = batch if phase == "decode" else 1
                kv_tokens = context if phase == "decode" else m
                blocks = -(-kv_tokens // page_size)
                page_bytes = 2 * requests * blocks * page_size * Hkv * D * 2
                caches = []
                for _ in range(_copies(page_bytes)):
                    cache = CacheManager([(first.cache_need(), None)], page_size, requests * blocks, requests, kv_tokens, bf, dev,
                                         prefix_cache=False)
                    for g in cache.groups:
                        g.k.normal_(0, 0.5)
                        g.v.normal_(0, 0.5)
                    for _r in range(requests):
                        cache.ensure(cache.admit(None), kv_tokens)
                    cache.sync_tables()
                    caches.append(cache)
                products = [mixers[0].project_qkv(ctx, hs[0])]
                if isinstance(products[0], ops.SplitSum):
                    products = [ops.SplitSum(products[0].slices.clone())]
                else:
                    products = [products[0].clone() for _ in range(len(hs))]
                views = [c.view(0) for c in caches]
                thunks = [(lambda v=v, i=i: first.attend(ctx, products[i % len(products)], v, True)) for i, v in enumerate(views)]
                if phase == "decode":
                    slices = products[0].slices.shape[0] if isinstance(products[0], ops.SplitSum) else 0
                    measure(f"decode: bias + RoPE + cache write + attention over {context} keys", m, thunks,
                            m * context * Hkv * D * 2 * 2 + max(slices, 1) * m * qkv_w * (4 if slices else 2), 4.0 * m * Hq * D * context)
                else:
                    measure(f"prefill: bias + RoPE + cache write + causal attention, {m} tokens", m, thunks,
                            m * qkv_w * 2 * 2 + m * Hq * D * 2, 4.0 * Hq * D * m * (m + 1) / 2)
                del caches, views, thunks
            if want(f"{phase}: o_proj product"):
                outs = [torch.randn(m, first.q_size, device=dev, dtype=bf) for _ in range(act_copies)]
                measure(f"{phase}: o_proj product", m, [(lambda mx=mx, i=i: mx.project_out(ctx, outs[i % len(outs)])) for i, mx in enumerate(mixers)],
                        H * first.q_size * 2 + m * first.q_size * 2 + m * H * 2, 2.0 * m * H * first.q_size)
            del mixers, first
        # ---- the feed-forward in its two stages
        if wants_ffn:
            one = build_part("feed_forward", ffn_spec, rt)
            ffns = [one] + [build_part("feed_forward", ffn_spec, rt) for _ in range(_copies(one.w_gate_up.numel() * 2) - 1)]
            for f in ffns:
                _fill(f)
            inter = one.intermediate
            if want(f"{phase}: gate/up product"):
                measure(f"{phase}: gate/up product + SiLU.mul", m, [(lambda f=f, i=i: f.gate_up(ctx, hs[i % len(hs)])) for i, f in enumerate(ffns)],
                        2 * inter * H * 2 + m * H * 2 + m * inter * 2, 2.0 * m * 2 * inter * H)
            if want(f"{phase}: down product"):
                acts = [torch.randn(m, inter, device=dev, dtype=bf) * 0.1 for _ in range(_copies(m * inter * 2) if phase == "prefill" else 1)]
                measure(f"{phase}: down product", m, [(lambda f=f, i=i: f.down(ctx, acts[i % len(acts)])) for i, f in enumerate(ffns)],
                        H * inter * 2 + m * inter * 2 + m * H * 2, 2.0 * m * H * inter)
            del ffns, one
        del hs
        torch.cuda.empty_cache()
    # ---- the head and the sampler of a decode step
    ws = Workspace(dev)
    ctx = _context(rt, ws, status, [context - 1] * batch, list(range(batch)), list(range(batch)), list(range(batch)), [1] * batch,
                   [context] * batch)
    if want("decode: output matrix"):
        heads = [build_part("head", spec.head, rt) for _ in range(_copies(V * H * 2))]
        for hd in heads:
            _fill(hd)
        y = torch.randn(batch, H, device=dev, dtype=bf)
        logits = torch.empty(batch, V, device=dev)
        measure("decode: output matrix (logits, fp32)", batch, [(lambda hd=hd: hd.forward(ctx, logits, y, batch)) for hd in heads],
                V * H * 2 + batch * H * 2 + batch * V * 4, 2.0 * batch * V * H)
        del heads
    if want("decode: greedy sampling"):
        sets = [torch.randn(batch, V, device=dev) for _ in range(_copies(batch * V * 4))]
        ids = torch.zeros(batch, dtype=torch.int32, device=dev)
        measure("decode: greedy sampling", batch, [(lambda lg=lg: ops.sample(ids, lg, batch)) for lg in sets], batch * V * 4, 0.0, reps=8)
    if int(status) != 0:
        raise RuntimeError(f"a kernel reported status {int(status)} during the kernel table")
    return rows


def format_table(rows: list[dict]) -> str:
    width = max(28, max(len(r["kernel"]) for r in rows))
    head = f"{'operation':66s} {'rows':>5s} {'kernel':{width}s} {'us':>9s} {'MB':>9s} {'GFLOP':>9s} {'floor us':>9s} {'frac':>6s}"
    lines = [head, "-" * len(head)]
    for r in rows:
        lines.append(f"{r['op']:66s} {r['rows']:5d} {r['kernel']:{width}s} {r['us']:9.2f} {r['mbytes']:9.2f} {r['gflop']:9.2f} "
                     f"{r['floor_us']:9.2f} {r['frac']:6.3f}")
    return "\n".join(lines)
