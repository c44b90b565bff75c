"""Each CUDA kernel alone against a plain fp32 torch computation of the same operation,
at sizes other than the tiny models': odd widths, head sizes from 16 to 256, permuted
pages, windows.  Where random inputs would hide a fault, inputs are made so that it shows."""
import math

import numpy as np
import pytest
import torch

import plain_qwen2

pytestmark = pytest.mark.gpu

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": dict(atol=3e-5, rtol=3e-5), "bfloat16": dict(atol=2.5e-2, rtol=2.5e-2)}


def ops():
    from tessweave_engine_b200.csrc import ops as o
    return o


def dev(t, dtype=None):
    return t.to("cuda", dtype) if dtype else t.to("cuda")


def status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(100, 37), (3584, 1000)])
def test_embed(dtype, hidden, vocab):
    torch.manual_seed(0)
    table = dev(torch.randn(vocab, hidden), DTYPES[dtype])
    ids = torch.tensor([0, vocab - 1, 5, 5, 17], dtype=torch.int32, device="cuda")
    resid = torch.full((5, hidden), 7.0, device="cuda")
    st = status()
    ops().embed(resid, table, ids, 5, st)
    assert torch.equal(resid, table[ids.long()].float()) and int(st) == 0
    bad = torch.tensor([3, vocab], dtype=torch.int32, device="cuda")
    ops().embed(resid, table, bad, 2, st)
    assert int(st) == 1 and float(resid[1].abs().sum()) == 0          # refused, not read out of bounds


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [96, 1000, 3584, 5120])
def test_add_rmsnorm(dtype, hidden):
    torch.manual_seed(1)
    dt = DTYPES[dtype]
    n, eps = 9, 1e-5
    resid = dev(torch.randn(n, hidden) * 3)
    delta = dev(torch.randn(n, hidden), dt)
    weight = dev(1 + 0.1 * torch.randn(hidden))
    want_resid = resid + delta.float()
    want = plain_qwen2.rms_norm(want_resid.cpu(), weight.cpu(), eps)
    out = torch.empty(n, hidden, device="cuda", dtype=dt)
    r = resid.clone()
    ops().add_rmsnorm(out, r, delta, weight, eps, n)
    assert torch.allclose(r, want_resid, atol=1e-6)
    assert torch.allclose(out.float().cpu(), want, **TOL[dtype])
    # no delta: the stream is only read
    r2 = resid.clone()
    ops().add_rmsnorm(out, r2, None, weight, eps, n)
    assert torch.equal(r2, resid)
    assert torch.allclose(out.float().cpu(), plain_qwen2.rms_norm(resid.cpu(), weight.cpu(), eps), **TOL[dtype])
    # selected rows: the stream stays as it was, the delta is still counted
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device="cuda")
    r3 = resid.clone()
    out3 = torch.empty(3, hidden, device="cuda", dtype=dt)
    ops().add_rmsnorm(out3, r3, delta, weight, eps, 3, rows)
    assert torch.equal(r3, resid)
    assert torch.allclose(out3.float().cpu(), want[rows.long().cpu()], **TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul(dtype):
    torch.manual_seed(2)
    dt = DTYPES[dtype]
    n, inter = 5, 200
    gu = dev(torch.randn(n, 2 * inter) * 4, dt)
    out = torch.empty(n, inter, device="cuda", dtype=dt)
    ops().silu_mul(out, gu, n)
    g, u = gu.float().cpu()[:, :inter], gu.float().cpu()[:, inter:]
    assert torch.allclose(out.float().cpu(), g * torch.sigmoid(g) * u, **TOL[dtype])
    # columns in groups of eight gates and their eight ups
    ops().silu_mul(out, gu, n, interleaved=True)
    pairs = gu.float().cpu().reshape(n, inter // 8, 2, 8)
    g, u = pairs[:, :, 0].reshape(n, inter), pairs[:, :, 1].reshape(n, inter)
    assert torch.allclose(out.float().cpu(), g * torch.sigmoid(g) * u, **TOL[dtype])


def paged_setup(lengths, page, kv_heads, head_dim, dtype, seed=0, extra_pages=5):
    """Random keys/values for requests of the given lengths, scattered over permuted pages."""
    g = torch.Generator().manual_seed(seed)
    blocks = [math.ceil(n / page) for n in lengths]
    total = sum(blocks) + extra_pages
    perm = torch.randperm(total, generator=g).tolist()
    width = max(blocks) + 1
    table = torch.full((len(lengths) + 2, width), -1, dtype=torch.int32)
    slots = list(range(len(lengths), 0, -1))                       # request i uses table row slots[i]
    k_pages = torch.full((total, kv_heads, page, head_dim), float("nan"))
    v_pages = torch.full((total, kv_heads, page, head_dim), float("nan"))
    ks, vs = [], []
    cursor = 0
    for i, n in enumerate(lengths):
        k = torch.randn(n, kv_heads, head_dim, generator=g)
        v = torch.randn(n, kv_heads, head_dim, generator=g)
        ks.append(k); vs.append(v)
        for b in range(blocks[i]):
            pid = perm[cursor]; cursor += 1
            table[slots[i], b] = pid
            chunk = slice(b * page, min(n, (b + 1) * page))
            m = chunk.stop - chunk.start
            k_pages[pid, :, :m] = k[chunk].transpose(0, 1)
            v_pages[pid, :, :m] = v[chunk].transpose(0, 1)
    return dict(table=dev(table), slots=slots, k_pages=dev(k_pages, dtype), v_pages=dev(v_pages, dtype), k=ks, v=vs)


def dense_attention(q, k, v, positions, window=None):
    """q: [rows, Hq, D] at the given positions of one request; k, v: [n, Hkv, D]; fp32."""
    rep = q.shape[1] // k.shape[1]
    kk, vv = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
    s = torch.einsum("rhd,nhd->hrn", q, kk) * q.shape[-1] ** -0.5
    p = torch.arange(k.shape[0])
    pos = torch.as_tensor(positions)
    visible = p[None, :] <= pos[:, None]
    if window:
        visible &= p[None, :] > pos[:, None] - window
    s = s.masked_fill(~visible[None], float("-inf"))
    return torch.einsum("hrn,nhd->rhd", torch.softmax(s, -1), vv)


CASES = [(8, 8, 16), (8, 2, 32), (8, 1, 64), (6, 3, 48), (28, 4, 128), (4, 2, 256), (3, 1, 80)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d", CASES)
@pytest.mark.parametrize("window", [0, 24])
def test_attention_generic_ragged_rows(dtype, hq, hkv, d, window):
    """Decode rows and prompt portions of four requests in one launch (lengths 1/17/65/257
    as tools/validate_cuda.py:25-57), pages in random order, page size 16 and 8."""
    dt = DTYPES[dtype]
    lengths = [1, 17, 65, 257]
    page = 16 if d != 48 else 8
    setup = paged_setup(lengths, page, hkv, d, dt, seed=hq * 100 + d)
    rows_of = [[0], [16], list(range(60, 65)), [0, 1, 15, 16, 17, 255, 256]]       # request -> positions in this step
    g = torch.Generator().manual_seed(5)
    n = sum(len(r) for r in rows_of)
    q = torch.randn(n, hq, d, generator=g)
    positions, seq_of_token = [], []
    for i, r in enumerate(rows_of):
        positions += r; seq_of_token += [i] * len(r)
    qd = dev(q.reshape(n, hq * d), dt)
    out = torch.full((n, hq * d), float("nan"), device="cuda", dtype=dt)
    st = status()
    ops().attention_generic(out, qd, dev(torch.tensor(positions, dtype=torch.int32)),
                            dev(torch.tensor(seq_of_token, dtype=torch.int32)),
                            dev(torch.tensor(setup["slots"], dtype=torch.int32)), setup["table"], setup["k_pages"],
                            setup["v_pages"], n, hq, hkv, d, window, d ** -0.5, st)
    assert int(st) == 0
    cursor = 0
    for i, r in enumerate(rows_of):
        rq = qd[cursor:cursor + len(r)].float().cpu().reshape(len(r), hq, d)
        k = setup["k"][i].to(dt).float(); v = setup["v"][i].to(dt).float()
        want = dense_attention(rq, k, v, r, window or None)
        got = out[cursor:cursor + len(r)].float().cpu().reshape(len(r), hq, d)
        assert torch.allclose(got, want, **TOL[dtype]), f"request {i}"
        cursor += len(r)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", ["first_of_page", "last_of_page", "position_zero", "window_edge_inside", "window_edge_outside"])
def test_attention_finds_one_far_key(dtype, where):
    """One key among hundreds is made to dominate (its score stands out by a scaled query and
    key).  The output must be that key's value: a kernel that skips a page, misreads a page's
    first or last slot, or is off by one at a window's edge shows here, which random inputs hide."""
    dt = DTYPES[dtype]
    hq, hkv, d, page, n = 4, 2, 32, 16, 400
    window = 0
    pos = n - 1
    target = {"first_of_page": 16 * 7, "last_of_page": 16 * 9 + 15, "position_zero": 0}.get(where)
    if where.startswith("window_edge"):
        window = 100
        target = pos - window + 1 if where.endswith("inside") else pos - window
    setup = paged_setup([n], page, hkv, d, dt, seed=3)
    q = torch.randn(1, hq, d) * 0.1
    direction = torch.randn(d); direction /= direction.norm()
    q[0, :] = direction * 12.0
    kp, vp = setup["k_pages"], setup["v_pages"]
    pid = int(setup["table"][setup["slots"][0], target // page])
    kp[pid, :, target % page] = (direction * 12.0).to(dt).cuda()           # score 144 / sqrt(32) ~ 25, far above the rest
    marker = torch.arange(d, dtype=torch.float32) / d + 2.0
    vp[pid, :, target % page] = marker.to(dt).cuda()
    out = torch.empty(1, hq * d, device="cuda", dtype=dt)
    st = status()
    ops().attention_generic(out, dev(q.reshape(1, hq * d), dt), dev(torch.tensor([pos], dtype=torch.int32)),
                            dev(torch.tensor([0], dtype=torch.int32)), dev(torch.tensor(setup["slots"], dtype=torch.int32)),
                            setup["table"], kp, vp, 1, hq, hkv, d, window, d ** -0.5, st)
    k = setup["k"][0].clone(); v = setup["v"][0].clone()
    k[target] = direction * 12.0; v[target] = marker
    want = dense_attention(q.to(dt).float(), k.to(dt).float(), v.to(dt).float(), [pos], window or None)
    got = out.float().cpu().reshape(1, hq, d)
    assert torch.allclose(got, want, **TOL[dtype])
    hit = (got[0, 0] - marker).abs().max() < 0.5
    assert bool(hit) == (where != "window_edge_outside")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 16, 16), (3, 1, 32, 8), (6, 3, 48, 4), (28, 4, 128, 16)])
def test_rope_kv_write(dtype, hq, hkv, d, page):
    """Bias, rotation and the scatter into pages, against plain_qwen2.rope; tokens of two
    requests at scattered positions, tables with pages in reverse order."""
    dt = DTYPES[dtype]
    torch.manual_seed(4)
    theta = 1e6 if d >= 32 else 1e4
    positions = [0, 1, page - 1, page, 3 * page + 2, 1500, page - 1, page]
    seq_of_token = [0, 0, 0, 0, 0, 0, 1, 1]
    n = len(positions)
    width = (hq + 2 * hkv) * d
    qkv = torch.randn(n, width)
    bias = torch.randn(width) * 0.5
    blocks = 1500 // page + 1
    pages = blocks + 4
    table = torch.full((3, blocks), -1, dtype=torch.int32)
    table[2, :] = torch.arange(blocks - 1, -1, -1, dtype=torch.int32)           # request 0 -> row 2
    table[0, :2] = torch.tensor([pages - 1, pages - 2], dtype=torch.int32)      # request 1 -> row 0
    kp = torch.zeros(pages, hkv, page, d, device="cuda", dtype=dt)
    vp = torch.zeros_like(kp)
    inv = dev(theta ** (-torch.arange(0, d, 2, dtype=torch.float32) / d))
    x = dev(qkv, dt)
    st = status()
    ops().rope_kv_write(x, dev(bias), dev(torch.tensor(positions, dtype=torch.int32)),
                        dev(torch.tensor(seq_of_token, dtype=torch.int32)), dev(torch.tensor([2, 0], dtype=torch.int32)),
                        dev(table), inv, kp, vp, n, hq, hkv, d, True, st)
    assert int(st) == 0
    src = qkv.to(dt).float() + bias
    q_want = plain_qwen2.rope(src[:, :hq * d].reshape(n, hq, d), positions, theta)
    k_want = plain_qwen2.rope(src[:, hq * d:(hq + hkv) * d].reshape(n, hkv, d), positions, theta)
    v_want = src[:, (hq + hkv) * d:].reshape(n, hkv, d)
    tol = TOL[dtype] if dtype == "bfloat16" else dict(atol=2e-5, rtol=1e-5)
    assert torch.allclose(x[:, :hq * d].float().cpu().reshape(n, hq, d), q_want, **tol)
    rows = {0: 2, 1: 0}
    for i, (p, s) in enumerate(zip(positions, seq_of_token)):
        pid = int(table[rows[s], p // page])
        assert torch.allclose(kp[pid, :, p % page].float().cpu(), k_want[i], **tol), f"k of token {i}"
        assert torch.allclose(vp[pid, :, p % page].float().cpu(), v_want[i], **tol), f"v of token {i}"
    written = sum(1 for _ in positions)
    assert int((kp.float().abs().sum(-1) > 0).sum()) == written * hkv          # nothing else was touched
    # a position without a page is refused and reported, not written somewhere
    st2 = status()
    ops().rope_kv_write(x, None, dev(torch.tensor([5 * page], dtype=torch.int32)), dev(torch.tensor([1], dtype=torch.int32)),
                        dev(torch.tensor([2, 0], dtype=torch.int32)), dev(table), inv, kp, vp, 1, hq, hkv, d, True, st2)
    assert int(st2) == 2


def test_sample_greedy_and_temperature():
    torch.manual_seed(6)
    vocab = 152064
    logits = torch.randn(6, vocab) * 2
    logits[1, 777] = 50; logits[1, 90000] = 50                 # a tie: the lowest index wins
    logits[2, vocab - 1] = 60
    logits[3, 0] = 60
    out = torch.zeros(6, dtype=torch.int32, device="cuda")
    ops().sample(out, dev(logits), 6)
    assert out.tolist() == [int(logits[i].argmax()) if i != 1 else 777 for i in range(6)]
    # a greedy row is shared by eight blocks: ties inside one block's part and across parts, rows whose length is
    # no multiple of four (no 16-byte loads), rows shorter than the eight parts, a row of equal values
    for vocab2 in (5, 7, 131, 1000, 4099):
        rows = torch.randn(9, vocab2)
        rows[1] = 3.0
        rows[2, vocab2 - 1] = 9.0; rows[2, vocab2 // 2] = 9.0
        rows[3, 0] = 9.0; rows[3, vocab2 - 1] = 9.0
        rows[4, min(vocab2 - 1, vocab2 // 8 + 1)] = 9.0; rows[4, min(vocab2 - 1, vocab2 // 8 + 2)] = 9.0
        got = torch.zeros(9, dtype=torch.int32, device="cuda")
        ops().sample(got, dev(rows), 9)
        assert got.tolist() == [int(torch.nonzero(rows[i] == rows[i].max())[0]) for i in range(9)], vocab2
    # temperature rows beside greedy rows; each row's draw depends on its own seed and counter only
    temps = [0.0, 0.8, 1.0, 2.0, 0.8, 0.3]
    seeds = [0, 11, 12, 13, 11, 99]
    counters = [0, 0, 5, 7, 1, 2]
    small = torch.randn(6, 1000) * 3
    out2 = torch.zeros(6, dtype=torch.int32, device="cuda")
    ops().sample(out2, dev(small), 6, dev(torch.tensor(temps)), dev(torch.tensor(seeds)), dev(torch.tensor(counters)))
    want = [plain_qwen2.choose(small[i], temps[i], seeds[i], counters[i]) for i in range(6)]
    assert out2.tolist() == want
    alone = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops().sample(alone, dev(small[4:5]), 1, dev(torch.tensor([0.8])), dev(torch.tensor([11])), dev(torch.tensor([1])))
    assert int(alone) == want[4]
    # the sampling package's entry point, which the step function uses: the same tokens from plain Python lists
    from tessweave_engine_b200.sampling import choose_tokens
    assert choose_tokens(dev(small), temps, seeds, counters).tolist() == want
    assert choose_tokens(dev(logits)).tolist() == out.tolist()
    # many draws follow the distribution
    row = torch.tensor([[0.0, 1.0, 2.0, -30.0, 0.5]]).repeat(4000, 1)
    out3 = torch.zeros(4000, dtype=torch.int32, device="cuda")
    ops().sample(out3, dev(row), 4000, dev(torch.ones(4000)), dev(torch.full((4000,), 3)), dev(torch.arange(4000)))
    freq = np.bincount(out3.cpu().numpy(), minlength=5) / 4000
    assert np.abs(freq - torch.softmax(row[0], 0).numpy()).max() < 0.03


# ---------------------------------------------------------------------------
# bf16 tensor-core attention: the same cases through the decode and the prefill kernel
# ---------------------------------------------------------------------------
TC_CASES = [(8, 8, 16), (8, 2, 32), (8, 1, 64), (6, 3, 48), (28, 4, 128), (4, 2, 256), (3, 1, 80), (40, 2, 64)]


def run_tensor_core_attention(setup, rows_of, q, hq, hkv, d, window, nsplit=None, merge_in_scratch=False, tcgen05=False,
                              tma=False, stages=0):
    """rows_of: request -> the consecutive positions it brings; the request holds exactly
    positions 0..last.  Requests with one row go through the decode kernel (with ``tma`` the one fed by TMA)."""
    o = ops()
    n = sum(len(r) for r in rows_of)
    qd = dev(q.reshape(n, hq * d), torch.bfloat16)
    out = torch.full((n, hq * d), float("nan"), device="cuda", dtype=torch.bfloat16)
    starts, cursor = [], 0
    for r in rows_of:
        starts.append(cursor); cursor += len(r)
    i32 = lambda v: dev(torch.tensor(v, dtype=torch.int32))
    q_start, q_len, kv_len, slot = i32(starts), i32([len(r) for r in rows_of]), i32([r[-1] + 1 for r in rows_of]), i32(setup["slots"])
    st = status()
    singles = any(len(r) == 1 for r in rows_of)
    if any(len(r) > 1 for r in rows_of):
        prefill = o.attention_prefill_tcgen05 if tcgen05 else o.attention_prefill
        prefill(out, qd, q_start, q_len, kv_len, slot, setup["table"], setup["k_pages"], setup["v_pages"],
                            len(rows_of), max(len(r) for r in rows_of), hq, hkv, d, window, d ** -0.5, singles, st)
    if singles:
        max_kv = max(r[-1] + 1 for r in rows_of)
        ns = nsplit or o.decode_splits(len(rows_of), hkv, hq // hkv, max_kv)
        scratch = torch.full((o.decode_scratch_floats(hq, d),), float("nan"), device="cuda")
        counters = torch.zeros(o.decode_counter_ints(len(rows_of), hkv, hq // hkv), dtype=torch.int32, device="cuda")
        for _ in range(2):      # twice: the counters must come back to zero
            out.fill_(float("nan")) if not any(len(r) > 1 for r in rows_of) else None
            if tma:
                o.attention_decode_tma(out, qd, None, None, None, False, q_start, q_len, kv_len, slot, setup["table"],
                                       setup["k_pages"], setup["v_pages"], len(rows_of), hq, hkv, d, window, d ** -0.5, ns,
                                       scratch, counters, st, merge_in_scratch=merge_in_scratch, stages=stages)
            else:
                o.attention_decode(out, qd, q_start, q_len, kv_len, slot, setup["table"], setup["k_pages"], setup["v_pages"],
                                   len(rows_of), hq, hkv, d, window, d ** -0.5, ns, scratch, counters, st,
                                   merge_in_scratch=merge_in_scratch)
        assert int(counters.abs().sum()) == 0
    assert int(st) == 0
    return out.float().cpu().reshape(n, hq, d), qd.float().cpu().reshape(n, hq, d)


@pytest.mark.parametrize("hq,hkv,d", TC_CASES)
@pytest.mark.parametrize("window", [0, 24])
def test_tensor_core_attention_mixed_rows(hq, hkv, d, window):
    """Two decode rows (lengths 1 and 257+) beside two prompt portions, one of which starts in the
    middle of its request (keys already cached), pages in random order."""
    lengths = [1, 300, 65, 257]
    page = 16 if d != 48 else 8
    setup = paged_setup(lengths, page, hkv, d, torch.bfloat16, seed=hq * 100 + d)
    rows_of = [[0], [299], list(range(0, 65)), list(range(200, 257))]
    g = torch.Generator().manual_seed(5)
    n = sum(len(r) for r in rows_of)
    q = torch.randn(n, hq, d, generator=g)
    got, qr = run_tensor_core_attention(setup, rows_of, q, hq, hkv, d, window)
    cursor = 0
    for i, r in enumerate(rows_of):
        k = setup["k"][i].to(torch.bfloat16).float(); v = setup["v"][i].to(torch.bfloat16).float()
        want = dense_attention(qr[cursor:cursor + len(r)], k, v, r, window or None)
        assert torch.allclose(got[cursor:cursor + len(r)], want, **TOL["bfloat16"]), f"request {i}"
        cursor += len(r)


@pytest.mark.parametrize("tma", [False, True])
@pytest.mark.parametrize("merge_in_scratch", [False, True])
@pytest.mark.parametrize("nsplit", [1, 2, 7, 16, 17, 64])
def test_decode_attention_any_split(nsplit, merge_in_scratch, tma):
    """The split count must not matter, also when most slices are empty; neither may the way the
    slices are merged (inside a cluster up to 16 slices, through scratch memory beyond)."""
    hq, hkv, d = 14, 2, 64
    lengths = [5, 64, 65, 1000]
    setup = paged_setup(lengths, 16, hkv, d, torch.bfloat16, seed=9)
    rows_of = [[n - 1] for n in lengths]
    q = torch.randn(4, hq, d, generator=torch.Generator().manual_seed(1))
    got, qr = run_tensor_core_attention(setup, rows_of, q, hq, hkv, d, 0, nsplit=nsplit, merge_in_scratch=merge_in_scratch,
                                        tma=tma)
    for i, r in enumerate(rows_of):
        k = setup["k"][i].to(torch.bfloat16).float(); v = setup["v"][i].to(torch.bfloat16).float()
        assert torch.allclose(got[i:i + 1], dense_attention(qr[i:i + 1], k, v, r), **TOL["bfloat16"]), f"request {i}"


@pytest.mark.parametrize("kind", ["decode", "decode_tma", "prefill"])
@pytest.mark.parametrize("where", ["first_of_page", "last_of_page", "position_zero", "tile_edge", "window_edge_inside",
                                   "window_edge_outside"])
def test_tensor_core_attention_finds_one_far_key(kind, where):
    """As above for the fp32 kernel: one dominating key at a page's first or last slot, at a
    64-key tile's edge, at position 0 and at both sides of a window's edge."""
    hq, hkv, d, page, n = 4, 2, (64 if kind == "decode_tma" else 32), 16, 400
    window = 0
    rows = [n - 1] if kind.startswith("decode") else list(range(n - 5, n))
    pos = rows[0]
    target = {"first_of_page": 16 * 7, "last_of_page": 16 * 9 + 15, "position_zero": 0, "tile_edge": 63}.get(where)
    if where.startswith("window_edge"):
        window = 100
        target = pos - window + 1 if where.endswith("inside") else pos - window
    setup = paged_setup([n], page, hkv, d, torch.bfloat16, seed=3)
    direction = torch.randn(d, generator=torch.Generator().manual_seed(2)); direction /= direction.norm()
    q = torch.randn(len(rows), hq, d) * 0.1
    q[0, :] = direction * 12.0
    kp, vp = setup["k_pages"], setup["v_pages"]
    pid = int(setup["table"][setup["slots"][0], target // page])
    kp[pid, :, target % page] = (direction * 12.0).to(torch.bfloat16).cuda()
    marker = torch.arange(d, dtype=torch.float32) / d + 2.0
    vp[pid, :, target % page] = marker.to(torch.bfloat16).cuda()
    got, qr = run_tensor_core_attention(setup, [rows], q, hq, hkv, d, window, tma=kind == "decode_tma")
    k = setup["k"][0].clone(); v = setup["v"][0].clone()
    k[target] = direction * 12.0; v[target] = marker
    want = dense_attention(qr, k.to(torch.bfloat16).float(), v.to(torch.bfloat16).float(), rows, window or None)
    assert torch.allclose(got, want, **TOL["bfloat16"])
    hit = (got[0, 0] - marker).abs().max() < 0.5
    assert bool(hit) == (where != "window_edge_outside")


# ---------------------------------------------------------------------------
# tcgen05 attention for prompt portions (TMA, accumulators and probabilities in tensor memory)
# ---------------------------------------------------------------------------
TC5_CASES = [
    # hq, hkv, d, page, lengths, rows of each request, window
    (1, 1, 64, 16, [100], [(0, 100)], 0),                                   # one tile of keys, one tile of rows
    (2, 1, 128, 16, [300], [(0, 300)], 0),                                  # several tiles, both row tiles
    (28, 4, 128, 16, [300, 65, 257], [(0, 300), (0, 65), (200, 257)], 0),   # groups of 7: rows of a token straddle tiles
    (28, 4, 128, 16, [700], [(100, 700)], 200),                             # a window that drops whole tiles
    (8, 1, 64, 32, [1000, 130], [(0, 1000), (128, 130)], 0),                # a two-token portion beside a long one
    (6, 2, 128, 128, [513], [(0, 513)], 0),                                 # a page = a tile
    (6, 2, 64, 256, [513], [(0, 513)], 24),                                 # a page = two tiles
    (6, 2, 64, 8, [513], [(500, 513)], 0),                                  # sixteen pages to a tile
    (5, 5, 128, 16, [1200], [(0, 1200)], 0),                                # no grouping
]


@pytest.mark.parametrize("hq,hkv,d,page,lengths,spans,window", TC5_CASES)
def test_tcgen05_attention(hq, hkv, d, page, lengths, spans, window):
    """Freed and unused cache slots hold NaN here, so a value row past a request's end that
    reached a product would show."""
    setup = paged_setup(lengths, page, hkv, d, torch.bfloat16, seed=hq * 10 + d)
    rows_of = [list(range(a, b)) for a, b in spans]
    n = sum(len(r) for r in rows_of)
    q = torch.randn(n, hq, d, generator=torch.Generator().manual_seed(5))
    got, qr = run_tensor_core_attention(setup, rows_of, q, hq, hkv, d, window, tcgen05=True)
    cursor = 0
    for i, r in enumerate(rows_of):
        k = setup["k"][i].to(torch.bfloat16).float(); v = setup["v"][i].to(torch.bfloat16).float()
        want = dense_attention(qr[cursor:cursor + len(r)], k, v, r, window or None)
        assert torch.allclose(got[cursor:cursor + len(r)], want, **TOL["bfloat16"]), f"request {i}"
        cursor += len(r)


@pytest.mark.parametrize("where", ["first_of_page", "last_of_page", "position_zero", "tile_edge", "next_tile",
                                   "window_edge_inside", "window_edge_outside"])
def test_tcgen05_attention_finds_one_far_key(where):
    """One dominating key among 700, at a page's first and last slot, at both sides of a 128-key
    tile's edge, at position 0 and at both sides of a window's edge.  Scores that large also
    make the rows' maxima jump, so the accumulator in tensor memory is rescaled."""
    hq, hkv, d, page, n = 4, 2, 128, 16, 700
    window = 0
    rows = list(range(n - 40, n))
    pos = rows[0]
    target = {"first_of_page": 16 * 7, "last_of_page": 16 * 9 + 15, "position_zero": 0, "tile_edge": 127,
              "next_tile": 128}.get(where)
    if where.startswith("window_edge"):
        window = 300
        target = pos - window + 1 if where.endswith("inside") else pos - window
    setup = paged_setup([n], page, hkv, d, torch.bfloat16, seed=3)
    direction = torch.randn(d, generator=torch.Generator().manual_seed(2)); direction /= direction.norm()
    q = torch.randn(len(rows), hq, d) * 0.1
    q[0, :] = direction * 12.0
    kp, vp = setup["k_pages"], setup["v_pages"]
    pid = int(setup["table"][setup["slots"][0], target // page])
    kp[pid, :, target % page] = (direction * 12.0).to(torch.bfloat16).cuda()
    marker = torch.arange(d, dtype=torch.float32) / d + 2.0
    vp[pid, :, target % page] = marker.to(torch.bfloat16).cuda()
    got, qr = run_tensor_core_attention(setup, [rows], q, hq, hkv, d, window, tcgen05=True)
    k = setup["k"][0].clone(); v = setup["v"][0].clone()
    k[target] = direction * 12.0; v[target] = marker
    want = dense_attention(qr, k.to(torch.bfloat16).float(), v.to(torch.bfloat16).float(), rows, window or None)
    assert torch.allclose(got, want, **TOL["bfloat16"])
    hit = (got[0, 0] - marker).abs().max() < 0.5
    assert bool(hit) == (where != "window_edge_outside")


def test_tcgen05_attention_refuses_other_shapes():
    o = ops()
    assert not o.tcgen05_attention_supported(torch.bfloat16, 80, 16)
    assert not o.tcgen05_attention_supported(torch.bfloat16, 128, 48)
    assert not o.tcgen05_attention_supported(torch.float32, 128, 16)
    setup = paged_setup([40], 16, 1, 32, torch.bfloat16)
    q = dev(torch.randn(40, 32), torch.bfloat16)
    i32 = lambda v: dev(torch.tensor(v, dtype=torch.int32))
    with pytest.raises(Exception, match="tcgen05 attention"):
        o.attention_prefill_tcgen05(torch.empty_like(q), q, i32([0]), i32([40]), i32([40]), i32(setup["slots"]), setup["table"],
                                    setup["k_pages"], setup["v_pages"], 1, 40, 1, 1, 32, 0, 32 ** -0.5, False, status())


# ---------------------------------------------------------------------------
# matrix products with few rows
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("n,k", [(100, 64), (37, 200), (4608, 3584), (1000, 18944)])
def test_gemm_small_m(m, n, k):
    """Weight-streaming product against fp32 torch, whole and split over k; n and k with ragged
    tails (n no multiple of 16, k no multiple of 32)."""
    torch.manual_seed(m * 1000 + n)
    x = dev(torch.randn(m, k) * 0.5, torch.bfloat16)
    w = dev(torch.randn(n, k) * 0.05, torch.bfloat16)
    want = x.float() @ w.float().t()
    tol = dict(atol=2e-3 * max(1.0, float(want.abs().max())), rtol=0)
    out32 = torch.full((m, n), float("nan"), device="cuda")
    ops().gemm_small_m(out32, x, w, m)
    assert torch.allclose(out32, want, **tol)
    out16 = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    ops().gemm_small_m(out16, x, w, m)
    assert torch.allclose(out16.float(), want, atol=tol["atol"] + 8e-3 * float(want.abs().max()), rtol=0)
    for kper in (32, 256, 416, 896):         # 896: few blocks and long slices, two warps share a row tile (m <= 8)
        if kper >= k:
            continue
        split = -(-k // kper)
        slices = torch.full((split, m, n), float("nan"), device="cuda")
        ops().gemm_small_m(slices, x, w, m, kper)
        assert torch.allclose(slices.sum(0), want, **tol)
        from tessweave_engine_b200.csrc.ops import SplitSum
        dense = SplitSum(slices).dense(torch.float32)
        assert torch.allclose(dense, want, **tol)
        # consumers that add the slices themselves
        if n == 1000:
            resid = dev(torch.randn(m, n))
            weight = dev(1 + 0.1 * torch.randn(n))
            out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
            r = resid.clone()
            ops().add_rmsnorm(out, r, SplitSum(slices), weight, 1e-6, m)
            assert torch.allclose(r, resid + dense, atol=1e-5)
            assert torch.allclose(out.float().cpu(), plain_qwen2.rms_norm((resid + dense).cpu(), weight.cpu(), 1e-6),
                                  **TOL["bfloat16"])


@pytest.mark.parametrize("m", [1, 5, 8])
@pytest.mark.parametrize("inter,k", [(200, 96), (328, 4160)])
def test_gemm_small_m_fused_silu(m, inter, k):
    """gate/up rows in groups of eight: the kernel writes silu(gate) * up directly.  The second shape (few
    row tiles, long k) takes the variant in which two warps share a row tile's values of k."""
    torch.manual_seed(m)
    x = dev(torch.randn(m, k), torch.bfloat16)
    wg, wu = torch.randn(inter, k) * 0.2 * (96 / k) ** 0.5, torch.randn(inter, k) * 0.2 * (96 / k) ** 0.5
    packed = torch.stack((wg.reshape(inter // 8, 8, k), wu.reshape(inter // 8, 8, k)), 1).reshape(2 * inter, k)
    w = dev(packed, torch.bfloat16)
    out = torch.full((m, inter), float("nan"), device="cuda", dtype=torch.bfloat16)
    ops().gemm_small_m(out, x, w, m, silu_mul_pairs=True)
    g = x.float().cpu() @ wg.to(torch.bfloat16).float().t()
    u = x.float().cpu() @ wu.to(torch.bfloat16).float().t()
    assert torch.allclose(out.float().cpu(), g * torch.sigmoid(g) * u, **TOL["bfloat16"])


def test_decode_attention_many_pages_per_block():
    """Pages of 4 tokens and one slice: a block walks 375 block-table entries, more than it keeps
    in shared memory, so the entries beyond come straight from the table."""
    hq, hkv, d = 6, 3, 32
    setup = paged_setup([1500, 9], 4, hkv, d, torch.bfloat16, seed=11)
    rows_of = [[1499], [8]]
    q = torch.randn(2, hq, d, generator=torch.Generator().manual_seed(3))
    got, qr = run_tensor_core_attention(setup, rows_of, q, hq, hkv, d, 0, nsplit=1)
    for i, r in enumerate(rows_of):
        k = setup["k"][i].to(torch.bfloat16).float(); v = setup["v"][i].to(torch.bfloat16).float()
        assert torch.allclose(got[i:i + 1], dense_attention(qr[i:i + 1], k, v, r), **TOL["bfloat16"])


# ---------------------------------------------------------------------------
# products with many rows on pairs of thread blocks (tcgen05.mma.cta_group::2)
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 1000, 3584), (512, 768, 1024), (1, 16, 8), (700, 4608, 200)])
@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
def test_gemm_tcgen05_pair(m, n, k, out_dtype):
    """Whole tiles, ragged tiles in every direction (rows, columns, k), one row, bf16 and fp32 results."""
    g = torch.Generator().manual_seed(m + n + k)
    x = dev(torch.randn(m, k, generator=g), torch.bfloat16)
    w = dev(torch.randn(n, k, generator=g) * 0.05, torch.bfloat16)
    out = torch.full((m, n), float("nan"), device="cuda", dtype=out_dtype)
    st = status()
    ops().gemm_tcgen05_pair(out, x, w, m, st)
    assert int(st) == 0
    want = x.float() @ w.float().t()
    tol = dict(rtol=2e-2, atol=2e-2) if out_dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-3)
    assert torch.allclose(out.float(), want, **tol)


@pytest.mark.parametrize("m,n,k", [(300, 1024, 512), (600, 20000, 512), (257, 48, 64)])
def test_gemm_tcgen05_pair_silu_mul(m, n, k):
    """The fused epilogue: weight rows in groups of eight gates and their eight ups."""
    g = torch.Generator().manual_seed(7)
    x = dev(torch.randn(m, k, generator=g), torch.bfloat16)
    w = dev(torch.randn(n, k, generator=g) * 0.05, torch.bfloat16)
    out = torch.full((m, n // 2), float("nan"), device="cuda", dtype=torch.bfloat16)
    st = status()
    ops().gemm_tcgen05_pair(out, x, w, m, st, silu_mul_pairs=True)
    assert int(st) == 0
    y = (x.float() @ w.float().t()).reshape(m, n // 16, 2, 8)
    want = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(m, n // 2)
    assert torch.allclose(out.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("m,n,k", [(9, 300, 200), (16, 256, 128), (100, 520, 3592), (20, 40000, 256)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_gemm_tcgen05_stream(m, n, k, out_dtype):
    """The persistent weight-streaming kernel against fp32 torch: token tile widths 16, 32 and 128, rows and k
    with ragged tails, more work items than blocks (the last shape)."""
    g = torch.Generator().manual_seed(m + n)
    x = dev(torch.randn(m + 3, k, generator=g) * 0.5, torch.bfloat16)          # rows beyond m must not be read into the result
    w = dev(torch.randn(n, k, generator=g) * 0.05, torch.bfloat16)
    want = x[:m].float() @ w.float().t()
    st = status()
    out = torch.full((m + 1, n), float("nan"), device="cuda", dtype=out_dtype)
    ops().gemm_tcgen05_stream(out, x, w, m, st)
    assert int(st) == 0
    tol = dict(rtol=2e-2, atol=2e-2) if out_dtype == torch.bfloat16 else dict(rtol=1e-4, atol=1e-3)
    assert torch.allclose(out[:m].float(), want, **tol)
    assert bool(torch.isnan(out[m].float()).all()), "a row beyond m was written"


@pytest.mark.parametrize("m,n,k,kper", [(33, 1000, 512, 128), (64, 4608, 3584, 896), (128, 130, 8 * 75, 192)])
def test_gemm_tcgen05_stream_slices(m, n, k, kper):
    """The same as fp32 slices over k (token tile widths 64 and 128 among them, a last slice shorter than the
    others): each slice is the product over its own values of k."""
    g = torch.Generator().manual_seed(m + n)
    x = dev(torch.randn(m + 3, k, generator=g) * 0.5, torch.bfloat16)
    w = dev(torch.randn(n, k, generator=g) * 0.05, torch.bfloat16)
    want = x[:m].float() @ w.float().t()
    st = status()
    split = -(-k // kper)
    slices = torch.full((split, m, n), float("nan"), device="cuda")
    ops().gemm_tcgen05_stream(slices, x, w, m, st, kper=kper)
    assert int(st) == 0
    assert torch.allclose(slices.sum(0), want, atol=2e-3 * max(1.0, float(want.abs().max())), rtol=0)
    for i in range(split):
        part = x[:m, i * kper:(i + 1) * kper].float() @ w[:, i * kper:(i + 1) * kper].float().t()
        assert torch.allclose(slices[i], part, atol=2e-3 * max(1.0, float(part.abs().max())), rtol=0)


@pytest.mark.parametrize("m,n,k", [(17, 48, 64), (24, 37888, 512), (64, 1040, 3584), (9, 16, 72)])
def test_gemm_tcgen05_stream_silu_mul(m, n, k):
    """The fused epilogue: weight rows in groups of eight gates and their eight ups (a gate's up is eight
    tensor-memory lanes further)."""
    g = torch.Generator().manual_seed(11)
    x = dev(torch.randn(m, k, generator=g), torch.bfloat16)
    w = dev(torch.randn(n, k, generator=g) * 0.05, torch.bfloat16)
    out = torch.full((m, n // 2), float("nan"), device="cuda", dtype=torch.bfloat16)
    st = status()
    ops().gemm_tcgen05_stream(out, x, w, m, st, silu_mul_pairs=True)
    assert int(st) == 0
    y = (x.float() @ w.float().t()).reshape(m, n // 16, 2, 8)
    want = (torch.nn.functional.silu(y[:, :, 0]) * y[:, :, 1]).reshape(m, n // 2)
    assert torch.allclose(out.float(), want, rtol=2e-2, atol=2e-2)


@pytest.mark.parametrize("nslices", [1, 2, 5, 9])
@pytest.mark.parametrize("interleaved,inter", [(True, 200), (False, 100), (True, 13824)])
def test_silu_mul_from_slices(nslices, interleaved, inter):
    """SiLU.mul straight from the fp32 slices of a gate/up product split over k: the slices are added in the
    order the other consumers of a split product use, so the result equals densify-then-SiLU.mul bit for bit."""
    m = 11
    g = torch.Generator().manual_seed(nslices + inter)
    slices = dev(torch.randn(nslices, m, 2 * inter, generator=g))
    out = torch.full((m, inter), float("nan"), device="cuda", dtype=torch.bfloat16)
    o = ops()
    o.silu_mul(out, o.SplitSum(slices), m, interleaved)
    dense = slices.sum(0)
    if interleaved:
        y = dense.reshape(m, inter // 8, 2, 8)
        gate, up = y[:, :, 0].reshape(m, inter), y[:, :, 1].reshape(m, inter)
    else:
        gate, up = dense[:, :inter], dense[:, inter:]
    want = torch.nn.functional.silu(gate) * up
    assert torch.allclose(out.float(), want, rtol=1e-2, atol=1e-2)
    # bit for bit against the two-kernel way (slices added by the reduce kernel in fp32, then SiLU.mul in fp32)
    summed = o.SplitSum(slices).dense(torch.float32)
    two = torch.empty(m, inter, device="cuda")
    o.silu_mul(two, summed, m, interleaved)
    assert torch.equal(out, two.to(torch.bfloat16))


def test_products_with_a_prefetch_give_the_same_bits_and_refuse_a_misaligned_one():
    """Asking for the next matrix to be brought into L2 changes no result; a tensor that does not start on a
    16-byte boundary is refused by the entry point before anything is launched."""
    g = torch.Generator().manual_seed(5)
    nxt = dev(torch.randn(300, 72, generator=g), torch.bfloat16)
    o = ops()
    assert o.weight_head(nxt, 1 << 10).numel() == 512 and o.weight_head(nxt, 1 << 30).numel() == nxt.numel()
    assert o.weight_head(nxt, 0) is None and o.weight_head(None, 64) is None and o.weight_head(nxt.t(), 64) is None
    # the small-M product, plain and with SiLU.mul
    x = dev(torch.randn(5, 96, generator=g), torch.bfloat16)
    w = dev(torch.randn(208, 96, generator=g) * 0.1, torch.bfloat16)
    for silu in (False, True):
        shape = (5, 104) if silu else (5, 208)
        a = torch.full(shape, float("nan"), device="cuda", dtype=torch.bfloat16)
        b = torch.full(shape, float("nan"), device="cuda", dtype=torch.bfloat16)
        o.gemm_small_m(a, x, w, 5, silu_mul_pairs=silu)
        o.gemm_small_m(b, x, w, 5, silu_mul_pairs=silu, prefetch=o.weight_head(nxt, 1 << 14))
        assert torch.equal(a, b) and not torch.isnan(a.float()).any()
        c = torch.full(shape, float("nan"), device="cuda", dtype=torch.bfloat16)
        with pytest.raises(RuntimeError, match="gemm_small_m"):
            o.gemm_small_m(c, x, w, 5, silu_mul_pairs=silu, prefetch=nxt.view(-1)[1:])
        assert torch.isnan(c.float()).all()
    # the tcgen05 stream product
    x = dev(torch.randn(24, 128, generator=g), torch.bfloat16)
    w = dev(torch.randn(272, 128, generator=g) * 0.1, torch.bfloat16)
    st = status()
    a = torch.full((24, 136), float("nan"), device="cuda", dtype=torch.bfloat16)
    b = torch.full((24, 136), float("nan"), device="cuda", dtype=torch.bfloat16)
    o.gemm_tcgen05_stream(a, x, w, 24, st, silu_mul_pairs=True)
    o.gemm_tcgen05_stream(b, x, w, 24, st, silu_mul_pairs=True, prefetch=o.weight_head(nxt, 1 << 14))
    assert int(st) == 0 and torch.equal(a, b) and not torch.isnan(a.float()).any()
    c = torch.full((24, 136), float("nan"), device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="gemm_tcgen05_stream"):
        o.gemm_tcgen05_stream(c, x, w, 24, st, silu_mul_pairs=True, prefetch=nxt.view(-1)[1:])
    assert torch.isnan(c.float()).all()


def test_gemm_tcgen05_stream_refuses_what_it_cannot_do():
    x = dev(torch.randn(130, 64), torch.bfloat16)
    w = dev(torch.randn(32, 64), torch.bfloat16)
    with pytest.raises(Exception, match="gemm_tcgen05_stream"):
        ops().gemm_tcgen05_stream(torch.empty(130, 32, device="cuda"), x, w, 130, status())            # more than 128 rows
    with pytest.raises(Exception, match="gemm_tcgen05_stream"):
        ops().gemm_tcgen05_stream(torch.empty(2, 9, 32, device="cuda"), x, w, 9, status(), kper=48)      # kper no multiple of 64
    with pytest.raises(Exception, match="gemm_tcgen05_stream"):
        ops().gemm_tcgen05_stream(torch.empty(9, 12, device="cuda", dtype=torch.bfloat16), x, dev(torch.randn(24, 64), torch.bfloat16),
                                  9, status(), silu_mul_pairs=True)                                        # rows no multiple of 16


# ---------------------------------------------------------------------------
# decode attention that makes q, k and v of the new token itself
# ---------------------------------------------------------------------------
@pytest.mark.parametrize("hq,hkv,d", [(28, 4, 128), (6, 3, 48), (8, 8, 16), (20, 2, 64), (4, 2, 256)])
@pytest.mark.parametrize("split_source", [0, 2, 3, 4, 5, 9])
@pytest.mark.parametrize("window", [0, 40])
def test_decode_attention_fused_with_rotation_and_cache_write(hq, hkv, d, split_source, window):
    """The fused kernel (the one that loads keys through registers) against the two kernels it replaces (bias +
    rotation + cache write, then decode attention): strong against the two drifting apart, blind to a fault they
    share -- that is what test_rope_kv_write (against the plain rotation) and, for the fused arithmetic as a whole,
    test_decode_attention_tma_makes_q_k_v_itself and the replay tests (against the plain implementation) are for.
    The same attention output and the same cache contents, bit for bit, for requests whose
    newest position is a page's first slot, its last slot, position 0 and somewhere in between.  The product
    comes as bf16 rows (0) or as that many fp32 slices: up to four are loaded ahead of the keys, more afterwards.
    One of the two runs also asks for a tensor to be prefetched into L2, which changes nothing."""
    o = ops()
    lengths = [1, 16 * 9 + 1, 16 * 11, 300]
    page = 16
    setup = paged_setup(lengths, page, hkv, d, torch.bfloat16, seed=hq + d)
    n = len(lengths)
    width = (hq + 2 * hkv) * d
    g = torch.Generator().manual_seed(3)
    bias = dev(torch.randn(width, generator=g))
    inv = dev(1e4 ** (-torch.arange(0, d, 2, dtype=torch.float32) / d))
    i32 = lambda v: dev(torch.tensor(v, dtype=torch.int32))
    q_start, q_len, kv_len, slot = i32(list(range(n))), i32([1] * n), i32(lengths), i32(setup["slots"])
    positions, seq_of = i32([m - 1 for m in lengths]), i32(list(range(n)))
    if split_source:
        slices = dev(torch.randn(split_source, n, width, generator=g))
        source = o.SplitSum(slices)
        dense = torch.zeros(n, width, device="cuda", dtype=torch.bfloat16)
    else:
        dense = dev(torch.randn(n, width, generator=g), torch.bfloat16)
        source = None
    ns = 3
    scratch = torch.full((o.decode_scratch_floats(hq, d),), float("nan"), device="cuda")
    counters = torch.zeros(o.decode_counter_ints(n, hkv, hq // hkv), dtype=torch.int32, device="cuda")
    st = status()
    # the two kernels
    k_a, v_a = setup["k_pages"].clone(), setup["v_pages"].clone()
    qkv_a = dense.clone()
    o.rope_kv_write(qkv_a, bias, positions, seq_of, slot, setup["table"], inv, k_a, v_a, n, hq, hkv, d, True, st, source=source)
    out_a = torch.full((n, hq * d), float("nan"), device="cuda", dtype=torch.bfloat16)
    o.attention_decode(out_a, qkv_a[:, : hq * d], q_start, q_len, kv_len, slot, setup["table"], k_a, v_a, n, hq, hkv, d, window,
                       d ** -0.5, ns, scratch, counters, st)
    # the fused kernel, through both ways of merging the slices
    for merge_in_scratch in (False, True):
        k_b, v_b = setup["k_pages"].clone(), setup["v_pages"].clone()
        out_b = torch.full((n, hq * d), float("nan"), device="cuda", dtype=torch.bfloat16)
        o.attention_decode_fused(out_b, source if source is not None else dense, bias, inv, True, q_start, q_len, kv_len, slot,
                                 setup["table"], k_b, v_b, n, hq, hkv, d, window, d ** -0.5, ns, scratch, counters, st,
                                 merge_in_scratch=merge_in_scratch, prefetch=None if merge_in_scratch else bias)
        assert int(st) == 0
        assert torch.equal(k_a.view(torch.int16), k_b.view(torch.int16)), "keys written differ"
        assert torch.equal(v_a.view(torch.int16), v_b.view(torch.int16)), "values written differ"
        assert not torch.isnan(out_b.float()).any()
        assert torch.equal(out_a.view(torch.int16), out_b.view(torch.int16)), "attention output differs"


# ---------------------------------------------------------------------------
# decode attention fed by TMA
# ---------------------------------------------------------------------------
TMA_CASES = [
    # hq, hkv, d, page
    (28, 4, 128, 16),       # the benchmark's layer
    (40, 8, 128, 16),       # groups of five
    (14, 2, 64, 8),
    (9, 1, 64, 32),         # nine heads in a group: two head tiles
    (20, 2, 64, 4),         # sixteen boxes to a tile
    (4, 2, 256, 16),
    (6, 1, 128, 64),        # a page is a tile
    (16, 2, 128, 128),      # a page is two tiles
]


@pytest.mark.parametrize("hq,hkv,d,page", TMA_CASES)
@pytest.mark.parametrize("window", [0, 40, 100])
@pytest.mark.parametrize("nsplit,stages", [(1, 2), (3, 0), (5, 3), (17, 2)])
def test_decode_attention_tma(hq, hkv, d, page, window, nsplit, stages):
    """Requests of 1 to 1,000 keys on permuted pages whose unused slots hold NaN, every one bringing its newest
    token: whole, in slices merged inside a cluster and through scratch memory, with windows that start inside a
    tile, and with rings of two stages (every stage is used many times) up to the deepest."""
    lengths = [1, 17, 64, 65, 129, 300, 1000]
    setup = paged_setup(lengths, page, hkv, d, torch.bfloat16, seed=hq + d + page)
    rows_of = [[n - 1] for n in lengths]
    q = torch.randn(len(lengths), hq, d, generator=torch.Generator().manual_seed(window + nsplit))
    for merge_in_scratch in ((False, True) if 1 < nsplit <= 16 else (False,)):
        got, qr = run_tensor_core_attention(setup, rows_of, q, hq, hkv, d, window, nsplit=nsplit, tma=True, stages=stages,
                                            merge_in_scratch=merge_in_scratch)
        for i, r in enumerate(rows_of):
            k = setup["k"][i].to(torch.bfloat16).float(); v = setup["v"][i].to(torch.bfloat16).float()
            want = dense_attention(qr[i:i + 1], k, v, r, window or None)
            assert torch.isfinite(got[i]).all(), f"request {i}: a slot that holds no key was read"
            assert torch.allclose(got[i:i + 1], want, **TOL["bfloat16"]), f"request {i} ({lengths[i]} keys)"


@pytest.mark.parametrize("hq,hkv,d", [(28, 4, 128), (20, 2, 64), (4, 2, 256), (9, 1, 64)])
@pytest.mark.parametrize("split_source", [0, 1, 3, 4, 9])
@pytest.mark.parametrize("window", [0, 40])
def test_decode_attention_tma_makes_q_k_v_itself(hq, hkv, d, split_source, window):
    """The TMA kernel on a decode-only step's untouched q/k/v product: bias, rotation by position, the write of the
    new key and value and the attention, against the plain formulas (rope and dense attention in fp32 on the CPU)
    and, for what lands in the cache, bit for bit against the kernel that does only that.  Newest positions at a
    page's first and last slot, at position 0 and in between; the new key's row reaches the products from the
    block's own arithmetic, so a copy that read the page before the write cannot matter."""
    o = ops()
    lengths = [1, 16 * 9 + 1, 16 * 11, 300, 64]
    page, theta = 16, 1e4
    setup = paged_setup(lengths, page, hkv, d, torch.bfloat16, seed=hq + d)
    n = len(lengths)
    width = (hq + 2 * hkv) * d
    g = torch.Generator().manual_seed(3)
    bias = dev(torch.randn(width, generator=g))
    inv = dev(theta ** (-torch.arange(0, d, 2, dtype=torch.float32) / d))
    i32 = lambda v: dev(torch.tensor(v, dtype=torch.int32))
    q_start, q_len, kv_len, slot = i32(list(range(n))), i32([1] * n), i32(lengths), i32(setup["slots"])
    positions, seq_of = i32([m - 1 for m in lengths]), i32(list(range(n)))
    if split_source:
        slices = dev(torch.randn(split_source, n, width, generator=g))
        source, dense = o.SplitSum(slices), torch.zeros(n, width, device="cuda", dtype=torch.bfloat16)
        product = slices.sum(0).cpu()
    else:
        dense = dev(torch.randn(n, width, generator=g), torch.bfloat16)
        source, product = None, dense.float().cpu()
    scratch = torch.full((o.decode_scratch_floats(hq, d),), float("nan"), device="cuda")
    counters = torch.zeros(o.decode_counter_ints(n, hkv, hq // hkv), dtype=torch.int32, device="cuda")
    st = status()
    # what the plain formulas give
    x = product + bias.cpu()
    pos = [m - 1 for m in lengths]
    q_new = plain_qwen2.rope(x[:, : hq * d].reshape(n, hq, d), pos, theta)
    k_new = plain_qwen2.rope(x[:, hq * d:(hq + hkv) * d].reshape(n, hkv, d), pos, theta)
    v_new = x[:, (hq + hkv) * d:].reshape(n, hkv, d)
    # the cache as the kernel that only writes leaves it
    k_a, v_a = setup["k_pages"].clone(), setup["v_pages"].clone()
    o.rope_kv_write(dense.clone(), bias, positions, seq_of, slot, setup["table"], inv, k_a, v_a, n, hq, hkv, d, True, st, source=source)
    for ns, merge_in_scratch in ((1, False), (3, False), (3, True)):
        k_b, v_b = setup["k_pages"].clone(), setup["v_pages"].clone()
        out = torch.full((n, hq * d), float("nan"), device="cuda", dtype=torch.bfloat16)
        o.attention_decode_tma(out, None, source if source is not None else dense, bias, inv, True, q_start, q_len, kv_len, slot,
                               setup["table"], k_b, v_b, n, hq, hkv, d, window, d ** -0.5, ns, scratch, counters, st,
                               merge_in_scratch=merge_in_scratch, prefetch=bias if ns == 1 else None)
        assert int(st) == 0
        assert torch.equal(k_a.view(torch.int16), k_b.view(torch.int16)) and torch.equal(v_a.view(torch.int16), v_b.view(torch.int16))
        got = out.float().cpu().reshape(n, hq, d)
        for i, m in enumerate(lengths):
            k = setup["k"][i].clone(); v = setup["v"][i].clone()
            k[m - 1], v[m - 1] = k_new[i], v_new[i]
            want = dense_attention(q_new[i:i + 1].to(torch.bfloat16).float(), k.to(torch.bfloat16).float(),
                                   v.to(torch.bfloat16).float(), [m - 1], window or None)
            assert torch.allclose(got[i:i + 1], want, **TOL["bfloat16"]), f"request {i} ({m} keys), {ns} slices"
    # a layer that reads another layer's cache: nothing is written, the newest key is already there
    k_c, v_c = k_a.clone(), v_a.clone()
    out_c = torch.full((n, hq * d), float("nan"), device="cuda", dtype=torch.bfloat16)
    o.attention_decode_tma(out_c, None, source if source is not None else dense, bias, inv, False, q_start, q_len, kv_len, slot,
                           setup["table"], k_c, v_c, n, hq, hkv, d, window, d ** -0.5, 3, scratch, counters, st)
    assert torch.equal(k_c.view(torch.int16), k_a.view(torch.int16)) and torch.equal(out_c, out) and int(st) == 0


def test_decode_attention_tma_refuses_and_reports():
    """Shapes the kernel does not take are refused in words; a block table without a page sets the page bit of the
    status word and the kernel returns (it reads nothing out of bounds)."""
    o = ops()
    hq, hkv, d = 4, 2, 64
    assert not o.decode_tma_supported(torch.bfloat16, 32, 16) and not o.decode_tma_supported(torch.float32, 64, 16)
    assert not o.decode_tma_supported(torch.bfloat16, 64, 24) and o.decode_tma_supported(torch.bfloat16, 64, 128)
    setup = paged_setup([100], 16, hkv, d, torch.bfloat16, seed=1)
    i32 = lambda v: dev(torch.tensor(v, dtype=torch.int32))
    q = dev(torch.randn(1, hq * d), torch.bfloat16)
    out = torch.zeros(1, hq * d, device="cuda", dtype=torch.bfloat16)
    scratch = torch.zeros(o.decode_scratch_floats(hq, d), device="cuda")
    counters = torch.zeros(o.decode_counter_ints(1, hkv, 2), dtype=torch.int32, device="cuda")
    args = (i32([0]), i32([1]), i32([100]), i32(setup["slots"]), setup["table"], setup["k_pages"], setup["v_pages"], 1, hq, hkv, d,
            0, d ** -0.5)
    with pytest.raises(o.KernelError, match="slices"):
        o.attention_decode_tma(out, q, None, None, None, False, *args, 129, scratch, counters, status())
    with pytest.raises(o.KernelError, match="aligned"):
        o.attention_decode_tma(out, dev(torch.zeros(hq * d + 8), torch.bfloat16)[1:hq * d + 1].view(1, -1), None, None, None, False,
                               *args, 2, scratch, counters, status())
    table = setup["table"].clone()
    table[setup["slots"][0], 3] = -1                         # keys 48..63 have no page
    st = status()
    o.attention_decode_tma(out, q, None, None, None, False, args[0], args[1], args[2], args[3], table, *args[5:], 2, scratch,
                           counters, st)
    assert int(st) == 2
