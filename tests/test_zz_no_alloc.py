"""The allocation-free decode attention entry point, called through its exported C symbol.

``tw_attn_decode_static`` is for callers that must not allocate device memory when they need
attention (a serving loop that cannot afford the device-wide stall of cudaMalloc, a component
with a memory budget fixed at start-up): its scratch lives in an array inside the library's
device image.  The test calls it twice in a row, with different inputs, and compares each
result with the ordinary entry point, which gets a scratch buffer from the caller.  The second
call finds the first call's leftovers in the array and must not be disturbed by them.  A call
that needs more scratch than the array holds must be refused with a message, not run.

The file sorts last, so a run that stops at the first failure has run every other test before.
It works alone in a fresh process as well as after the other tests.
"""
import ctypes
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

HQ, HKV, D, PAGE = 14, 2, 64, 16


def make_case(seed, lengths):
    g = torch.Generator().manual_seed(seed)
    n = len(lengths)
    blocks = [-(-length // PAGE) for length in lengths]
    pages = sum(blocks) + 3
    perm = torch.randperm(pages, generator=g).tolist()
    table = torch.full((n, max(blocks)), -1, dtype=torch.int32)
    cursor = 0
    for i, b in enumerate(blocks):
        table[i, :b] = torch.tensor(perm[cursor:cursor + b], dtype=torch.int32)
        cursor += b
    dev = lambda t, dt=None: t.to("cuda", dt) if dt else t.to("cuda")
    return dict(
        q=dev(torch.randn(n, HQ * D, generator=g), torch.bfloat16),
        k=dev(torch.randn(pages, HKV, PAGE, D, generator=g), torch.bfloat16),
        v=dev(torch.randn(pages, HKV, PAGE, D, generator=g), torch.bfloat16),
        table=dev(table), q_start=dev(torch.arange(n, dtype=torch.int32)),
        q_len=dev(torch.ones(n, dtype=torch.int32)), kv_len=dev(torch.tensor(lengths, dtype=torch.int32)),
        slot=dev(torch.arange(n, dtype=torch.int32)), n=n, pages=pages)


def call_static(lib, case, nsplit, status):
    out = torch.full((case["n"], HQ * D), float("nan"), device="cuda", dtype=torch.bfloat16)
    fn = lib.tw_attn_decode_static
    fn.restype = c_int
    ptr = lambda t: c_void_p(t.data_ptr())
    code = fn(ptr(out), c_int(out.stride(0)), ptr(case["q"]), c_int(case["q"].stride(0)), ptr(case["q_start"]),
              ptr(case["q_len"]), ptr(case["kv_len"]), ptr(case["slot"]), ptr(case["table"]),
              c_int(case["table"].shape[1]), ptr(case["k"]), ptr(case["v"]), c_int(case["n"]), c_int(HQ), c_int(HKV),
              c_int(PAGE), c_int(case["pages"]), c_int(0), c_float(D ** -0.5), c_int(nsplit), ptr(status),
              c_void_p(torch.cuda.current_stream().cuda_stream))
    return code, out


def call_ordinary(case, nsplit, status):
    from tessweave_engine_b200.csrc import ops
    out = torch.full((case["n"], HQ * D), float("nan"), device="cuda", dtype=torch.bfloat16)
    scratch = torch.empty(ops.decode_scratch_floats(HQ, D), device="cuda")
    counters = torch.zeros(ops.decode_counter_ints(case["n"], HKV, HQ // HKV), dtype=torch.int32, device="cuda")
    ops.attention_decode(out, case["q"], case["q_start"], case["q_len"], case["kv_len"], case["slot"], case["table"],
                         case["k"], case["v"], case["n"], HQ, HKV, D, 0, D ** -0.5, nsplit, scratch, counters, status)
    return out


def test_static_scratch_entry_point_matches_the_ordinary_one():
    from tessweave_engine_b200.csrc.build import load_library
    lib = load_library("attention_bf16", {"TW_HEAD_DIM": D})
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    before = torch.cuda.memory_allocated()
    for seed, lengths, nsplit in ((1, [700, 33, 1, 256], 6), (2, [90, 1500, 64], 9)):
        case = make_case(seed, lengths)
        want = call_ordinary(case, nsplit, status)
        code, got = call_static(lib, case, nsplit, status)
        torch.cuda.synchronize()
        assert code == 0, lib.tw_attn_decode_static_last_error
        assert int(status) == 0
        assert torch.isfinite(got.float()).all()
        assert torch.allclose(got.float(), want.float(), atol=2.5e-2, rtol=2.5e-2)
        del case, want, got
    assert torch.cuda.memory_allocated() <= before + (1 << 20)       # nothing is left allocated behind the calls
    # a call beyond the array's size is refused before anything is launched
    big = make_case(3, [64] * 64)
    lib.tw_attn_decode_static_last_error.restype = ctypes.c_char_p
    code, out = call_static(lib, big, 128, status)
    torch.cuda.synchronize()
    assert code == -2
    message = lib.tw_attn_decode_static_last_error().decode()
    assert "static array holds" in message and "128 slices" in message
    assert torch.isnan(out.float()).all()                               # nothing ran


def test_entry_points_refuse_what_the_kernel_cannot_take():
    """More slices than the merge has shared memory for, and a query the kernel's 16-byte loads cannot read,
    are refused by the C entry points themselves before anything is launched: the return code says so and
    the output is untouched.  (Nothing oversized is ever run.)"""
    from tessweave_engine_b200.csrc import ops
    from tessweave_engine_b200.csrc.build import load_library
    lib = load_library("attention_bf16", {"TW_HEAD_DIM": D})
    lib.tw_attn_decode_max_splits.restype = c_int
    limit = lib.tw_attn_decode_max_splits()
    assert limit == ops.DECODE_MAX_SPLITS
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    case = make_case(4, [1000])
    code, out = call_static(lib, case, limit + 1, status)        # 3.7 MB of partial results would fit the array
    torch.cuda.synchronize()
    assert code == 1 and torch.isnan(out.float()).all()           # cudaErrorInvalidValue, nothing ran
    code, out = call_static(lib, case, 1000, status)
    assert code == 1 and torch.isnan(out.float()).all()
    # a query that starts 2 bytes into a row
    shifted = dict(case, q=torch.zeros(HQ * D + 8, device="cuda", dtype=torch.bfloat16)[1:HQ * D + 1].view(1, HQ * D))
    assert shifted["q"].data_ptr() % 16 != 0
    code, out = call_static(lib, shifted, 4, status)
    torch.cuda.synchronize()
    assert code == 716 and torch.isnan(out.float()).all()         # cudaErrorMisalignedAddress
    # the Python wrappers say the same in words
    scratch = torch.empty(ops.decode_scratch_floats(HQ, D), device="cuda")
    counters = torch.zeros(ops.decode_counter_ints(1, HKV, HQ // HKV), dtype=torch.int32, device="cuda")
    out = torch.zeros(1, HQ * D, device="cuda", dtype=torch.bfloat16)
    for q, nsplit, word in ((case["q"], limit + 1, "slices"), (shifted["q"], 4, "aligned")):
        with pytest.raises(ops.KernelError, match=word):
            ops.attention_decode(out, q, case["q_start"], case["q_len"], case["kv_len"], case["slot"], case["table"],
                                 case["k"], case["v"], 1, HQ, HKV, D, 0, D ** -0.5, nsplit, scratch, counters, status)
    assert int(status) == 0
