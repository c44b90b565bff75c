"""Python side of the CUDA kernels: thin launch wrappers over the compiled libraries.

Each wrapper checks what the kernel assumes (device, element type, contiguity,
sizes it can take) and raises a clear error otherwise; a kernel is never handed
a shape it would compute wrongly.  There is no fallback: if a library cannot be
compiled or loaded, the call fails.  Launches go to torch's current stream, so
they order with library matrix products and can be captured in CUDA graphs.
"""
from __future__ import annotations

import ctypes
from ctypes import c_void_p, c_int, c_float, c_long
from dataclasses import dataclass

import torch

from .build import load_library

F32, BF16 = 0, 1


class KernelError(RuntimeError):
    pass


@dataclass
class SplitSum:
    """The result of a matrix product that was split over k: fp32 slices [slices, rows, width]
    whose sum (in slice order) is the product.  Kernels that consume it add the slices
    themselves; ``dense()`` adds them for anyone else."""
    slices: torch.Tensor

    def dense(self, dtype: torch.dtype, out: torch.Tensor | None = None) -> torch.Tensor:
        n, rows, width = self.slices.shape
        out = out if out is not None else torch.empty(rows, width, dtype=dtype, device=self.slices.device)
        code = _fn("gemm_smallm", "tw_reduce_partial")(_ptr(out), _ptr(self.slices), c_int(n), c_long(rows * width),
                                                       c_int(dtype_code(dtype)), _stream())
        _check(code, "reduce_partial")
        return out


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 activations, not {dtype}")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    # the raw handle of torch's current stream (what torch.cuda.current_stream().cuda_stream gives, without
    # building a Stream object for every launch)
    return c_void_p(torch._C._cuda_getCurrentRawStream(torch.cuda.current_device()))


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


def _cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernel operands must live on a CUDA device; this engine has no CPU path")


def _check(code: int, what: str) -> None:
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code} at launch "
                          f"({torch.cuda.get_device_name() if torch.cuda.is_available() else 'no device'})")


_sigs_done: set[str] = set()
LAUNCHES = [0]      # kernel launchers called so far (each call launches at least one kernel)
CALL_LOG: list[str] | None = None     # when a list: the launchers called, by name (who measures asks which kernel ran)


def note_call(name: str) -> None:
    if CALL_LOG is not None:
        CALL_LOG.append(name)


def _fn(lib_name: str, fn_name: str, defines=None):
    LAUNCHES[0] += 1
    note_call(fn_name)
    lib = load_library(lib_name, defines)
    fn = getattr(lib, fn_name)
    key = f"{lib_name}:{fn_name}:{defines}"
    if key not in _sigs_done:
        fn.restype = c_int
        _sigs_done.add(key)
    return fn


# ---------------------------------------------------------------------------
def embed(resid: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, n_tokens: int, status: torch.Tensor,
          device_tokens: torch.Tensor | None = None) -> None:
    """resid[n] = float(table[ids[n]]); resid is fp32 [>=n_tokens, hidden].  An id -(i + 1) is
    replaced by ``device_tokens[i]`` (int32, on the device) inside the kernel."""
    _cuda(resid, table, ids, status, device_tokens)
    _need(device_tokens is None or device_tokens.dtype == torch.int32, "embed: device tokens must be int32")
    _need(resid.dtype == torch.float32 and resid.is_contiguous(), "embed: residual stream must be contiguous fp32")
    _need(table.is_contiguous() and ids.dtype == torch.int32, "embed: table contiguous, ids int32")
    _need(resid.shape[0] >= n_tokens and ids.numel() >= n_tokens and resid.shape[1] == table.shape[1],
          "embed: shapes disagree")
    code = _fn("elementwise", "tw_embed")(_ptr(resid), _ptr(table), _ptr(ids), _ptr(device_tokens),
                                          c_int(0 if device_tokens is None else device_tokens.numel()), c_int(n_tokens),
                                          c_int(table.shape[1]), c_int(table.shape[0]),
                                          c_int(dtype_code(table.dtype)), _ptr(status), _stream())
    _check(code, "embed")


def add_rmsnorm(out: torch.Tensor, resid: torch.Tensor, delta, weight: torch.Tensor,
                eps: float, n_rows: int, rows: torch.Tensor | None = None) -> None:
    """resid += delta (in place, fp32) and out = rmsnorm(resid) * weight.

    ``delta`` is None, a tensor of the output's type, or a ``SplitSum`` (fp32 slices of a
    matrix product split over k, added here in slice order).  With ``rows`` (int32 indices)
    only those rows are normalised, into out[0..n_rows), and the residual stream is left
    as it was.
    """
    partial, nsplit, split_stride = None, 0, 0
    if isinstance(delta, SplitSum):
        partial, nsplit, split_stride = delta.slices, delta.slices.shape[0], delta.slices.stride(0)
        _need(partial.dtype == torch.float32 and partial.shape[2] == resid.shape[1] and partial[0].is_contiguous(),
              "rmsnorm: split sum must be fp32 [slices, rows, hidden]")
        delta = None
    _cuda(out, resid, delta, weight, rows, partial)
    hidden = resid.shape[1]
    _need(resid.dtype == torch.float32 and resid.is_contiguous(), "rmsnorm: residual stream must be contiguous fp32")
    _need(weight.dtype == torch.float32 and weight.numel() == hidden, "rmsnorm: weight must be fp32 [hidden]")
    _need(out.is_contiguous() and out.shape[1] == hidden and out.shape[0] >= n_rows, "rmsnorm: bad output")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous() and delta.shape[1] == hidden,
              "rmsnorm: delta must match the output type and width")
    if rows is not None:
        _need(rows.dtype == torch.int32 and rows.numel() >= n_rows, "rmsnorm: rows must be int32")
    else:
        _need(resid.shape[0] >= n_rows, "rmsnorm: fewer residual rows than asked")
    code = _fn("elementwise", "tw_add_rmsnorm")(_ptr(out), _ptr(resid), _ptr(delta), _ptr(partial), c_int(nsplit),
                                                c_long(split_stride), _ptr(weight), c_float(eps),
                                                c_int(n_rows), c_int(hidden), _ptr(rows),
                                                c_int(dtype_code(out.dtype)), _stream())
    _check(code, "add_rmsnorm")


def rope_kv_write(qkv: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor, seq_of_token: torch.Tensor,
                  seq_slot: torch.Tensor, block_table: torch.Tensor, inv_freq: torch.Tensor | None,
                  k_pages: torch.Tensor, v_pages: torch.Tensor, n_tokens: int, n_q_heads: int, n_kv_heads: int,
                  head_dim: int, write_cache: bool, status: torch.Tensor, source: "SplitSum | None" = None) -> None:
    """Add the bias, rotate q and k by position, store k and v in their cache pages.

    qkv: [>=n_tokens, (Hq + 2 Hkv) * D]; k_pages/v_pages: [pages, Hkv, page, D].  With
    ``source`` the projection is read from the fp32 slices of a split product instead of
    ``qkv``; the rotated q is written to ``qkv`` either way.
    """
    _cuda(qkv, bias, positions, seq_of_token, seq_slot, block_table, inv_freq, k_pages, v_pages, status)
    width = (n_q_heads + 2 * n_kv_heads) * head_dim
    partial, nsplit, split_stride = None, 0, 0
    if source is not None:
        partial, nsplit, split_stride = source.slices, source.slices.shape[0], source.slices.stride(0)
        _need(partial.is_cuda and partial.dtype == torch.float32 and partial.shape[2] == width
              and partial[0].is_contiguous() and partial.shape[1] >= n_tokens, "rope: bad split source")
    _need(qkv.stride(1) == 1 and qkv.shape[1] == width, "rope: qkv row must be [q | k | v] heads")
    _need(head_dim % 2 == 0, f"rope: head_dim {head_dim} must be even")
    _need(k_pages.dtype == qkv.dtype and v_pages.dtype == qkv.dtype and k_pages.is_contiguous()
          and v_pages.is_contiguous(), "rope: cache pages must be contiguous and of the activation type")
    _need(tuple(k_pages.shape[1:]) == (n_kv_heads, k_pages.shape[2], head_dim) and v_pages.shape == k_pages.shape,
          "rope: cache pages must be [pages, kv_heads, page, head_dim]")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2 and block_table.is_contiguous(),
          "rope: block table must be contiguous int32 [requests, blocks]")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() == width, "rope: bias must be fp32 [(Hq+2Hkv)*D]")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2, "rope: inv_freq must be fp32 [D/2]")
    code = _fn("elementwise", "tw_rope_kv_write")(
        _ptr(qkv), c_int(qkv.stride(0)), _ptr(partial), c_int(nsplit), c_long(split_stride), _ptr(bias),
        _ptr(positions), _ptr(seq_of_token), _ptr(seq_slot),
        _ptr(block_table), c_int(block_table.shape[1]), _ptr(inv_freq), _ptr(k_pages), _ptr(v_pages),
        c_int(n_tokens), c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(k_pages.shape[2]),
        c_int(k_pages.shape[0]), c_int(1 if write_cache else 0), c_int(dtype_code(qkv.dtype)), _ptr(status), _stream())
    _check(code, "rope_kv_write")


def rotate_heads(rows: torch.Tensor, bias: torch.Tensor | None, positions: torch.Tensor, seq_of_token: torch.Tensor,
                 inv_freq: torch.Tensor | None, n_tokens: int, n_heads: int, head_dim: int) -> None:
    """In place on the first ``n_heads`` heads of each packed row: add the bias, then rotate
    by position (either may be absent).  Nothing is written to a cache."""
    _cuda(rows, bias, positions, seq_of_token, inv_freq)
    _need(rows.stride(1) == 1 and rows.shape[1] >= n_heads * head_dim and head_dim % 2 == 0, "rotate_heads: bad rows")
    if bias is not None:
        _need(bias.dtype == torch.float32 and bias.numel() >= n_heads * head_dim, "rotate_heads: bias must be fp32")
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2, "rotate_heads: inv_freq fp32 [D/2]")
    code = _fn("elementwise", "tw_rope_kv_write")(
        _ptr(rows), c_int(rows.stride(0)), _ptr(None), c_int(0), c_long(0), _ptr(bias), _ptr(positions),
        _ptr(seq_of_token), _ptr(None), _ptr(None),
        c_int(0), _ptr(inv_freq), _ptr(None), _ptr(None), c_int(n_tokens), c_int(n_heads), c_int(0), c_int(head_dim),
        c_int(1), c_int(0), c_int(0), c_int(dtype_code(rows.dtype)), _ptr(None), _stream())
    _check(code, "rotate_heads")


def silu_mul(out: torch.Tensor, gate_up, n_rows: int, interleaved: bool = False) -> None:
    """out[n, i] = silu(gate[n, i]) * up[n, i].  Columns of ``gate_up`` are [all gates | all ups],
    or with ``interleaved`` groups of 16: eight gates followed by their eight ups.  ``gate_up`` may be a
    ``SplitSum`` (fp32 slices of the product, added here in slice order); ``out`` is then bfloat16."""
    inter = out.shape[1]
    if isinstance(gate_up, SplitSum):
        slices = gate_up.slices
        _cuda(out, slices)
        _need(out.dtype == torch.bfloat16 and out.is_contiguous() and slices.dtype == torch.float32 and slices.dim() == 3
              and slices.shape[1] >= n_rows and slices.shape[2] == 2 * inter and slices[0].is_contiguous()
              and inter % 4 == 0 and (not interleaved or inter % 8 == 0) and out.shape[0] >= n_rows,
              "silu_mul: slices must be fp32 [slices, rows, 2I], the output bf16 [rows, I], I a multiple of 4 (8 interleaved)")
        code = _fn("elementwise", "tw_silu_mul_slices")(_ptr(out), _ptr(slices), c_int(slices.shape[0]), c_long(slices.stride(0)),
                                                        c_int(n_rows), c_int(inter), c_int(1 if interleaved else 0), _stream())
        _check(code, "silu_mul_slices")
        return
    _cuda(out, gate_up)
    _need(gate_up.shape[1] == 2 * inter and gate_up.is_contiguous() and out.is_contiguous()
          and gate_up.dtype == out.dtype, "silu_mul: gate_up must be contiguous [n, 2I] of the output type")
    _need(not interleaved or inter % 8 == 0, "silu_mul: interleaved columns need a multiple of 8")
    code = _fn("elementwise", "tw_silu_mul")(_ptr(out), _ptr(gate_up), c_int(n_rows), c_int(inter),
                                             c_int(1 if interleaved else 0), c_int(dtype_code(out.dtype)), _stream())
    _check(code, "silu_mul")


def attention_generic(out: torch.Tensor, q: torch.Tensor, positions: torch.Tensor, seq_of_token: torch.Tensor,
                      seq_slot: torch.Tensor, block_table: torch.Tensor, k_pages: torch.Tensor, v_pages: torch.Tensor,
                      n_tokens: int, n_q_heads: int, n_kv_heads: int, head_dim: int, window: int, scale: float,
                      status: torch.Tensor) -> None:
    """Exact paged causal attention, one block per (token, head).  q may be a column
    slice of the packed qkv buffer (row stride is passed on)."""
    _cuda(out, q, positions, seq_of_token, seq_slot, block_table, k_pages, v_pages, status)
    _need(head_dim <= 256, f"attention: head_dim {head_dim} above 256 is not supported")
    _need(n_q_heads % n_kv_heads == 0, "attention: query heads must be a multiple of key/value heads")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and q.dtype == out.dtype == k_pages.dtype, "attention: bad operands")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention: bad block table")
    code = _fn("attention_generic", "tw_attn_generic")(
        _ptr(out), c_int(out.stride(0)), _ptr(q), c_int(q.stride(0)), _ptr(positions), _ptr(seq_of_token),
        _ptr(seq_slot), _ptr(block_table), c_int(block_table.shape[1]), _ptr(k_pages), _ptr(v_pages), c_int(n_tokens),
        c_int(n_q_heads), c_int(n_kv_heads), c_int(head_dim), c_int(k_pages.shape[2]), c_int(k_pages.shape[0]),
        c_int(window), c_float(scale), c_int(dtype_code(q.dtype)), _ptr(status), _stream())
    _check(code, "attention_generic")


def sample(out: torch.Tensor, logits: torch.Tensor, n_rows: int, temperature: torch.Tensor | None = None,
           seed: torch.Tensor | None = None, counter: torch.Tensor | None = None) -> None:
    """out[r] = chosen token of row r (int32).  Rows with temperature 0 are greedy."""
    _cuda(out, logits, temperature, seed, counter)
    _need(logits.dtype == torch.float32 and logits.is_contiguous() and logits.dim() == 2, "sample: logits fp32 [rows, vocab]")
    _need(out.dtype == torch.int32 and out.numel() >= n_rows, "sample: out must be int32")
    if temperature is not None:
        _need(temperature.dtype == torch.float32 and seed is not None and counter is not None
              and seed.dtype == torch.int64 and counter.dtype == torch.int64, "sample: temperature fp32, seed/counter int64")
    code = _fn("sampling", "tw_sample")(_ptr(out), _ptr(logits), c_int(n_rows), c_int(logits.shape[1]),
                                        _ptr(temperature), _ptr(seed), _ptr(counter), _stream())
    _check(code, "sample")


# ---------------------------------------------------------------------------
# bf16 tensor-core attention (one compiled library per head size)
# ---------------------------------------------------------------------------
DECODE_MAX_SPLITS = 128          # most slices of a request's keys (the merge keeps two floats per head and slice in shared memory)
DECODE_SCRATCH_UNITS = 1024      # most (request, split) pairs whose partial results fit the scratch buffer
_SM_COUNT = 148


def tensor_core_attention_supported(dtype: torch.dtype, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256


def tcgen05_attention_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """The tcgen05 prefill attention takes bfloat16, head sizes 64 and 128, and pages of at least
    8 keys that divide a tile of 128 keys or are a multiple of it."""
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and page_size >= 8
            and (128 % page_size == 0 or page_size % 128 == 0))


TCGEN05_ATTENTION_MIN_TOKENS = 128


def prefer_tcgen05_attention(dtype: torch.dtype, head_dim: int, page_size: int, max_q_len: int) -> bool:
    """Whether a step whose longest portion has ``max_q_len`` tokens runs its prompt attention on
    the tcgen05 kernel.  TESSWEAVE_PREFILL_ATTENTION=mma|tcgen05 forces one of the two (the latter
    only for shapes the kernel takes)."""
    import os
    if not tcgen05_attention_supported(dtype, head_dim, page_size):
        return False
    forced = os.environ.get("TESSWEAVE_PREFILL_ATTENTION")
    if forced == "mma":
        return False
    if forced == "tcgen05":
        return True
    return max_q_len >= TCGEN05_ATTENTION_MIN_TOKENS


def decode_splits(n_seqs: int, n_kv_heads: int, group: int, max_kv_len: int) -> int:
    """How many slices the keys of a request are cut into, so that the launch fills the GPU.
    Up to 16 slices merge inside a thread-block cluster, which saves 2-3 us over the merge through
    scratch memory; clusters of 15 and 16 are only placed well when there are few of them, so with many
    (request, head) groups 15 and 16 slices become 14 (measured on B200, batch 8, 4 key/value heads,
    4096 keys, a whole decode step: 3.61 ms with 13 or 14 slices, 3.64 with 12, 3.94 with 16, 4.02 with 15)."""
    import os
    forced = os.environ.get("TESSWEAVE_DECODE_SPLITS")
    if forced:
        return max(1, min(int(forced), 128, DECODE_SCRATCH_UNITS // max(1, n_seqs)))
    head_tiles = (group + 7) // 8
    tiles = max(1, -(-max_kv_len // 64))
    groups = max(1, n_seqs * n_kv_heads * head_tiles)
    # the kernel fits four blocks on an SM; aim at a little under one full wave of blocks
    room = 7 * _SM_COUNT // 2
    target = max(1, (room + groups // 2) // groups)        # rounded: 1.9 blocks' worth of room is two slices
    if target > 4 and target * groups > room:
        # clusters of five and more blocks are no longer all placed at once when the launch has more than 3.5 blocks
        # per SM (batch 12, 4 key/value heads, a whole decode step: 3.81 ms with 10 slices, 4.21 with 11)
        target = max(4, room // groups)
    elif 1 < target <= 4 and target * groups > 15 * _SM_COUNT // 4:
        # small clusters fill the SMs a little further (batch 44: 528 blocks of 3 slices, 5.23 ms against 5.51 with 2),
        # but not to the last slot (batch 48: 576 blocks, 6.56 ms against 5.59 with 2)
        target = max(1, (15 * _SM_COUNT // 4) // groups)
    nsplit = max(1, min(tiles, target, 128, DECODE_SCRATCH_UNITS // max(1, n_seqs)))
    if 16 < nsplit <= 64 and max_kv_len <= 8192:
        # up to 8,192 keys the merge inside a cluster beats more slices merged through scratch memory (4,096 keys:
        # batch 3 / 4 / 6 steps take 3.24 / 3.26 / 3.37 ms with 14-16 slices against 3.30 / 3.33 / 3.52 with 21-32);
        # with longer contexts and few requests more slices win (16,384 keys, batch 2: 3.62 ms with 64, 3.83 with 16)
        nsplit = 16
    if 14 < nsplit <= 16 and groups > 8:
        nsplit = 14          # at every context length: 16,384 keys 4.53 ms with 14 slices, 5.20 with 16; 32,768 keys 5.85 and 7.05
    # the kernel cuts the keys into slices of a multiple of 64 keys: no slice without keys
    per = -(-(-(-max_kv_len // nsplit)) // 64) * 64
    return max(1, -(-max_kv_len // per))


def decode_scratch_floats(n_q_heads: int, head_dim: int) -> int:
    return DECODE_SCRATCH_UNITS * n_q_heads * (head_dim + 2)


def decode_counter_ints(n_seqs: int, n_kv_heads: int, group: int) -> int:
    """int32 counters (zero before the first launch, left zero by every launch) the split
    decode kernel uses to find the block that finishes last."""
    return max(n_seqs, DECODE_SCRATCH_UNITS) * n_kv_heads * ((group + 7) // 8)


def _attn_common_checks(out, q, block_table, k_pages, v_pages, n_q_heads, n_kv_heads, head_dim):
    _need(tensor_core_attention_supported(q.dtype, head_dim),
          f"tensor-core attention takes bfloat16 and head sizes that are multiples of 16 up to 256, not {q.dtype}/{head_dim}")
    _need(n_q_heads % n_kv_heads == 0, "attention: query heads must be a multiple of key/value heads")
    _need(q.stride(1) == 1 and out.stride(1) == 1 and out.dtype == q.dtype == k_pages.dtype == v_pages.dtype,
          "attention: operands must be bfloat16 with unit inner stride")
    _need(q.stride(0) % 2 == 0 and q.storage_offset() % 2 == 0 and out.stride(0) % 2 == 0, "attention: rows must be 4-byte aligned")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape[3] == head_dim
          and k_pages.shape[1] == n_kv_heads, "attention: cache pages must be contiguous [pages, kv_heads, page, head_dim]")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention: bad block table")


def attention_decode(out, q, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, k_pages, v_pages, n_seqs,
                     n_q_heads, n_kv_heads, head_dim, window, scale, nsplit, scratch, counters, status,
                     merge_in_scratch: bool = False) -> None:
    """Split-KV attention for the requests of the batch that bring one token (others are skipped).
    Up to 16 slices merge inside a thread-block cluster; more (or all, with ``merge_in_scratch``)
    merge through ``scratch`` (fp32, the slices' partial results) and ``counters`` (int32, all
    zero, left zero), which find the block that finishes last."""
    _cuda(out, q, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, k_pages, v_pages, scratch, counters, status)
    _attn_common_checks(out, q, block_table, k_pages, v_pages, n_q_heads, n_kv_heads, head_dim)
    _need(out.stride(0) % 4 == 0 and out.data_ptr() % 8 == 0, "attention_decode: output rows must be 8-byte aligned")
    _need(q.data_ptr() % 16 == 0 and q.stride(0) % 8 == 0, "attention_decode: rows of q must be 16-byte aligned")
    _need(1 <= nsplit <= DECODE_MAX_SPLITS, f"attention_decode: 1 to {DECODE_MAX_SPLITS} slices, not {nsplit}")
    if nsplit > 1:
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.data_ptr() % 16 == 0
              and scratch.numel() >= n_seqs * n_q_heads * nsplit * (head_dim + 2), "attention_decode: scratch too small")
        _need(counters is not None and counters.dtype == torch.int32
              and counters.numel() >= n_seqs * n_kv_heads * ((n_q_heads // n_kv_heads + 7) // 8),
              "attention_decode: too few counters")
    code = _fn("attention_bf16", "tw_attn_decode", {"TW_HEAD_DIM": head_dim})(
        _ptr(out), c_int(out.stride(0)), _ptr(q), c_int(q.stride(0)), _ptr(seq_q_start), _ptr(seq_q_len),
        _ptr(seq_kv_len), _ptr(seq_slot), _ptr(block_table), c_int(block_table.shape[1]), _ptr(k_pages), _ptr(v_pages),
        c_int(n_seqs), c_int(n_q_heads), c_int(n_kv_heads), c_int(k_pages.shape[2]), c_int(k_pages.shape[0]),
        c_int(window), c_float(scale), c_int(nsplit), c_int(1 if merge_in_scratch else 0), _ptr(scratch), _ptr(counters),
        _ptr(status), _stream())
    _check(code, "attention_decode")


WEIGHT_PREFETCH_BYTES = 24 << 20


def weight_prefetch_bytes() -> int:
    """How much of the weights that the part after the attention streams first (the feed-forward's first matrix)
    a decode step's attention asks into L2 while its slices merge.  Measured on a 7B-size layer: 24 to 32 MB is
    best at 1, 8 and 64 requests; more competes with the output product that runs in between, and asking for
    that product's own matrix gains nothing.  TESSWEAVE_WEIGHT_PREFETCH_MB overrides it; 0 switches it off."""
    import os
    mb = os.environ.get("TESSWEAVE_WEIGHT_PREFETCH_MB")
    return WEIGHT_PREFETCH_BYTES if mb is None else max(0, int(mb)) << 20


PRODUCT_PREFETCH_BYTES = 16 << 20


def weight_head(w: torch.Tensor | None, nbytes: int, skip_bytes: int = 0) -> torch.Tensor | None:
    """``nbytes`` of a contiguous weight from byte ``skip_bytes`` on as a flat view (what there is of them), or None."""
    if w is None or nbytes <= 0 or not w.is_contiguous():
        return None
    size = w.element_size()
    part = w.view(-1)[skip_bytes // size: (skip_bytes + nbytes) // size]
    return part if part.numel() else None


OUTPUT_PRODUCT_PREFETCH_BYTES = 24 << 20


def output_product_prefetch_bytes() -> int:
    """How much more of the feed-forward's first matrix the attention's output product asks into L2 when its own
    stream of weights ends, after what the attention kernel asked for.  The feed-forward's product is resident by
    then and fetches its first rows itself; these are rows it reaches later.  Measured on a 7B-size layer, whole
    decode steps: 8 / 16 / 24 / 32 / 48 / 64 / 96 MB give 0.6 / 1.0 / 1.2 / 1.2 / 1.1 / 0.6 / 0 % at 8 requests and
    the same at one; at the 14B sizes 16 and 24 MB are better than 32 (one request: 2 and 1 %).
    TESSWEAVE_OUTPUT_PREFETCH_MB overrides it; 0 switches it off."""
    import os
    mb = os.environ.get("TESSWEAVE_OUTPUT_PREFETCH_MB")
    return OUTPUT_PRODUCT_PREFETCH_BYTES if mb is None else max(0, int(mb)) << 20


def product_prefetch_bytes() -> int:
    """How much of the next matrix a small-batch product asks into L2 when its own stream of weights ends
    (gate/up before down).  Measured on a 7B-size layer: 8 to 24 MB are alike, 0.6 to 0.8 % of a step at 1 and 8
    requests.  Before a product that is resident early (q/k/v behind the norm, the attention's output product)
    the same request makes the step slower, so only the feed-forward uses it.  TESSWEAVE_PRODUCT_PREFETCH_MB
    overrides it; 0 switches it off."""
    import os
    mb = os.environ.get("TESSWEAVE_PRODUCT_PREFETCH_MB")
    return PRODUCT_PREFETCH_BYTES if mb is None else max(0, int(mb)) << 20


def weight_prefetch_min_cache_bytes() -> int:
    """The attention of a decode step prefetches weights only if it reads at least this much of the cache: a
    shorter kernel ends while the output product still fetches its own matrix, and the prefetch gets in its way
    (one request at 512 keys of a 7B-size layer: 1.4% slower with it).  TESSWEAVE_WEIGHT_PREFETCH_MIN_KB overrides."""
    import os
    kb = os.environ.get("TESSWEAVE_WEIGHT_PREFETCH_MIN_KB")
    return (2 << 20) if kb is None else int(kb) << 10


def fused_decode_enabled() -> bool:
    """TESSWEAVE_FUSED_DECODE=0 keeps bias, rotation and cache write of decode-only steps in a kernel of their own."""
    import os
    return os.environ.get("TESSWEAVE_FUSED_DECODE", "1") != "0"


def attention_decode_fused(out, source, bias, inv_freq, write_cache, seq_q_start, seq_q_len, seq_kv_len, seq_slot,
                           block_table, k_pages, v_pages, n_seqs, n_q_heads, n_kv_heads, head_dim, window, scale,
                           nsplit, scratch, counters, status, merge_in_scratch: bool = False,
                           prefetch: torch.Tensor | None = None) -> None:
    """Decode attention straight from the q/k/v product of a decode-only step: the kernel adds ``bias``,
    rotates q and k by position (``inv_freq``), writes the new key and value into their cache pages
    (``write_cache``) and attends.  ``source`` is the product: a ``SplitSum`` of fp32 slices or a bf16
    [rows, (Hq + 2 Hkv) D] tensor.  ``prefetch``: a contiguous tensor the next kernel streams (its weights);
    the blocks ask for it to be brought into L2 once their keys are in.  The other arguments are those of
    ``attention_decode``."""
    width = (n_q_heads + 2 * n_kv_heads) * head_dim
    partial = dense = None
    nslices = slice_stride = dense_stride = 0
    if isinstance(source, SplitSum):
        partial = source.slices
        _need(partial.is_cuda and partial.dtype == torch.float32 and partial.dim() == 3 and partial.shape[2] == width
              and partial[0].is_contiguous(), "attention_decode_fused: bad split source")
        nslices, slice_stride = partial.shape[0], partial.stride(0)
    else:
        dense = source
        _need(dense.is_cuda and dense.dtype == torch.bfloat16 and dense.dim() == 2 and dense.shape[1] == width
              and dense.stride(1) == 1, "attention_decode_fused: the product must be bf16 [rows, (Hq + 2 Hkv) D]")
        dense_stride = dense.stride(0)
    _cuda(out, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, k_pages, v_pages, scratch, counters, status,
          bias, inv_freq)
    _need(tensor_core_attention_supported(out.dtype, head_dim) and out.dtype == k_pages.dtype == v_pages.dtype,
          "attention_decode_fused: bfloat16 and a head size that is a multiple of 16 up to 256")
    _need(n_q_heads % n_kv_heads == 0, "attention: query heads must be a multiple of key/value heads")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape[3] == head_dim
          and k_pages.shape[1] == n_kv_heads and v_pages.shape == k_pages.shape,
          "attention: cache pages must be contiguous [pages, kv_heads, page, head_dim]")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention: bad block table")
    _need(out.stride(1) == 1 and out.stride(0) % 4 == 0 and out.data_ptr() % 8 == 0,
          "attention_decode_fused: output rows must be 8-byte aligned")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == width), "attention_decode_fused: bias must be fp32")
    _need(inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2),
          "attention_decode_fused: inv_freq must be fp32 [D/2]")
    _need(1 <= nsplit <= DECODE_MAX_SPLITS, f"attention_decode_fused: 1 to {DECODE_MAX_SPLITS} slices, not {nsplit}")
    if nsplit > 1:
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.data_ptr() % 16 == 0
              and scratch.numel() >= n_seqs * n_q_heads * nsplit * (head_dim + 2), "attention_decode: scratch too small")
        _need(counters is not None and counters.dtype == torch.int32
              and counters.numel() >= n_seqs * n_kv_heads * ((n_q_heads // n_kv_heads + 7) // 8),
              "attention_decode: too few counters")
    code = _fn("attention_bf16", "tw_attn_decode_fused", {"TW_HEAD_DIM": head_dim})(
        _ptr(out), c_int(out.stride(0)), _ptr(partial), c_int(nslices), ctypes.c_longlong(slice_stride), _ptr(dense),
        c_int(dense_stride), _ptr(bias), _ptr(inv_freq), c_int(1 if write_cache else 0), _ptr(seq_q_start), _ptr(seq_q_len),
        _ptr(seq_kv_len), _ptr(seq_slot), _ptr(block_table), c_int(block_table.shape[1]), _ptr(k_pages), _ptr(v_pages),
        c_int(n_seqs), c_int(n_q_heads), c_int(n_kv_heads), c_int(k_pages.shape[2]), c_int(k_pages.shape[0]),
        c_int(window), c_float(scale), c_int(nsplit), c_int(1 if merge_in_scratch else 0), _ptr(scratch), _ptr(counters),
        _ptr(status), _ptr(prefetch), ctypes.c_longlong(prefetch.numel() * prefetch.element_size() if prefetch is not None else 0),
        _stream())
    _check(code, "attention_decode_fused")


# ---------------------------------------------------------------------------
# decode attention fed by TMA (head sizes that are multiples of 64)
# ---------------------------------------------------------------------------
def decode_tma_supported(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether single-token requests attend through ``attention_decode_tma``: bfloat16, a head size of 64, 128,
    192 or 256, and pages that are a whole fraction (at least 4 keys) or a whole multiple of a 64-key tile.
    TESSWEAVE_DECODE_TMA=0 keeps the kernel that loads keys through registers."""
    import os
    if os.environ.get("TESSWEAVE_DECODE_TMA", "1") == "0":
        return False
    return (dtype == torch.bfloat16 and head_dim % 64 == 0 and 64 <= head_dim <= 256 and page_size >= 4
            and (64 % page_size == 0 or page_size % 64 == 0))


def decode_tma_splits(n_seqs: int, n_kv_heads: int, group: int, max_kv_len: int) -> int:
    """How many slices the TMA decode attention cuts a request's keys into.  Two blocks share an SM (a ring of
    three 64-key tiles each), and a block alone does not pull its share of the bandwidth, so the launch is filled
    to about 256 blocks -- not to the last of the 296 places: clusters that do not all find room at once start a
    second round (measured on B200 at 4,096 keys, whole decode steps of the 7B-sized model: batch 8 with 8 slices
    3.33 ms, with 4 slices 3.53, with 9 (288 blocks) 3.75; batch 12 with 5 slices 3.61 ms, with 6 (288 blocks)
    4.07, with 3 (144 blocks) 4.71; batch 4 with 13 slices 3.15 ms, with 14 or 16 3.5; batch 2 with 8 slices 3.18
    ms, with 12 or 16 3.4 to 3.5).  Few requests with long contexts take more slices and merge through scratch
    memory (16,384 keys, batch 2, 12 layers: 1.56 ms with 32 slices, 1.89 with 16).
    TESSWEAVE_DECODE_SPLITS forces a number."""
    import os
    forced = os.environ.get("TESSWEAVE_DECODE_SPLITS")
    tiles = max(1, -(-max_kv_len // 64))
    most = min(tiles, DECODE_MAX_SPLITS, DECODE_SCRATCH_UNITS // max(1, n_seqs))
    if forced:
        return max(1, min(int(forced), most))
    groups = max(1, n_seqs * n_kv_heads * ((group + 7) // 8))
    if groups <= 8 and max_kv_len > 8192:
        want = min(32, 256 // groups)
    elif groups <= 4:
        want = 16
    elif groups <= 8:
        want = 8
    elif groups <= 16:
        want = 13
    else:
        want = max(1, 256 // groups)
    nsplit = max(1, min(want, most))
    per = -(-(-(-max_kv_len // nsplit)) // 64) * 64          # slices are whole tiles: no slice without keys
    return max(1, -(-max_kv_len // per))


DECODE_TMA_CLUSTER_SLICES = 16      # more slices than this merge through scratch memory, without clusters


def decode_attention_resident_early(blocks: int, nsplit: int) -> bool:
    """Whether the q/k/v product of a decode-only step lets the TMA decode attention become resident while it runs
    (griddepcontrol.launch_dependents at its start), so that the attention's copies are under way when the
    product ends.  Clusters are only all placed at once on a GPU that is mostly free: measured on B200, whole
    steps of the 7B-sized model, with the trigger against without: 40 to 64 blocks (1 or 2 requests) 1.4 to 1.7 %
    faster, 144 and 156 blocks (4 requests at 512 keys, 3 at 4,096) 1.7 and 1.1 % faster, 208 blocks (4 requests
    at 4,096 keys) 9 % slower, 256 blocks (8 requests) 5 to 10 % slower; launches that merge through scratch
    memory (no clusters) 1 % faster at 128 and at 256 blocks.  TESSWEAVE_DECODE_EARLY=0/1 forces it."""
    import os
    forced = os.environ.get("TESSWEAVE_DECODE_EARLY")
    if forced is not None:
        return forced == "1"
    return nsplit > DECODE_TMA_CLUSTER_SLICES or blocks * 10 <= _SM_COUNT * 11


def attention_decode_tma(out, q, source, bias, inv_freq, write_cache, seq_q_start, seq_q_len, seq_kv_len, seq_slot,
                         block_table, k_pages, v_pages, n_seqs, n_q_heads, n_kv_heads, head_dim, window, scale, nsplit,
                         scratch, counters, status, merge_in_scratch: bool = False, prefetch: torch.Tensor | None = None,
                         stages: int = 0) -> None:
    """Split-KV attention for the requests of the batch that bring one token, keys and values brought in by TMA.
    Either ``q`` (bf16 [rows, Hq D], 16-byte aligned rows) or ``source`` -- the step's untouched q/k/v product, a
    ``SplitSum`` or a bf16 [rows, (Hq + 2 Hkv) D] tensor, which the kernel biases, rotates and (``write_cache``)
    stores itself -- is given.  The other arguments are those of ``attention_decode`` / ``attention_decode_fused``;
    ``stages`` is the depth of a block's ring of 64-key tiles (0: chosen from the size of the launch)."""
    import os
    width = (n_q_heads + 2 * n_kv_heads) * head_dim
    partial = dense = None
    nslices = slice_stride = dense_stride = 0
    if isinstance(source, SplitSum):
        partial = source.slices
        _need(partial.is_cuda and partial.dtype == torch.float32 and partial.dim() == 3 and partial.shape[2] == width
              and partial[0].is_contiguous(), "attention_decode_tma: bad split source")
        nslices, slice_stride = partial.shape[0], partial.stride(0)
    elif source is not None:
        dense = source
        _need(dense.is_cuda and dense.dtype == torch.bfloat16 and dense.dim() == 2 and dense.shape[1] == width
              and dense.stride(1) == 1, "attention_decode_tma: the product must be bf16 [rows, (Hq + 2 Hkv) D]")
        dense_stride = dense.stride(0)
    else:
        _need(q is not None and q.is_cuda and q.dtype == torch.bfloat16 and q.stride(1) == 1 and q.data_ptr() % 16 == 0
              and q.stride(0) % 8 == 0, "attention_decode_tma: q must be bf16 with 16-byte aligned rows")
    _cuda(out, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, k_pages, v_pages, scratch, counters, status,
          bias, inv_freq, prefetch)
    _need(decode_tma_supported(out.dtype, head_dim, k_pages.shape[2]) or os.environ.get("TESSWEAVE_DECODE_TMA") == "0",
          f"attention_decode_tma does not take head size {head_dim} with pages of {k_pages.shape[2]} keys in {out.dtype}")
    _need(out.dtype == k_pages.dtype == v_pages.dtype == torch.bfloat16, "attention_decode_tma: bfloat16 only")
    _need(n_q_heads % n_kv_heads == 0, "attention: query heads must be a multiple of key/value heads")
    _need(k_pages.is_contiguous() and v_pages.is_contiguous() and k_pages.shape[3] == head_dim
          and k_pages.shape[1] == n_kv_heads and v_pages.shape == k_pages.shape
          and k_pages.data_ptr() % 16 == 0 and v_pages.data_ptr() % 16 == 0,
          "attention: cache pages must be contiguous, 16-byte aligned [pages, kv_heads, page, head_dim]")
    _need(block_table.dtype == torch.int32 and block_table.is_contiguous(), "attention: bad block table")
    _need(out.stride(1) == 1 and out.stride(0) % 4 == 0 and out.data_ptr() % 8 == 0,
          "attention_decode_tma: output rows must be 8-byte aligned")
    _need(bias is None or (bias.dtype == torch.float32 and bias.numel() == width), "attention_decode_tma: bias must be fp32")
    _need(inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.numel() == head_dim // 2),
          "attention_decode_tma: inv_freq must be fp32 [D/2]")
    _need(1 <= nsplit <= DECODE_MAX_SPLITS, f"attention_decode_tma: 1 to {DECODE_MAX_SPLITS} slices, not {nsplit}")
    if nsplit > 1:
        _need(scratch is not None and scratch.dtype == torch.float32 and scratch.data_ptr() % 16 == 0
              and scratch.numel() >= n_seqs * n_q_heads * nsplit * (head_dim + 2), "attention_decode: scratch too small")
        _need(counters is not None and counters.dtype == torch.int32
              and counters.numel() >= n_seqs * n_kv_heads * ((n_q_heads // n_kv_heads + 7) // 8),
              "attention_decode: too few counters")
    stages = stages or int(os.environ.get("TESSWEAVE_DECODE_STAGES", "0"))
    code = _fn("attention_decode_tma", "tw_attn_decode_tma", {"TW_HEAD_DIM": head_dim})(
        _ptr(out), c_int(out.stride(0)), _ptr(q), c_int(q.stride(0) if q is not None else 0), _ptr(partial), c_int(nslices),
        ctypes.c_longlong(slice_stride), _ptr(dense), c_int(dense_stride), _ptr(bias), _ptr(inv_freq),
        c_int(1 if write_cache else 0), _ptr(seq_q_start), _ptr(seq_q_len), _ptr(seq_kv_len), _ptr(seq_slot),
        _ptr(block_table), c_int(block_table.shape[1]), _ptr(k_pages), _ptr(v_pages), c_int(n_seqs), c_int(n_q_heads),
        c_int(n_kv_heads), c_int(k_pages.shape[2]), c_int(k_pages.shape[0]), c_int(window), c_float(scale), c_int(nsplit),
        c_int(stages), c_int(1 if merge_in_scratch else 0), _ptr(scratch), _ptr(counters), _ptr(status), _ptr(prefetch),
        ctypes.c_longlong(prefetch.numel() * prefetch.element_size() if prefetch is not None else 0), _stream())
    _check(code, "attention_decode_tma")


def attention_prefill_tcgen05(out, q, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, k_pages, v_pages, n_seqs,
                              max_q_len, n_q_heads, n_kv_heads, head_dim, window, scale, skip_single, status) -> None:
    """The same as ``attention_prefill`` on the 5th-generation tensor cores (TMA, tcgen05.mma,
    accumulators in tensor memory), for the shapes ``tcgen05_attention_supported`` names."""
    _cuda(out, q, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, k_pages, v_pages, status)
    _attn_common_checks(out, q, block_table, k_pages, v_pages, n_q_heads, n_kv_heads, head_dim)
    _need(tcgen05_attention_supported(q.dtype, head_dim, k_pages.shape[2]),
          f"tcgen05 attention does not take head size {head_dim} with pages of {k_pages.shape[2]} keys")
    _need(q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0,
          "tcgen05 attention: rows of q and out must be 16-byte aligned")
    code = _fn("attention_tcgen05", "tw_attn_prefill_tc5", {"TW_HEAD_DIM": head_dim})(
        _ptr(out), c_int(out.stride(0)), _ptr(q), c_int(q.stride(0)), _ptr(seq_q_start), _ptr(seq_q_len),
        _ptr(seq_kv_len), _ptr(seq_slot), _ptr(block_table), c_int(block_table.shape[1]), _ptr(k_pages), _ptr(v_pages),
        c_int(n_seqs), c_int(max_q_len), c_int(n_q_heads), c_int(n_kv_heads), c_int(k_pages.shape[2]),
        c_int(k_pages.shape[0]), c_int(window), c_float(scale), c_int(1 if skip_single else 0), _ptr(status), _stream())
    _check(code, "attention_prefill_tcgen05")


def attention_prefill(out, q, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, k_pages, v_pages, n_seqs,
                      max_q_len, n_q_heads, n_kv_heads, head_dim, window, scale, skip_single, status) -> None:
    """Flash attention over the paged cache for the requests that bring several tokens."""
    _cuda(out, q, seq_q_start, seq_q_len, seq_kv_len, seq_slot, block_table, k_pages, v_pages, status)
    _attn_common_checks(out, q, block_table, k_pages, v_pages, n_q_heads, n_kv_heads, head_dim)
    code = _fn("attention_bf16", "tw_attn_prefill", {"TW_HEAD_DIM": head_dim})(
        _ptr(out), c_int(out.stride(0)), _ptr(q), c_int(q.stride(0)), _ptr(seq_q_start), _ptr(seq_q_len),
        _ptr(seq_kv_len), _ptr(seq_slot), _ptr(block_table), c_int(block_table.shape[1]), _ptr(k_pages), _ptr(v_pages),
        c_int(n_seqs), c_int(max_q_len), c_int(n_q_heads), c_int(n_kv_heads), c_int(k_pages.shape[2]),
        c_int(k_pages.shape[0]), c_int(window), c_float(scale), c_int(1 if skip_single else 0), _ptr(status), _stream())
    _check(code, "attention_prefill")


# ---------------------------------------------------------------------------
# matrix products with few rows
# ---------------------------------------------------------------------------
SMALL_M_LIMIT = 8          # rows up to which the weight-streaming kernel is used
_TARGET_WARPS = 2400       # warps in flight that keep the memory system busy


def small_m_supported(x: torch.Tensor, w: torch.Tensor, m: int) -> bool:
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and 0 < m <= SMALL_M_LIMIT
            and w.shape[1] % 8 == 0 and w.is_contiguous() and x.is_contiguous())


SMALL_M_ROWS_PER_BLOCK = 64      # weight rows of a block of csrc/gemm_smallm.cu (four warps of 16 rows)
SMALL_M_BLOCKS_PER_SM = 5        # how many of its blocks an SM holds


def small_m_split(n: int, k: int, max_slices: int = 12, sms: int | None = None) -> tuple[int, int]:
    """(slices, k per slice): enough slices that rows / 16 * slices warps fill the GPU, each
    slice a multiple of 32 wide and at least 256.  ``max_slices``: the most slices the consumer wants to add
    (the kernel then gives a row tile to two warps where that fills the GPU better).

    All blocks of such a launch are resident at once and share the memory bandwidth about equally, so the launch
    takes as long as the SM with the most blocks: among the slice counts near the one that fills the GPU, the one
    that leaves the SMs most evenly loaded is taken.  Measured on B200, whole decode steps of the 7B-sized model
    (3,584 rows in blocks of 64: 56 blocks per slice): 11 slices = 616 blocks, 4.2 per SM, 3.18 ms; 10 slices =
    560 blocks, 3.8 per SM, 3.13 ms; 13 slices 3.17; 9 slices 3.18; 8 slices (448 blocks, which the kernel doubles:
    6 per SM, two rounds) 3.30; at the 14B sizes (5,120 rows: 80 blocks per slice) 9 slices = 720 blocks 6.88 ms,
    8 slices = 640 blocks 6.93."""
    sms = sms or _SM_COUNT
    tiles = -(-n // 16)
    if tiles >= 1024:          # enough rows to fill the GPU without slices
        return 1, -(-k // 32) * 32
    want = max(1, min(12, max_slices, -(-_TARGET_WARPS // tiles)))
    best = None
    for wanted in range(min(12, max_slices, want + 1), max(0, want - 3), -1):
        kper = max(256, -(-(-(-k // wanted)) // 32) * 32)
        kper = min(kper, -(-k // 32) * 32)
        slices = -(-k // kper)
        blocks = -(-n // SMALL_M_ROWS_PER_BLOCK) * slices
        if blocks * 10 <= sms * 32 and kper >= 512:  # the kernel then gives every row tile to two warps: twice the blocks
            blocks = -(-n // (SMALL_M_ROWS_PER_BLOCK // 2)) * slices
        most = -(-blocks // sms)                     # blocks of the fullest SM
        even = blocks / (most * sms) if most <= SMALL_M_BLOCKS_PER_SM else 0.0
        # fewer slices than wanted only where that evens the load out by a tenth or more
        score = even - 0.03 * abs(want - wanted)
        if best is None or score > best[0]:
            best = (score, slices, kper)
    return best[1], best[2]


def gemm_small_m(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, m: int, kper: int | None = None,
                 silu_mul_pairs: bool = False, early_dependents: bool = False,
                 prefetch: torch.Tensor | None = None) -> None:
    """out[:m] = x[:m] @ w.T for m <= 64 rows.  ``out`` is bf16 or fp32 [>=m, n]; or, when the
    product is split over k (kper < k), fp32 slices [slices, m, n]; or, with ``silu_mul_pairs``
    (rows of w in groups of eight gates and their eight ups), bf16 [>=m, n / 2] = silu(gate) * up.
    ``early_dependents``: the kernel launched next may become resident while this one runs (it waits for
    the result itself); worth it when that kernel is small.  ``prefetch``: a contiguous, 16-byte aligned tensor
    that the kernel after this one streams; the blocks ask for it to be brought into L2 when their own stream ends."""
    _cuda(out, x, w)
    if prefetch is not None:
        _need(prefetch.is_cuda and prefetch.is_contiguous(), "gemm_small_m: the tensor to prefetch must be contiguous")
    n, k = w.shape
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and x.is_contiguous()
          and x.shape[1] == k and k % 8 == 0 and m <= 64, "gemm_small_m: bf16 operands, k a multiple of 8, m <= 64")
    kper = kper or -(-k // 32) * 32
    split = -(-k // kper)
    if silu_mul_pairs:
        _need(split == 1 and n % 16 == 0 and out.dtype == torch.bfloat16 and out.dim() == 2 and out.stride(1) == 1
              and out.shape[0] >= m and out.shape[1] == n // 2, "gemm_small_m: bad fused silu output")
        mode, stride = 3, out.stride(0)
    elif split > 1:
        _need(out.dtype == torch.float32 and out.dim() == 3 and out.shape[0] == split and out.shape[1] == m
              and out.shape[2] == n and out.is_contiguous(), "gemm_small_m: split output must be fp32 [slices, m, n]")
        mode, stride = 2, n
    else:
        _need(out.dim() == 2 and out.stride(1) == 1 and out.shape[0] >= m and out.shape[1] == n
              and out.dtype in (torch.bfloat16, torch.float32), "gemm_small_m: bad output")
        mode, stride = (0 if out.dtype == torch.bfloat16 else 1), out.stride(0)
    if early_dependents:
        mode |= 16          # the kernel after this one may become resident while this one runs
    code = _fn("gemm_smallm", "tw_gemm_smallm")(_ptr(w), _ptr(x), c_int(m), c_int(n), c_int(k), c_int(kper), _ptr(out),
                                                c_int(mode), c_int(stride), _ptr(prefetch),
                                                ctypes.c_longlong(prefetch.numel() * prefetch.element_size()
                                                                  if prefetch is not None else 0), _stream())
    _check(code, "gemm_small_m")


# ---------------------------------------------------------------------------
# matrix products of prompt steps on pairs of thread blocks
# ---------------------------------------------------------------------------
PAIR_MIN_M = 768           # rows from which the fused gate/up product may run on block pairs


def pair_tiles_efficiency(m: int, n: int, sms: int | None = None) -> float:
    """The share of the block pairs' time that is useful work: rows padded to tiles of 256, and the 256 x 256 tiles
    dealt to sms / 2 pairs in whole rounds."""
    pairs = max(1, (sms or _SM_COUNT) // 2)
    tiles_m, tiles_n = -(-m // 256), -(-n // 256)
    tiles = tiles_m * tiles_n
    return (m / (tiles_m * 256)) * (tiles / pairs) / -(-tiles // pairs)


def pair_product_preferred(x: torch.Tensor, w: torch.Tensor, m: int) -> bool:
    """Whether the gate/up product with the SiLU.mul epilogue runs on ``gemm_tcgen05_pair``.  Measured on B200
    against the library's product plus the separate SiLU.mul kernel: at 37,888 x 3,584 the pairs take 155.7 /
    200.5 / 280.4 / 387 us at 768 / 1,024 / 1,536 / 2,048 rows against 156.2 / 204.8 / 298.0 / 396, but 146.8
    against 124.0 at 544 rows (padded to 768) and 109.6 against 108.1 at 512; at 27,648 x 5,120 they lose where
    the tiles do not fill whole rounds of pairs (1,280 rows: 271.9 against 260.7).  So: from 768 rows, and only
    where padding and rounds leave at least 93 % of the pairs' time useful.  TESSWEAVE_PAIR_GEMM=0 keeps the library,
    =force takes the pairs for every shape beyond 64 rows."""
    import os
    choice = os.environ.get("TESSWEAVE_PAIR_GEMM", "1")
    if choice == "0":
        return False
    takes = (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.shape[0] % 16 == 0
             and w.shape[1] % 8 == 0 and x.is_contiguous() and w.is_contiguous())
    if choice == "force":          # every shape the kernel takes (tests run whole models through it this way)
        return takes and m > 64
    return takes and m >= PAIR_MIN_M and pair_tiles_efficiency(m, w.shape[0]) >= 0.93


def gemm_tcgen05_pair(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, m: int, status: torch.Tensor,
                      silu_mul_pairs: bool = False) -> None:
    """out[:m] = x[:m] @ w.T for many rows, on pairs of thread blocks (tcgen05.mma.cta_group::2,
    256 x 256 tiles).  ``out`` is bf16 or fp32 [>=m, n]; with ``silu_mul_pairs`` (rows of w in
    groups of eight gates and their eight ups) it is bf16 [>=m, n / 2] = silu(gate) * up."""
    _cuda(out, x, w, status)
    n, k = w.shape
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and x.is_contiguous()
          and x.shape[1] == k and k % 8 == 0, "gemm_tcgen05_pair: contiguous bf16 operands, k a multiple of 8")
    _need(x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0, "gemm_tcgen05_pair: operands must be 16-byte aligned")
    if silu_mul_pairs:
        _need(n % 16 == 0 and out.dtype == torch.bfloat16 and out.dim() == 2 and out.stride(1) == 1 and out.shape[0] >= m
              and out.shape[1] == n // 2 and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0,
              "gemm_tcgen05_pair: the SiLU.mul output must be bf16 [m, n / 2] with 16-byte aligned rows")
        mode = 3
    else:
        _need(out.dim() == 2 and out.stride(1) == 1 and out.shape[0] >= m and out.shape[1] == n
              and out.dtype in (torch.bfloat16, torch.float32), "gemm_tcgen05_pair: bad output")
        mode = 0 if out.dtype == torch.bfloat16 else 1
    code = _fn("gemm_tcgen05_pair", "tw_gemm_tcgen05_pair")(_ptr(x), _ptr(w), c_int(m), c_int(n), c_int(k), _ptr(out),
                                                            c_int(mode), c_int(out.stride(0)), _ptr(status), _stream())
    _check(code, "gemm_tcgen05_pair")


# ---------------------------------------------------------------------------
# matrix products of decode steps with more requests than the small-M kernel takes
# ---------------------------------------------------------------------------
STREAM_MIN_M, STREAM_MAX_M = 9, 128     # rows the persistent weight-streaming tcgen05 kernel takes
STREAM_MIN_WEIGHTS = 48_000_000         # elements of w from which it is the product path


def stream_product_preferred(x: torch.Tensor, w: torch.Tensor, m: int) -> bool:
    """Whether a product of ``m`` rows runs on ``gemm_tcgen05_stream`` (persistent, the weights as the 128-row
    operand): 9 to 64 rows and a large matrix.  Measured on B200 at 7B layer sizes, 16 / 64 rows: down 25.9 / 28.1
    us against the library's 28.9 / 31.1, gate/up with SiLU.mul 47.5 / 51.7 against 46.6 / 48.1 plus 2.5 / 3.5 for
    the separate SiLU.mul kernel, logits 171 / 181 against 179 / 183; the smaller q/k/v and o_proj products
    (8.8 / 10.7 against 8.6 / 8.9) stay with the library, whose split over k is reduced inside its kernel.
    TESSWEAVE_STREAM_GEMM=0 keeps the library everywhere; TESSWEAVE_STREAM_MAX_M and TESSWEAVE_STREAM_MIN_WEIGHTS
    move the bounds."""
    import os
    if os.environ.get("TESSWEAVE_STREAM_GEMM", "1") == "0":
        return False
    top = min(STREAM_MAX_M, int(os.environ.get("TESSWEAVE_STREAM_MAX_M", "64")))
    least = int(os.environ.get("TESSWEAVE_STREAM_MIN_WEIGHTS", str(STREAM_MIN_WEIGHTS)))
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and STREAM_MIN_M <= m <= top
            and w.numel() >= least and w.shape[1] % 8 == 0 and x.is_contiguous() and w.is_contiguous()
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


_stream_sms: list[int] = [0]


def _stream_sm_count() -> int:
    if not _stream_sms[0]:
        _stream_sms[0] = int(_fn("gemm_tcgen05_stream", "tw_gemm_tcgen05_stream_sm_count")())
    return _stream_sms[0]


def stream_whole_k_balanced(n: int, sms: int | None = None) -> bool:
    """Whether the 128-row tiles of a matrix of ``n`` rows, not split over k (the SiLU.mul epilogue needs whole
    sums), keep the persistent kernel's blocks evenly busy: 296 tiles on 148 SMs do (two each), 216 do not (68
    blocks get two, 80 one; the 14B gate/up product measured slower than the library that way)."""
    sms = sms or _stream_sm_count()
    tiles = -(-n // 128)
    return tiles / sms >= 0.85 * -(-tiles // sms)


def stream_split_gate_up_enabled() -> bool:
    """TESSWEAVE_STREAM_SPLIT_GATE_UP=1: a gate/up product whose row tiles alone do not balance (14B: 216 tiles)
    runs on the persistent kernel in slices over k that the SiLU.mul kernel adds.  Off by default: measured at 14B
    layer sizes a decode step is 1 % shorter with it at batch 12 and 24 and 2.5 % longer at batch 32, where the
    library's product is at its best."""
    import os
    return os.environ.get("TESSWEAVE_STREAM_SPLIT_GATE_UP", "0") == "1"


def stream_split(n: int, k: int, allow: bool = True, sms: int | None = None) -> tuple[int, int]:
    """(slices, k per slice) for the persistent kernel: its work items are (128-row tile of w, slice of k), dealt
    round robin to one block per SM.  The choice minimises the k-blocks of the busiest block, each item charged
    four more for its start and its result; up to 12 slices."""
    kbs = -(-k // 64)
    if not allow:
        return 1, kbs * 64
    sms = sms or _stream_sm_count()
    tiles = -(-n // 128)
    best = None
    for want in range(1, 13):
        per = -(-kbs // want)
        real = -(-kbs // per)
        cost = -(-tiles * real // sms) * (per + 4)
        if best is None or cost < best[0]:
            best = (cost, real, per * 64)
    return best[1], best[2]


def gemm_tcgen05_stream(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, m: int, status: torch.Tensor,
                        kper: int | None = None, silu_mul_pairs: bool = False, early_dependents: bool = False,
                        prefetch: torch.Tensor | None = None) -> None:
    """out[:m] = x[:m] @ w.T for up to 128 rows on the 5th-generation tensor cores, the weights streamed once by a
    persistent kernel.  ``out`` is bf16 or fp32 [>=m, n]; fp32 slices [slices, m, n] when ``kper`` (a multiple of
    64) is less than k; with ``silu_mul_pairs`` (rows of w in groups of eight gates and their eight ups) bf16
    [>=m, n / 2] = silu(gate) * up.  ``prefetch``: a contiguous, 16-byte aligned tensor that the kernel after
    this one streams; a block asks for its share of it to be brought into L2 once its own last copy is issued."""
    _cuda(out, x, w, status)
    if prefetch is not None:
        _need(prefetch.is_cuda and prefetch.is_contiguous(), "gemm_tcgen05_stream: the tensor to prefetch must be contiguous")
    n, k = w.shape
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.is_contiguous() and x.is_contiguous()
          and x.shape[1] == k and k % 8 == 0 and 0 < m <= STREAM_MAX_M and x.shape[0] >= m,
          "gemm_tcgen05_stream: contiguous bf16 operands, k a multiple of 8, up to 128 rows")
    _need(x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0, "gemm_tcgen05_stream: operands must be 16-byte aligned")
    kper = kper or -(-k // 64) * 64
    _need(kper % 64 == 0, "gemm_tcgen05_stream: k per slice must be a multiple of 64")
    split = -(-k // kper)
    if silu_mul_pairs:
        _need(split == 1 and n % 16 == 0 and out.dtype == torch.bfloat16 and out.dim() == 2 and out.stride(1) == 1
              and out.shape[0] >= m and out.shape[1] == n // 2, "gemm_tcgen05_stream: bad fused SiLU.mul output")
        mode, stride = 3, out.stride(0)
    elif split > 1:
        _need(out.dtype == torch.float32 and out.dim() == 3 and tuple(out.shape) == (split, m, n) and out.is_contiguous(),
              "gemm_tcgen05_stream: split output must be fp32 [slices, m, n]")
        mode, stride = 2, n
    else:
        _need(out.dim() == 2 and out.stride(1) == 1 and out.shape[0] >= m and out.shape[1] == n
              and out.dtype in (torch.bfloat16, torch.float32), "gemm_tcgen05_stream: bad output")
        mode, stride = (0 if out.dtype == torch.bfloat16 else 1), out.stride(0)
    if early_dependents:
        mode |= 16          # the kernel after this one may become resident while this one runs
    # the token rows the kernel reads: exactly m (rows beyond are filled with zeros by the copy engine)
    code = _fn("gemm_tcgen05_stream", "tw_gemm_tcgen05_stream")(_ptr(x), _ptr(w), c_int(m), c_int(n), c_int(k), c_int(kper),
                                                                _ptr(out), c_int(mode), c_int(stride), _ptr(status),
                                                                _ptr(prefetch), ctypes.c_longlong(
                                                                    prefetch.numel() * prefetch.element_size()
                                                                    if prefetch is not None else 0), _stream())
    _check(code, "gemm_tcgen05_stream")
