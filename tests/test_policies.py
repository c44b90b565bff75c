"""Host-side choices that need no GPU: how decode attention cuts a request's keys into slices, how a product
is split over k, which batch sizes a runner captures."""
import pytest

from tessweave_engine_b200.csrc import ops


@pytest.mark.parametrize("n_seqs", [1, 2, 7, 8, 16, 33, 64, 200])
@pytest.mark.parametrize("kv_heads,group", [(4, 7), (8, 5), (1, 3), (2, 16)])
@pytest.mark.parametrize("max_kv", [1, 63, 64, 65, 1000, 4096, 5000, 16384, 131072])
def test_decode_splits_cover_the_keys_without_an_empty_slice(n_seqs, kv_heads, group, max_kv):
    ns = ops.decode_splits(n_seqs, kv_heads, group, max_kv)
    assert 1 <= ns <= 128
    assert n_seqs * ns <= max(ops.DECODE_SCRATCH_UNITS, n_seqs)          # the scratch buffer holds every slice
    per = -(-(-(-max_kv // ns)) // 64) * 64                             # what the kernel computes: keys per slice
    assert per * ns >= max_kv                                           # all keys are covered
    assert per * (ns - 1) < max_kv                                      # and the last slice has at least one


@pytest.mark.parametrize("n,k", [(4608, 3584), (3584, 3584), (37888, 3584), (3584, 18944), (152064, 3584), (16, 8), (100, 200)])
def test_small_m_split_covers_k(n, k):
    slices, kper = ops.small_m_split(n, k)
    assert slices >= 1 and kper % 32 == 0 and kper >= 32
    assert slices * kper >= k and (slices - 1) * kper < k


def test_products_route_by_rows():
    assert ops.SMALL_M_LIMIT == 8 and ops.PAIR_MIN_M >= 256
    assert ops.TCGEN05_MIN_M == ops.SMALL_M_LIMIT + 1
