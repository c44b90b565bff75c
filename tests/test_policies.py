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
    assert ops.STREAM_MIN_M == ops.SMALL_M_LIMIT + 1


def test_split_policy_respects_the_consumers_limit():
    """A consumer that adds at most four slices gets at most four; the default stays at up to twelve."""
    from tessweave_engine_b200.csrc import ops
    slices, kper = ops.small_m_split(4608, 3584, max_slices=4)
    assert slices == 4 and kper % 32 == 0 and slices * kper >= 3584
    wide, _ = ops.small_m_split(4608, 3584)
    assert 4 < wide <= 12
    assert ops.small_m_split(152064, 3584, max_slices=4)[0] == 1       # enough rows: no slices at all


def test_timeline_groups_blocks_into_launches():
    """Blocks of two launches of one kernel in a row (told apart by their count), a second kernel overlapping
    the first, and the gap between launches."""
    import torch
    from tessweave_engine_b200.engine.timeline import group_launches, format_launches
    tag = lambda kernel, blocks: kernel | (blocks << 16)
    rows = []
    for b in range(3):                                   # kernel 5, 3 blocks: 1000..1400
        rows.append([tag(5, 3), b, 1000 + 10 * b, 1000 + 10 * b, 1300 + 50 * b])
    for b in range(2):                                   # kernel 3, 2 blocks, resident early, waits until 1400
        rows.append([tag(3, 2), b, 1200 + b, 1400, 1500 + b])
    for b in range(3):                                   # kernel 5 again, 3 blocks
        rows.append([tag(5, 3), b, 1600 + b, 1600 + b, 1900])
    entries = torch.tensor(rows, dtype=torch.int64)[torch.randperm(len(rows), generator=torch.Generator().manual_seed(0))]
    launches = group_launches(entries)
    assert [(l["kernel"], l["blocks"], l["seen"]) for l in launches] == [
        ("gemm_smallm", 3, 3), ("norm (cluster)", 2, 2), ("gemm_smallm", 3, 3)]
    assert launches[0]["start"] == 0.0 and abs(launches[0]["end"] - 0.4) < 1e-9 and abs(launches[0]["ramp"] - 0.02) < 1e-9
    assert launches[1]["gap"] < 0 and 0.199 <= launches[1]["waited"] <= 0.2            # launched while the first ran
    assert abs(launches[2]["gap"] - 0.099) < 1e-9                                      # after the later of the two ends
    assert "gemm_smallm" in format_launches(launches)
    assert group_launches(torch.zeros(0, 5, dtype=torch.int64)) == []


def test_stream_split_balances_items_over_the_blocks():
    """The persistent kernel's slices: none where the row tiles alone fill the GPU twice over, enough where a matrix
    has few rows, never more than twelve, k per slice a multiple of 64 that covers k."""
    from tessweave_engine_b200.csrc import ops
    assert ops.stream_split(37888, 3584, sms=148)[0] == 1          # 296 tiles: two items per block
    assert ops.stream_split(152064, 3584, sms=148)[0] == 1
    slices, kper = ops.stream_split(3584, 18944, sms=148)          # 28 tiles
    assert 4 <= slices <= 6 and kper % 64 == 0 and slices * kper >= 18944 and (slices - 1) * kper < 18944
    assert ops.stream_split(3584, 18944, allow=False, sms=148) == (1, 18944)
    for n, k in ((100, 64), (5120, 13824), (128, 100000)):
        slices, kper = ops.stream_split(n, k, sms=148)
        assert 1 <= slices <= 12 and kper % 64 == 0 and (slices - 1) * kper < k <= slices * kper


def test_fused_gate_up_needs_evenly_busy_blocks():
    from tessweave_engine_b200.csrc import ops
    assert ops.stream_whole_k_balanced(37888, sms=148)           # 296 tiles: two per block
    assert not ops.stream_whole_k_balanced(27648, sms=148)       # 216 tiles: 68 blocks with two, 80 with one
    assert ops.stream_whole_k_balanced(55296, sms=148)           # 432 tiles: 2.92 of 3


def test_decode_slices_leave_room_for_their_clusters():
    """Launches whose slices merge in clusters of five blocks and more stay under 3.5 blocks per SM: with more, some
    clusters start a wave late (batch 12 with 4 key/value heads took 11 slices = 528 blocks before, 10 now)."""
    from tessweave_engine_b200.csrc import ops
    room = 7 * ops._SM_COUNT // 2
    for batch in range(1, 65):
        for kv_heads, group, keys in ((4, 7, 4096), (8, 5, 1024), (2, 7, 16384)):
            n = ops.decode_splits(batch, kv_heads, group, keys)
            assert n >= 1
            if n > 4:
                assert n * batch * kv_heads * ((group + 7) // 8) <= room, (batch, kv_heads, group, keys, n)
    assert ops.decode_splits(12, 4, 7, 4096) == 10
    assert ops.decode_splits(8, 4, 7, 16384) <= 14 and ops.decode_splits(8, 4, 7, 32768) <= 14
    assert ops.decode_splits(44, 4, 7, 4096) == 3 and ops.decode_splits(48, 4, 7, 4096) == 2
    assert ops.decode_splits(8, 4, 7, 4096) == 13
    assert ops.decode_splits(16, 4, 7, 4096) == 8


def test_pair_product_only_where_its_tiles_fill_the_pairs():
    from tessweave_engine_b200.csrc import ops
    eff = lambda m, n: ops.pair_tiles_efficiency(m, n, sms=148)
    assert eff(2048, 37888) == 1.0 and eff(768, 37888) == 1.0
    assert eff(544, 37888) < 0.75                       # padded to 768 rows
    assert eff(1280, 27648) < 0.93 <= eff(1536, 27648)  # 540 tiles: 7.3 rounds of 74 pairs; 648 tiles: 8.76


def test_tma_decode_slices_fill_about_two_blocks_per_sm():
    """The slice count of the TMA decode attention: about 256 blocks for many requests, whole tiles of 64 keys per
    slice, no slice without keys, at most 128, and within the scratch buffer for any batch."""
    from tessweave_engine_b200.csrc import ops
    for batch in (1, 2, 3, 4, 6, 8, 12, 16, 24, 32, 48, 64, 200):
        for keys in (1, 63, 64, 65, 512, 4096, 16384, 100000):
            n = ops.decode_tma_splits(batch, 4, 7, keys)
            assert 1 <= n <= min(ops.DECODE_MAX_SPLITS, -(-keys // 64))
            assert batch * n <= max(batch, ops.DECODE_SCRATCH_UNITS)
            per = -(-(-(-keys // n)) // 64) * 64
            assert (n - 1) * per < keys                      # the last slice holds at least one key
            if batch >= 8 and keys >= 4096:
                assert n == 1 or batch * 4 * n <= 296        # never more blocks than two per SM, unless one per request is more
    assert ops.decode_tma_splits(8, 4, 7, 4096) == 8 and ops.decode_tma_splits(64, 4, 7, 4096) == 1
    assert ops.decode_tma_splits(8, 8, 5, 4096) == 4         # 14B sizes: twice the key/value heads, half the slices
    assert ops.decode_tma_supported(__import__("torch").bfloat16, 128, 16)


def test_small_decode_launches_become_resident_early(monkeypatch):
    """The q/k/v product lets the decode attention settle on the SMs while it runs only where that launch leaves
    most of the GPU free, or does not merge in clusters; at the benchmark's 7B sizes that is 1 to 3 requests."""
    monkeypatch.delenv("TESSWEAVE_DECODE_EARLY", raising=False)
    monkeypatch.delenv("TESSWEAVE_DECODE_SPLITS", raising=False)
    early = {}
    for batch in (1, 2, 3, 4, 8, 64):
        ns = ops.decode_tma_splits(batch, 4, 7, 4096)
        early[batch] = ops.decode_attention_resident_early(batch * 4 * ns, ns)
    assert early == {1: True, 2: True, 3: True, 4: False, 8: False, 64: False}
    ns = ops.decode_tma_splits(2, 4, 7, 16384)
    assert ns > ops.DECODE_TMA_CLUSTER_SLICES and ops.decode_attention_resident_early(2 * 4 * ns, ns)
    monkeypatch.setenv("TESSWEAVE_DECODE_EARLY", "0")
    assert not ops.decode_attention_resident_early(4, 1)
    monkeypatch.setenv("TESSWEAVE_DECODE_EARLY", "1")
    assert ops.decode_attention_resident_early(10_000, 2)


def test_split_products_load_the_sms_evenly():
    """All blocks of a split small-batch product are resident at once, so the launch is as slow as the fullest SM:
    3,584 rows (56 blocks of 64 rows per slice) take 10 slices (560 blocks, at most 4 on an SM), not the 11 that the
    count of warps alone asks for (616 blocks: 24 SMs would hold 5); 5,120 rows take 9 (720 blocks, 4.9 per SM)."""
    for n, k, slices in ((3584, 3584, 10), (3584, 18944, 10), (5120, 5120, 9), (5120, 13824, 9), (5120, 27648, 9)):
        got, kper = ops.small_m_split(n, k, sms=148)
        assert got == slices and kper % 32 == 0 and got * kper >= k > (got - 1) * kper
        blocks = -(-n // ops.SMALL_M_ROWS_PER_BLOCK) * got
        assert -(-blocks // 148) * 148 - blocks < 0.06 * blocks       # the fullest SM holds little more than its share
    assert ops.small_m_split(4608, 3584, max_slices=4, sms=148)[0] == 4
