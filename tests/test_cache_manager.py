"""The cache manager on the host: no page is lost, held twice or freed twice (no GPU)."""
import random

import pytest
import torch

from tessweave_engine_b200.cache import CacheManager, CapacityError
from tessweave_engine_b200.parts.base import FixedState, PagedKV

FULL = PagedKV(2, 16)
WINDOW = PagedKV(2, 16, window=20)


def manager(needs=None, pages=8, page=4, requests=4, context=64, prefix=True):
    needs = needs or [(FULL, None), (FULL, None)]
    return CacheManager(needs, page, pages, requests, context, torch.float32, "cpu", prefix_cache=prefix)


def free(m, gi=0):
    return len(m.groups[gi].free)


def test_groups_follow_needs():
    m = manager([(FULL, None), (WINDOW, None), (FULL, None), (None, 0), (FixedState(6), None)])
    assert len(m.groups) == 2 and m.groups[0].k.shape[0] == 2 and m.groups[1].k.shape[0] == 1
    assert m.groups[0].k.shape[1:] == (8, 2, 4, 16)
    assert m.view(3).k_pages.data_ptr() == m.view(0).k_pages.data_ptr()       # entry 3 reads entry 0's cache
    assert m.view(2).k_pages.data_ptr() != m.view(0).k_pages.data_ptr()
    assert m.view(4).state.shape == (4, 6)
    assert not m.prefix_cache                                                  # windows and state cannot share by hash


def test_shared_prefix_counts_and_partial_tail():
    m = manager()
    prompt = list(range(1, 10))                       # 9 tokens, page 4: two full blocks
    a = m.admit(prompt, reserve_tokens=12)
    assert a.cached_tokens == 0
    m.ensure(a, 9)
    m.advance(a, prompt, 9)
    m.check_invariants()
    b = m.admit(prompt, reserve_tokens=12)            # same prompt: both full blocks hit (cache.py:67-78)
    assert b.cached_tokens == 8 and b.tables[0][:2] == a.tables[0][:2]
    c = m.admit(prompt[:4] + [99, 98, 97, 96, 95], reserve_tokens=12)
    assert c.cached_tokens == 4                       # diverging tail: one block (test_engine.py:128-137)
    d = m.admit(prompt[:8], reserve_tokens=12)
    assert d.cached_tokens == 4                       # the last prompt token must run: hit stops before it
    for lease in (a, b, c, d):
        m.release(lease)
    m.check_invariants()
    assert free(m) == 8 - len(m.prefixes)
    m.clear_prefixes()
    assert free(m) == 8 and m.groups[0].promised == 0
    m.check_invariants()


def test_namespace_isolates():
    m = manager()
    p = list(range(9))
    a = m.admit(p, reserve_tokens=9, namespace="x")
    m.ensure(a, 9); m.advance(a, p, 9)
    assert m.admit(p, reserve_tokens=9, namespace="y").cached_tokens == 0
    assert m.admit(p, reserve_tokens=9, namespace="x").cached_tokens == 8


def test_eviction_never_frees_a_page_in_use():
    m = manager(pages=4, requests=3)
    p = list(range(9))
    a = m.admit(p, reserve_tokens=12)                 # 3 pages
    m.ensure(a, 9); m.advance(a, p, 9)
    m.release(a)                                      # 2 cached prefix pages stay, 2 pages free
    assert free(m) == 2 and len(m.prefixes) == 2
    b = m.admit(p, reserve_tokens=12)                 # hits both, needs 1 more
    assert b.cached_tokens == 8
    c = m.admit([50, 51, 52], reserve_tokens=4)       # 1 page: fits
    with pytest.raises(CapacityError):
        m.admit([60, 61, 62, 63, 64], reserve_tokens=8)   # would need eviction of pages b still holds
    m.check_invariants()
    assert b.tables[0][:2] == [p_ for p_ in b.tables[0][:2]] and all(m.groups[0].refs[x] >= 1 for x in b.tables[0][:2])
    m.release(b); m.release(c)
    d = m.admit([60, 61, 62, 63, 64] * 3, reserve_tokens=16)     # now the index entries are evicted
    m.ensure(d, 15)
    assert m.evictions >= 1
    m.check_invariants()


def test_admission_is_all_or_nothing_and_recovers():
    m = manager(pages=4, prefix=False)
    a = m.admit(None, reserve_tokens=12)
    with pytest.raises(CapacityError):
        m.admit(None, reserve_tokens=12)              # 3 + 3 > 4 (test_engine.py:160-170)
    m.check_invariants()
    assert len(m.leases) == 1 and m.groups[0].promised == 3
    m.ensure(a, 12)
    assert m.groups[0].promised == 0 and free(m) == 1
    m.release(a)
    b = m.admit(None, reserve_tokens=12)
    m.ensure(b, 12)
    m.check_invariants()


def test_unreserved_growth_runs_out_cleanly():
    m = manager(pages=3, prefix=False)
    a, b = m.admit(None), m.admit(None)
    m.ensure(a, 8)
    m.ensure(b, 4)
    with pytest.raises(CapacityError):
        m.ensure(b, 8)
    m.check_invariants()
    m.release(a)
    m.ensure(b, 8)
    m.check_invariants()


def test_double_release_is_an_error():
    m = manager()
    a = m.admit(None, reserve_tokens=4)
    m.ensure(a, 4)
    m.release(a)
    with pytest.raises(RuntimeError):
        m.release(a)
    with pytest.raises(RuntimeError):
        m._release_page(0, 0)


def test_window_group_gives_pages_back_and_reuses_them():
    m = manager([(WINDOW, None), (FULL, None)], pages=40, page=4, context=160, prefix=False)
    lease = m.admit(None, reserve_tokens=120, step_tokens=8)
    assert lease.promised[0] == (20 + 8 + 3) // 4 + 1 and lease.promised[1] == 30
    held = 0
    for step in range(15):
        held += 8
        m.ensure(lease, held)
        m.advance(lease, None, held)
        m.check_invariants()
        live = [p for p in lease.tables[0] if p >= 0]
        assert len(live) <= lease.promised[0] + len(live) and len(live) <= 8
        # every key the next token may see still has its page
        lo = max(0, held - 20 + 1)
        assert all(lease.tables[0][b] >= 0 for b in range(lo // 4, (held - 1) // 4 + 1))
        assert all(p >= 0 for p in lease.tables[1])
    assert lease.first_live_block[0] > 0 and lease.tables[0][0] == -1
    table = m.groups[0].host_table[lease.slot]
    assert int(table[0]) == -1 and int(table[(held - 1) // 4]) >= 0
    m.release(lease)
    m.check_invariants()
    assert free(m, 0) == 40 and free(m, 1) == 40


def test_state_slot_is_zeroed_at_admission():
    m = manager([(FixedState(5), None)], prefix=False)
    a = m.admit(None)
    m.state[0][a.slot] += 3
    slot = a.slot
    m.release(a)
    b = m.admit(None)
    assert b.slot == slot and float(m.state[0][slot].abs().sum()) == 0


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_invariant(seed):
    rng = random.Random(seed)
    window = seed % 2 == 1
    needs = [(WINDOW if window else FULL, None), (FULL, None)]
    m = manager(needs, pages=24, page=4, requests=5, context=96, prefix=not window)
    live = []
    prompts = [[rng.randrange(6) for _ in range(rng.randrange(1, 30))] for _ in range(8)]
    for _ in range(400):
        action = rng.random()
        if action < 0.3 and len(live) < 5:
            prompt = rng.choice(prompts)
            total = len(prompt) + rng.randrange(1, 20)
            try:
                lease = m.admit(prompt, reserve_tokens=total, step_tokens=8)
                live.append([lease, prompt + [rng.randrange(6) for _ in range(total - len(prompt))], lease.cached_tokens])
            except CapacityError:
                pass
        elif action < 0.8 and live:
            item = rng.choice(live)
            lease, tokens, done = item
            n = min(rng.randrange(1, 9), len(tokens) - done)
            if n > 0:
                m.ensure(lease, done + n)
                item[2] = done + n
                m.advance(lease, tokens, item[2])
        elif live:
            lease, _, _ = live.pop(rng.randrange(len(live)))
            m.release(lease)
        m.check_invariants()
    for lease, _, _ in live:
        m.release(lease)
    m.clear_prefixes()
    m.check_invariants()
    assert all(len(g.free) == g.num_pages and g.promised == 0 for g in m.groups)
    assert len(m.free_slots) == 5


def test_a_step_may_only_write_pages_its_request_holds_alone():
    """Shared pages are immutable: a write into a page with a second holder, or into a block without
    a page, is refused before the step runs (flow_engine/cache.py:3-5)."""
    m = manager()
    prompt = list(range(1, 10))
    a = m.admit(prompt, reserve_tokens=12)
    m.ensure(a, 9)
    m.check_writable(a.slot, 0, 9)                    # private pages: fine
    m.advance(a, prompt, 9)                           # blocks 0 and 1 are now in the prefix index too
    m.check_writable(a.slot, 8, 9)                    # the partial tail stays private
    with pytest.raises(RuntimeError, match="shared pages are immutable"):
        m.check_writable(a.slot, 7, 9)                # position 7 lies in a published block
    b = m.admit(prompt, reserve_tokens=12)            # hits both full blocks; computes from position 8
    m.ensure(b, 9)
    m.check_writable(b.slot, b.cached_tokens, 9)
    with pytest.raises(RuntimeError, match="shared pages are immutable"):
        m.check_writable(b.slot, 0, 9)
    with pytest.raises(RuntimeError, match="has no page"):
        m.check_writable(b.slot, 8, 13)               # block 3 was never ensured
    with pytest.raises(RuntimeError, match="holds no lease"):
        m.check_writable(3, 0, 1)
    m.release(a); m.release(b); m.clear_prefixes()
    m.check_invariants()


def test_windowed_group_with_two_steps_under_way():
    """With the next step launched before the current one has been accounted for, a windowed request holds
    the pages of its window plus those of BOTH steps: the promise made at admission covers them, so a pool
    that is promised to the last page never runs dry in the middle of a request."""
    needs = [(WINDOW, None)]                                       # window 20, pages of 4
    chunk = 8
    m = CacheManager(needs, 4, 12, 1, 256, torch.float32, "cpu", prefix_cache=False)
    need = m.pages_needed(200, 2 * chunk)[0]
    assert need == -(-(20 + 2 * chunk) // 4) + 1
    lease = m.admit(None, reserve_tokens=200, step_tokens=2 * chunk)
    assert m.groups[0].promised == need
    m.groups[0].promised += len(m.groups[0].free) - need           # everything else is promised to someone else
    done = 0
    m.ensure(lease, chunk)                                         # step A is launched
    for _ in range(20):
        m.ensure(lease, done + 2 * chunk)                          # step B is launched while A runs
        done += chunk
        m.advance(lease, None, done)                               # A is accounted for
        assert sum(p >= 0 for p in lease.tables[0]) <= need
    m.groups[0].promised -= len(m.groups[0].free) - lease.promised[0]
    m.release(lease)
    m.check_invariants()
