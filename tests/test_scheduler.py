"""The scheduler's decisions, driven with a stand-in step function on the CPU (no GPU)."""
import pytest
import torch

from helpers import make_folder
import tessweave_engine_b200 as tw
from tessweave_engine_b200.cache import CapacityError
from tessweave_engine_b200.config import EngineConfig
from tessweave_engine_b200.engine.scheduler import Engine


class FakeRunner:
    """Records every step; 'samples' token (sum of the row's tokens + position) % vocab."""

    def __init__(self, vocab):
        self.vocab, self.steps, self.fail_next = vocab, [], False
        self.pending = []

    def stage_sampling(self, temperature, seed, counter):
        self.sampling = list(zip(temperature, seed, counter))

    def step(self, entries):
        if self.fail_next:
            raise RuntimeError("injected failure")
        self.steps.append([(e.slot, list(e.tokens), e.start, list(e.want)) for e in entries])
        self.pending = [(e.tokens[w] + e.start + w) % self.vocab for e in entries for w in e.want]
        return torch.zeros(len(self.pending), 1)

    def sample(self, logits, greedy_only=False):
        return list(self.pending)


@pytest.fixture
def model(tmp_path):
    return tw.load_model(make_folder(tmp_path, "A"), "float32", "cpu")


def engine_for(model, **kw):
    defaults = dict(block_size=4, kv_blocks=32, max_context=64, prefill_chunk=4, min_prefill_chunk=1, max_active=4)
    defaults.update(kw)
    runner = FakeRunner(model.spec.vocab_size)
    return Engine(model, EngineConfig(**defaults), runner=runner), runner


def drain(engine, limit=500):
    for _ in range(limit):
        if not engine.step():
            return
    raise AssertionError("the engine did not come to rest")


def test_one_mixed_step_decode_first_under_the_budget(model):
    e, runner = engine_for(model, prefill_chunk=6, max_step_tokens=8)
    a = e.submit([1, 2, 3], max_tokens=4, ignore_eos=True)
    drain_steps = 0
    e.step()                                            # a: whole prompt (3 <= 6)
    assert runner.steps[-1] == [(a.lease.slot, [1, 2, 3], 0, [2])]
    b = e.submit(list(range(10, 30)), max_tokens=2, ignore_eos=True)
    c = e.submit(list(range(40, 50)), max_tokens=2, ignore_eos=True)
    e.step()
    rows = runner.steps[-1]
    assert rows[0][1] == [a.output[0]] and rows[0][2] == 3 and rows[0][3] == [0]      # decode row first
    assert [len(r[1]) for r in rows] == [1, 6, 1]       # budget 8: 1 decode + chunk 6 + 1 left for the next prompt
    assert rows[1][3] == [] and rows[2][3] == []        # unfinished prompts want no logits
    e.step()
    rows = runner.steps[-1]
    assert len(rows[0][1]) == 1 and sum(len(r[1]) for r in rows) <= 8
    drain(e)
    assert len(a.output) == 4 and len(b.output) == 2 and len(c.output) == 2
    assert e.stats()["free_blocks"] + e.stats()["cached_prefix_blocks"] == 32
    e.close()
    assert e.stats()["free_blocks"] == 32


def test_positions_and_tokens_are_consecutive(model):
    e, runner = engine_for(model, prefill_chunk=5)
    r = e.submit(list(range(100, 117)), max_tokens=3, ignore_eos=True)
    drain(e)
    seen = []
    for step in runner.steps:
        for slot, tokens, start, want in step:
            assert start == len(seen)
            seen.extend(tokens)
    assert seen == (r.prompt + r.output)[:len(seen)] and len(seen) == 17 + 2     # the last token is never fed


def test_validation_at_submit(model):
    e, _ = engine_for(model)
    for bad in ([], [256], [-1], [1.5]):
        with pytest.raises(ValueError):
            e.submit(bad)
    with pytest.raises(ValueError):
        e.submit([1] * 60, max_tokens=5)                 # beyond max_context
    with pytest.raises(ValueError):
        e.submit([1], max_tokens=0)
    with pytest.raises(ValueError):
        e.submit([1], temperature=2.5)
    small, _ = engine_for(model, kv_blocks=2)
    with pytest.raises(ValueError, match="exceeds the KV pool"):
        small.submit([1] * 8, max_tokens=4)


def test_admission_waits_for_pages_and_recovers(model):
    e, _ = engine_for(model, kv_blocks=4, prefix_cache=False)
    a = e.submit([1, 2, 3, 4, 5], max_tokens=6, ignore_eos=True)       # 3 pages
    b = e.submit([6, 7, 8, 9, 10], max_tokens=6, ignore_eos=True)      # 3 pages: must wait
    c = e.submit([11], max_tokens=1, ignore_eos=True)                  # would fit, but FIFO: waits behind b
    e.step()
    assert a.status == "active" and b.status == "waiting" and c.status == "waiting"
    drain(e)
    assert [x.status for x in (a, b, c)] == ["length"] * 3
    assert len(a.output) == 6 and len(b.output) == 6
    e.cache.check_invariants()
    assert e.stats()["free_blocks"] == 4


def test_queue_limit_and_cancel(model):
    e, _ = engine_for(model, max_queue=2, max_active=1)
    a = e.submit([1, 2, 3], max_tokens=20, ignore_eos=True)
    e.step()
    b = e.submit([4, 5], max_tokens=2)
    c = e.submit([6, 7], max_tokens=2)
    with pytest.raises(CapacityError):
        e.submit([8], max_tokens=2)
    e.cancel(b.id)
    e.cancel(a.id)
    assert a.status == "cancelled" and b.status == "cancelled"
    assert a.events.get_nowait()["type"] == "token"
    drain(e)
    assert c.status == "length"
    e.close()
    e.cache.check_invariants()
    assert e.stats()["free_blocks"] == 32 and e.stats()["cancelled"] == 2


def test_eos_stops_unless_ignored(model):
    e, runner = engine_for(model)
    eos = model.spec.eos_token_ids[0]
    prompt = [eos - 1]                                    # fake sampler: (token + position) % vocab
    r = e.submit(prompt, max_tokens=10)
    drain(e)
    assert r.output == [eos - 1, eos] and r.status == "stop"
    r2 = e.submit(prompt, max_tokens=5, ignore_eos=True)
    drain(e)
    assert r2.status == "length" and len(r2.output) == 5


def test_failed_step_ends_every_request_and_frees_pages(model):
    e, runner = engine_for(model)
    a = e.submit([1, 2, 3, 4, 5, 6], max_tokens=4)
    b = e.submit([7, 8], max_tokens=4)
    e.step()
    runner.fail_next = True
    with pytest.raises(RuntimeError, match="injected"):
        e.step()
    assert a.status == "error" and b.status == "error" and e.fatal
    done = [ev for ev in list(a.events.queue) if ev["type"] == "done"]
    assert done and done[0]["finish_reason"] == "error" and "injected" in done[0]["error"]
    e.cache.check_invariants()
    assert e.stats()["free_blocks"] + e.stats()["cached_prefix_blocks"] == 32 and not e.cache.leases
    with pytest.raises(RuntimeError):
        e.submit([1])


def test_slow_consumer_gets_an_error(model):
    e, _ = engine_for(model, max_context=1024, kv_blocks=256)
    r = e.submit([1, 2], max_tokens=400, ignore_eos=True)
    drain(e, limit=1000)
    assert r.status == "error"                            # nobody drained the bounded event queue
    assert list(r.events.queue)[-1]["type"] == "done"
    assert e.stats()["failed"] == 1 and not e.cache.leases


def test_prefix_hits_are_counted_like_the_reference(model):
    e, runner = engine_for(model, prefill_chunk=16)
    prompt = [1, 2, 3, 4, 5, 6, 7, 8, 9]
    a = e.submit(prompt, max_tokens=2, ignore_eos=True)
    drain(e)
    b = e.submit(prompt, max_tokens=2, ignore_eos=True)
    e.step()
    assert b.cached == 8                                  # tests/test_engine.py:113-126
    assert runner.steps[-1][0][1] == [9] and runner.steps[-1][0][2] == 8      # one prompt token is run
    c = e.submit([1, 2, 3, 4, 99, 98, 97], max_tokens=2, ignore_eos=True)
    e.step()
    assert c.cached == 4
    d = e.submit(prompt, max_tokens=2, namespace="other", ignore_eos=True)
    e.step()
    assert d.cached == 0
    drain(e)
    e.close()
    assert e.stats()["free_blocks"] == 32


def test_worker_thread_delivers_events(model):
    e, _ = engine_for(model)
    r = e.submit([3, 4, 5], max_tokens=3, ignore_eos=True)
    e.start()
    events = []
    while True:
        events.append(r.events.get(timeout=10))
        if events[-1]["type"] == "done":
            break
    e.close()
    assert [ev["type"] for ev in events] == ["token"] * 3 + ["done"]
    assert events[-1]["usage"] == {"prompt_tokens": 3, "completion_tokens": 3, "total_tokens": 6}


class ResolvingRunner(FakeRunner):
    def __init__(self, vocab):
        super().__init__(vocab)
        self.queue = []          # launched, unfinished steps in order
        self.results = {}        # launch number -> tokens
        self.count = 0
        self.max_in_flight = 0

    def launch(self, entries, temperature, seed, counter, device_refs=False):
        assert device_refs or all(t >= 0 for e in entries for t in e.tokens)
        if self.fail_next:
            raise RuntimeError("injected failure")
        self.count += 1
        self.queue.append((self.count, entries))
        self.max_in_flight = max(self.max_in_flight, len(self.queue))
        return self.count

    def _run(self, number, entries):
        prev = self.results.get(number - 1, [])
        rows, out = [], []
        for e in entries:
            toks = [prev[-(t + 1)] if t < 0 else t for t in e.tokens]
            rows.append((e.slot, toks, e.start, list(e.want)))
            out += [(toks[w] + e.start + w) % self.vocab for w in e.want]
        self.steps.append(rows)
        self.results[number] = out

    def finish(self, pending):
        while self.queue and self.queue[0][0] <= pending:
            number, entries = self.queue.pop(0)
            self._run(number, entries)
        return self.results[pending]


def lookahead_engine(model, lookahead, **kw):
    defaults = dict(block_size=4, kv_blocks=64, max_context=64, prefill_chunk=4, min_prefill_chunk=1, max_active=4,
                    lookahead=lookahead)
    defaults.update(kw)
    runner = ResolvingRunner(model.spec.vocab_size)
    return Engine(model, EngineConfig(**defaults), runner=runner), runner


def test_lookahead_gives_the_same_tokens_and_keeps_two_steps_in_flight(model):
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9], [20, 21, 22], [30, 31, 32, 33, 34, 35, 36, 37, 38, 39, 40]]
    outs = {}
    for look in (False, True):
        e, runner = lookahead_engine(model, look)
        reqs = [e.submit(p, max_tokens=5 + i, ignore_eos=True) for i, p in enumerate(prompts)]
        drain(e)
        outs[look] = [r.output for r in reqs]
        assert runner.max_in_flight == (2 if look else 1)
        e.cache.check_invariants()
        e.close()
        assert e.stats()["free_blocks"] == 64 and not e.cache.leases
    assert outs[True] == outs[False]
    assert all(len(o) == 5 + i for i, o in enumerate(outs[True]))


def test_lookahead_request_that_stops_keeps_its_pages_until_the_running_step_is_done(model):
    e, runner = lookahead_engine(model, True, prefix_cache=False)
    eos = model.spec.eos_token_ids[0]
    a = e.submit([eos - 1], max_tokens=10)              # second token is the stop token
    b = e.submit([5, 6], max_tokens=6, ignore_eos=True)
    e.step()            # prompts (and the step after them is launched)
    e.step()            # a's second token arrives: a stops while the step after is running
    assert a.status == "stop" and a.output == [eos - 1, eos]
    assert e.inflight is not None and len(e.inflight.deferred) == 1       # a's pages are still held
    assert len(e.cache.leases) == 2
    e.step()
    assert len(e.cache.leases) == 1                                        # given back once that step ended
    drain(e)
    assert len(b.output) == 6
    e.close()
    e.cache.check_invariants()
    assert e.stats()["free_blocks"] == 64


def test_lookahead_cancel_and_failure_leave_nothing_behind(model):
    e, runner = lookahead_engine(model, True)
    a = e.submit([1, 2, 3], max_tokens=20, ignore_eos=True)
    b = e.submit([4, 5, 6], max_tokens=20, ignore_eos=True)
    e.step(); e.step()
    e.cancel(a.id)
    assert a.status == "cancelled" and e.inflight.deferred
    e.step()
    runner.fail_next = True
    with pytest.raises(RuntimeError, match="injected"):
        e.step()
    assert b.status == "error" and e.inflight is None
    e.cache.check_invariants()
    assert not e.cache.leases and e.stats()["free_blocks"] + e.stats()["cached_prefix_blocks"] == 64


def test_small_budget_leaves_nobody_out(model):
    """A token budget below the number of active requests: the decode pass starts at a moving place, so
    every request advances within a few steps, and a prompt still being read always gets a token."""
    e, runner = engine_for(model, max_active=4, max_step_tokens=2, prefill_chunk=4)
    reqs = [e.submit([10 + i, 20 + i], max_tokens=6, ignore_eos=True) for i in range(4)]
    for _ in range(8):
        e.step()                                        # prompts go in two tokens at a time
    before = [len(r.output) for r in reqs]
    late = e.submit([1, 2, 3, 4, 5], max_tokens=2, ignore_eos=True)    # waits for a slot; nothing to check yet
    for _ in range(4):
        e.step()
    after = [len(r.output) for r in reqs]
    assert all(b > a for a, b in zip(before, after) if a < 6), (before, after)
    drain(e)
    assert all(len(r.output) == 6 for r in reqs) and len(late.output) == 2
    # decode rows never crowd out a prompt: with three decoding requests and budget 2, the reader still moves
    e2, runner2 = engine_for(model, max_active=4, max_step_tokens=2, prefill_chunk=4)
    for i in range(3):
        e2.submit([5 + i], max_tokens=30, ignore_eos=True)
    for _ in range(4):
        e2.step()
    reader = e2.submit(list(range(40, 52)), max_tokens=1, ignore_eos=True)
    for _ in range(14):
        e2.step()
    assert reader.computed >= 12 or reader.status == "length"
    e.close(); e2.close()


def test_failed_launch_of_the_step_ahead_waits_for_the_running_step(model):
    """The step launched ahead fails (here: the runner refuses it) while the step before it is still running:
    that step is waited for before any page is given back."""
    e, runner = lookahead_engine(model, True)
    a = e.submit([1, 2, 3], max_tokens=20, ignore_eos=True)
    e.step()
    assert len(runner.queue) == 1                       # one step under way, launched ahead
    launches = runner.count

    def failing_launch(entries, temperature, seed, counter, device_refs=False):
        assert runner.queue, "the step before is still running when the next launch fails"
        raise RuntimeError("injected launch failure")
    runner.launch = failing_launch
    with pytest.raises(RuntimeError, match="injected launch failure"):
        e.step()
    assert runner.count == launches and not runner.queue      # the running step was finished (waited for), not abandoned
    assert a.status == "error" and not e.cache.leases and not e.flights
    e.cache.check_invariants()
