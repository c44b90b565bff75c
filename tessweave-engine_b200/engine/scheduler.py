"""The scheduler: continuous batching with decode-first chunked prefill.

Requests wait in a FIFO, are admitted while request slots and pages allow, and then take part
in every step: a request whose prompt is in the cache brings one token (the one chosen last), a
request still reading its prompt brings the next portion, cut to the step's token budget.  All of
them run as ONE mixed batch through the step function; the reference runs the decode batch and
one prompt portion as two forwards per turn (flow_engine/engine.py:243-269).  The public names
(``submit, step, cancel, start, close, stats``), options, counters, events and finish reasons are
the reference's (flow_engine/engine.py:40-69); the request records and their bookkeeping live in
``requests.py``.

The engine works as a pipeline of *flights*.  A flight is one step that has been handed to the GPU:
which request brought how many tokens, whose last row is being sampled, and which pages must not
be given back before it has finished.  Up to two flights are under way: while the older one runs,
the next is planned and launched from what the older one *will* have done (its rows count as
computed; a token it is still choosing is named by its place among the chosen tokens and read on
the device).  ``step()`` completes the oldest flight.

When pages run out: a request is only admitted if the pages for its whole declared budget (prompt
+ max_tokens) can be promised, after evicting least recently used prefix entries; otherwise it
waits at the head of the queue and nobody behind it is tried (engine.py:96-113).  An admitted
request therefore never runs out of pages mid-way; nothing is preempted, swapped or recomputed.
A request larger than the whole pool is refused at submit (engine.py:81-82).
"""
from __future__ import annotations

import math
import threading
import time
import uuid
from collections import deque
from dataclasses import dataclass, field

import torch

from ..cache.manager import CacheManager, CapacityError
from ..config.engine_config import EngineConfig
from ..models.model import Model
from .requests import SLOW_CONSUMER, Request, RequestBook
from .runner import ModelRunner, StepEntry
from .trace import Trace

__all__ = ["Engine", "Request", "Flight", "plan_step"]


@dataclass
class Flight:
    """A step that has been handed to the GPU."""
    plan: list                                    # (request, tokens it brings)
    rows: dict                                    # request id -> tokens it brings
    sampling: list                                # requests whose last row is sampled, in row order
    sampled_index: dict                           # request id -> its place among the sampled rows
    started: float
    pending: object = None                        # the runner's handle, or None when the step ran synchronously
    tokens: list = field(default_factory=list)    # chosen tokens of a synchronous step
    deferred: list = field(default_factory=list)  # leases of requests that ended while this step ran


def plan_step(active: list[Request], done_ahead: dict, sampling_ahead: dict, budget: int, chunk: int,
              decode_cursor: int, prefill_cursor: int) -> list[tuple[Request, int]]:
    """Which requests bring how many tokens to the next step.

    ``done_ahead[id]`` tokens of a request are being computed by a step that is still running and
    count as done; a request in ``sampling_ahead`` gets a token from that step, which it brings by
    reference.  Order: single decode tokens first, then prompt portions of at most ``chunk`` tokens
    while ``budget`` lasts.  Both passes start at a cursor that moves on every step, so that under a
    budget smaller than the number of requests nobody is left out for good; and while a request is
    still reading its prompt, the decode pass leaves one token of the budget for it.
    """
    def done(r):
        return r.computed + done_ahead.get(r.id, 0)

    decoding = [r for r in active if done(r) >= len(r.prompt)
                and not (r.id in sampling_ahead and len(r.output) + 1 >= r.max_tokens)]   # that token is its last
    reading = [r for r in active if done(r) < len(r.prompt)]
    plan: list[tuple[Request, int]] = []
    room = budget - (1 if reading and budget > 1 else 0)
    if len(decoding) > room:
        first = decode_cursor % len(decoding)
        decoding = (decoding[first:] + decoding[:first])[:max(room, 0)]
    for r in decoding:
        plan.append((r, 1))
    budget -= len(decoding)
    if reading:
        first = prefill_cursor % len(reading)
        for r in reading[first:] + reading[:first]:
            count = min(chunk, len(r.prompt) - done(r), budget)
            if count <= 0:
                break
            plan.append((r, count))
            budget -= count
    return plan


class Engine:
    """One model worker owns every change to the cache; callers never run kernels."""

    def __init__(self, model: Model, config: EngineConfig | None = None, trace: Trace | None = None, runner=None):
        self.model = model
        self.config = cfg = config or EngineConfig()
        if cfg.max_context > model.spec.max_position_embeddings:
            raise ValueError("Requested context exceeds model configuration")
        self.device = model.runtime.device
        self.cache = CacheManager(model.cache_needs(), cfg.block_size, cfg.kv_blocks, cfg.max_active, cfg.max_context,
                                  model.runtime.dtype, self.device, cfg.prefix_cache)
        # ``runner`` lets a test drive the scheduler's decisions with a stand-in step function
        self.runner = runner if runner is not None else ModelRunner(
            model, self.cache, max_step_tokens=max(cfg.step_token_budget, cfg.max_active),
            max_step_seqs=cfg.max_active, max_logit_rows=cfg.max_active, cuda_graphs=cfg.cuda_graphs)
        self.trace = trace or Trace()
        self.book = RequestBook(self.trace, cfg.max_queue, model.spec.eos_token_ids)
        self.lock = threading.RLock()
        self.wake = threading.Event()
        self.running = False
        self.thread = None
        self.fatal = None
        self.flights: deque[Flight] = deque()      # launched and not yet completed, oldest first
        # run one step ahead: the next step is launched before the current one's tokens are on the host
        self.lookahead = bool(cfg.lookahead and hasattr(self.runner, "launch"))
        # a windowed group holds the pages of its window plus those of every step under way
        self.tokens_under_way = cfg.prefill_chunk * (2 if self.lookahead else 1)
        self.decode_cursor = 0
        self.prefill_cursor = 0
        self.chunk = cfg.prefill_chunk
        self.prefill_ms_per_token = None

    # the book's lists and counters under the names callers know
    waiting = property(lambda self: self.book.waiting)
    active = property(lambda self: self.book.active)
    requests = property(lambda self: self.book.by_id)
    counters = property(lambda self: self.book.counters)

    @property
    def inflight(self) -> Flight | None:
        """The youngest step under way (after ``step()`` returns: the one launched ahead), if any."""
        return self.flights[-1] if self.flights else None

    # ------------------------------------------------------------------ arrival
    def submit(self, tokens, max_tokens=128, temperature=0.0, seed=0, namespace="local", ignore_eos=False) -> Request:
        """Queue a request.  Raises ValueError for a request that can never run and CapacityError when
        the queue is full (the checks and their messages: flow_engine/engine.py:71-94)."""
        with self.lock:
            if self.fatal:
                raise RuntimeError(f"Engine failed: {self.fatal}")
            self._validate(tokens, max_tokens, temperature)
            request = Request(uuid.uuid4().hex, list(tokens), max_tokens, float(temperature), int(seed), namespace,
                              ignore_eos, tokens=list(tokens))
            self.book.enqueue(request)
            self.wake.set()
            return request

    def _validate(self, tokens, max_tokens, temperature) -> None:
        vocab = self.model.spec.vocab_size
        if not tokens or not all(type(t) is int and 0 <= t < vocab for t in tokens):
            raise ValueError("Prompt must contain valid token IDs")
        total = len(tokens) + max_tokens
        if max_tokens < 1 or total > self.config.max_context:
            raise ValueError("prompt_tokens + max_tokens exceeds configured context")
        if not (math.isfinite(temperature) and 0 <= temperature <= 2):
            raise ValueError("temperature must be finite and between 0 and 2")
        if any(pages > self.cache.num_pages for pages in self.cache.pages_needed(total, self.tokens_under_way)):
            raise ValueError("This request alone exceeds the KV pool; increase --kv-blocks or reduce tokens")

    def _admit(self) -> None:
        """First come, first served, the whole budget promised; if the head of the queue cannot get its
        pages, nobody behind it is tried, so a large request is not starved by small ones."""
        book, cfg = self.book, self.config
        while book.waiting and len(book.active) < cfg.max_active:
            request = book.waiting[0]
            budget = len(request.prompt) + request.max_tokens
            try:
                lease = self.cache.admit(request.prompt, reserve_tokens=budget, namespace=request.namespace,
                                         step_tokens=self.tokens_under_way)
            except CapacityError:
                return
            book.activate(request, lease, reserved_blocks=math.ceil(budget / cfg.block_size),
                          shared_blocks=lease.cached_tokens // cfg.block_size, **self.cache.stats())

    # ------------------------------------------------------------------ departure
    def _finish(self, request: Request, reason: str, error: str | None = None) -> None:
        """End a request.  Its pages go back at once unless a step under way still writes them; then they
        go back when that step has finished (never free storage that kernels in flight use)."""
        lease = self.book.retire(request, reason, error)
        if lease is None:
            return
        for flight in reversed(self.flights):
            if request.id in flight.rows:
                flight.deferred.append(lease)
                return
        self.cache.release(lease)

    def cancel(self, request_id: str) -> None:
        with self.lock:
            request = self.book.by_id.get(request_id)
            if request is not None:
                self._finish(request, "cancelled")

    def _release_deferred(self, flight: Flight) -> None:
        leases, flight.deferred = flight.deferred, []
        for lease in leases:
            self.cache.release(lease)

    # ------------------------------------------------------------------ one turn
    def plan(self, flight: Flight | None = None) -> list[tuple[Request, int]]:
        """The plan of the next step; with ``flight`` (a step still running), of the step after it."""
        plan = plan_step(self.book.active, flight.rows if flight else {}, flight.sampled_index if flight else {},
                         self.config.step_token_budget, self.chunk, self.decode_cursor, self.prefill_cursor)
        self.decode_cursor += 1
        self.prefill_cursor += 1
        return plan

    def step(self) -> bool:
        """Admit, keep the pipeline of steps full, complete the oldest step: sample, commit, finish.
        False when nothing is left to do."""
        with self.lock:
            try:
                return self._step()
            except Exception as exc:
                self._fail(exc)
                raise

    @torch.inference_mode()
    def _step(self) -> bool:
        self._admit()
        if not self.flights:
            if not self.book.active:
                return False
            self._launch(self.plan(), None)
        if self.lookahead and len(self.flights) == 1 and self.book.active:
            ahead = self.plan(self.flights[0])
            if ahead:
                # the step after the running one starts on the device before the running one's tokens are on the host
                self._launch(ahead, self.flights[0])
        self._complete(self.flights[0])
        return True

    def _launch(self, plan: list[tuple[Request, int]], after: Flight | None) -> Flight:
        """Hand one step to the runner without waiting for it."""
        ahead = after.rows if after else {}
        entries, sampling, temps, seeds, draws = [], [], [], [], []
        for request, count in plan:
            start = request.computed + ahead.get(request.id, 0)
            self.cache.ensure(request.lease, start + count)
            if start >= len(request.tokens):
                # the token this row feeds is being chosen by the step before: name it by its place there
                tokens = [-(after.sampled_index[request.id] + 1)]
                drawn = len(request.output) + 1
            else:
                tokens = request.tokens[start:start + count]
                drawn = len(request.output)
            ends_prompt = start + count >= len(request.prompt)
            entries.append(StepEntry(request.lease.slot, tokens, start, [count - 1] if ends_prompt else []))
            if ends_prompt:
                sampling.append(request)
                temps.append(request.temperature)
                seeds.append(request.seed)
                draws.append(drawn)
        flight = Flight(plan=plan, rows={r.id: c for r, c in plan}, sampling=sampling,
                        sampled_index={r.id: i for i, r in enumerate(sampling)}, started=time.perf_counter())
        if hasattr(self.runner, "launch"):
            flight.pending = self.runner.launch(entries, temps, seeds, draws, device_refs=after is not None)
        else:       # a stand-in runner without asynchronous steps
            self.runner.stage_sampling(temps, seeds, draws)
            logits = self.runner.step(entries)
            flight.tokens = self.runner.sample(logits, greedy_only=not any(temps)) if sampling else []
        self.flights.append(flight)
        return flight

    def _complete(self, flight: Flight) -> None:
        """Wait for the oldest step, move its requests on, commit its tokens, give back what was held for it."""
        assert self.flights and self.flights[0] is flight
        try:
            chosen = flight.tokens if flight.pending is None else self.runner.finish(flight.pending)
        finally:
            self.flights.popleft()
            self._release_deferred(flight)
        elapsed = (time.perf_counter() - flight.started) * 1000
        book = self.book
        book.counters["steps"] += 1
        prompt_tokens = decode_rows = 0
        for request, count in flight.plan:
            if not book.alive(request):
                continue                     # ended while the step ran; its rows are dropped
            if request.in_prompt:
                prompt_tokens += count
            else:
                decode_rows += 1
            request.computed += count
            self.cache.advance(request.lease, request.tokens, request.computed)
        book.counters["prefill_tokens"] += prompt_tokens
        for request, token in zip(flight.sampling, chosen):
            if book.alive(request):
                ending = book.add_token(request, int(token))
                if ending is not None:
                    self._finish(request, ending, SLOW_CONSUMER if ending == "error" else None)
        if prompt_tokens and self.config.adaptive_chunk:
            self._adapt_chunk(elapsed, prompt_tokens, decode_rows)
        self.trace.emit("step", phase="mixed", request_ids=[r.id for r, _ in flight.plan], batch=len(flight.plan),
                        tokens=sum(c for _, c in flight.plan), prefill_tokens=prompt_tokens, elapsed_ms=elapsed,
                        prefill_chunk=self.chunk, **self.cache.stats())

    def _drain(self) -> None:
        """Wait for every step that is still running; their results are dropped."""
        first_error = None
        while self.flights:
            flight = self.flights.popleft()
            try:
                if flight.pending is not None:
                    self.runner.finish(flight.pending)
            except Exception as exc:       # noqa: BLE001  (every flight is waited for; the first failure is reported)
                first_error = first_error or exc
            finally:
                self._release_deferred(flight)
        if first_error is not None:
            raise first_error

    def _adapt_chunk(self, elapsed_ms: float, prompt_tokens: int, decode_rows: int) -> None:
        """The reference's feedback controller (engine.py:261-268): a moving average of milliseconds per
        token steers the next portion towards ``target_step_ms``, within [min_prefill_chunk, prefill_chunk]."""
        cfg = self.config
        per_token = elapsed_ms / max(1, prompt_tokens + decode_rows)
        if self.prefill_ms_per_token is not None:
            per_token = 0.8 * self.prefill_ms_per_token + 0.2 * per_token
        self.prefill_ms_per_token = per_token
        left_for_prompts = max(1.0, cfg.target_step_ms - decode_rows * per_token)
        self.chunk = min(cfg.prefill_chunk, max(cfg.min_prefill_chunk, int(left_for_prompts / max(per_token, 1e-3))))

    def _fail(self, exc: Exception) -> None:
        """A failed step ends every request with an error and gives all pages back (engine.py:283-289):
        after every step under way has been waited for."""
        self.fatal = f"{type(exc).__name__}: {exc}"
        self.trace.emit("fatal", error=self.fatal)
        try:
            self._drain()
        except Exception:       # noqa: BLE001  (the first failure is the one reported)
            pass
        for request in list(self.book.by_id.values()):
            self._finish(request, "error", self.fatal)
        self.running = False

    # ------------------------------------------------------------------ worker thread
    def start(self) -> None:
        """Run ``step()`` on a thread of its own until ``close()``; consumers read the requests' events."""
        if self.running:
            return
        self.running = True
        self.thread = threading.Thread(target=self._work, name="tessweave-model-worker", daemon=True)
        self.thread.start()

    def _work(self) -> None:
        while self.running:
            try:
                busy = self.step()
            except Exception:   # noqa: BLE001  (step() has already ended every request with the error)
                self.running = False
                return
            if not busy:
                self.wake.wait(0.05)
                self.wake.clear()

    def close(self) -> None:
        self.running = False
        self.wake.set()
        if self.thread is not None:
            self.thread.join()           # the worker is between steps before anything is given back
            self.thread = None
        with self.lock:
            try:
                self._drain()
            finally:
                for request in list(self.book.by_id.values()):
                    self._finish(request, "cancelled")
                self.cache.clear_prefixes()
        self.trace.close()

    def stats(self) -> dict:
        with self.lock:
            book = self.book
            return {**book.counters, **self.cache.stats(), "active": len(book.active), "waiting": len(book.waiting),
                    "prefill_chunk": self.chunk, "ready": not self.fatal, "fatal": self.fatal,
                    "device": str(self.device), "dtype": str(self.model.runtime.dtype).replace("torch.", "")}

    # ------------------------------------------------------------------ convenience
    def run_until_done(self, limit: int = 1_000_000) -> None:
        """Step until nothing is left to do, acting as the consumer of every request's events (the
        bounded queues would otherwise end long generations with "Consumer too slow"); tokens stay
        available in ``request.output``."""
        for _ in range(limit):
            busy = self.step()
            with self.lock:
                self.book.drain_events()
            if not busy:
                return
        raise RuntimeError("the engine did not come to rest")
