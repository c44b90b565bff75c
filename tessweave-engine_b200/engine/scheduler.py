"""The scheduler: continuous batching with decode-first chunked prefill.

Requests wait in a FIFO, are admitted while request slots and pages allow, and
then take part in every step: a request whose prompt is in the cache brings one
token (the one sampled last), a request still reading its prompt brings the next
portion, cut to the step's token budget.  All of them run as ONE mixed batch
through the step function; the reference runs the decode batch and one prompt
portion as two forwards per turn (flow_engine/engine.py:243-269).  Names,
options, counters, events and finish reasons follow flow_engine/engine.py.

When pages run out: a request is only admitted if the pages for its whole
declared budget (prompt + max_tokens) can be promised, after evicting least
recently used prefix entries; otherwise it waits at the head of the queue and
nobody behind it is tried (engine.py:96-113).  An admitted request therefore
never runs out of pages mid-way; nothing is preempted, swapped or recomputed.
A request larger than the whole pool is refused at submit (engine.py:81-82).
"""
from __future__ import annotations

import math
import queue
import threading
import time
import uuid
from collections import deque
from dataclasses import dataclass, field

import torch

from ..cache.manager import CacheManager, CapacityError, Lease
from ..config.engine_config import EngineConfig
from ..models.model import Model
from .runner import ModelRunner, StepEntry
from .trace import Trace


@dataclass
class Request:
    """Per-request record (flow_engine/engine.py:15-32)."""
    id: str
    prompt: list[int]
    max_tokens: int
    temperature: float
    seed: int
    namespace: str
    ignore_eos: bool = False
    tokens: list[int] = field(default_factory=list)     # prompt + generated
    output: list[int] = field(default_factory=list)
    lease: Lease | None = None
    computed: int = 0                                   # tokens whose keys/values are in the cache
    cached: int = 0                                     # of these, taken from shared prefix pages
    status: str = "waiting"
    created: float = field(default_factory=time.perf_counter)
    first_token: float | None = None
    events: queue.Queue = field(default_factory=lambda: queue.Queue(maxsize=256))


@dataclass
class Flight:
    """A step that has been handed to the GPU."""
    plan: list                                   # (request, tokens it brings)
    rows: dict                                   # request id -> tokens it brings
    sampling: list                               # requests whose last row is sampled, in row order
    sampled_index: dict                          # request id -> its place among the sampled rows
    started: float
    pending: object = None                       # the runner's handle, or None when the step ran synchronously
    tokens: list = field(default_factory=list)   # chosen tokens of a synchronous step
    deferred: list = field(default_factory=list)  # leases of requests that ended while this step ran


class Engine:
    """One model worker owns every change to the cache; callers never run kernels."""

    def __init__(self, model: Model, config: EngineConfig | None = None, trace: Trace | None = None, runner=None):
        self.model = model
        self.config = config or EngineConfig()
        cfg = self.config
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
        self.waiting: deque[Request] = deque()
        self.active: list[Request] = []
        self.requests: dict[str, Request] = {}
        self.lock = threading.RLock()
        self.wake = threading.Event()
        self.running = False
        self.thread = None
        self.fatal = None
        self.inflight: Flight | None = None
        # run one step ahead: the next step is launched before the current one's tokens are on the host
        self.lookahead = bool(cfg.lookahead and hasattr(self.runner, "launch"))
        self.prefill_cursor = 0
        self.chunk = cfg.prefill_chunk
        self.prefill_ms_per_token = None
        self.counters = {"submitted": 0, "finished": 0, "cancelled": 0, "failed": 0,
                         "generated_tokens": 0, "prefill_tokens": 0, "steps": 0}

    # ------------------------------------------------------------------ submit / admit
    def submit(self, tokens, max_tokens=128, temperature=0.0, seed=0, namespace="local", ignore_eos=False) -> Request:
        """Queue a request (flow_engine/engine.py:71-94).  Raises ValueError for a request that
        can never run and CapacityError when the queue is full."""
        with self.lock:
            if self.fatal:
                raise RuntimeError(f"Engine failed: {self.fatal}")
            vocab = self.model.spec.vocab_size
            if not tokens or any(type(t) is not int or t < 0 or t >= vocab for t in tokens):
                raise ValueError("Prompt must contain valid token IDs")
            if max_tokens < 1 or len(tokens) + max_tokens > self.config.max_context:
                raise ValueError("prompt_tokens + max_tokens exceeds configured context")
            if not math.isfinite(temperature) or not 0 <= temperature <= 2:
                raise ValueError("temperature must be finite and between 0 and 2")
            if max(self.cache.pages_needed(len(tokens) + max_tokens, self.config.prefill_chunk),
                   default=0) > self.cache.num_pages:
                raise ValueError("This request alone exceeds the KV pool; increase --kv-blocks or reduce tokens")
            if len(self.waiting) >= self.config.max_queue:
                raise CapacityError("Waiting queue is full")
            r = Request(uuid.uuid4().hex, list(tokens), max_tokens, float(temperature), int(seed), namespace, ignore_eos)
            r.tokens = list(tokens)
            self.requests[r.id] = r
            self.waiting.append(r)
            self.counters["submitted"] += 1
            self.trace.emit("submit", request_id=r.id, prompt_tokens=len(tokens), max_tokens=max_tokens,
                            temperature=temperature, seed=seed)
            self.wake.set()
            return r

    def _admit(self) -> None:
        """FIFO admission with the whole budget promised (engine.py:96-113)."""
        while self.waiting and len(self.active) < self.config.max_active:
            r = self.waiting[0]
            try:
                lease = self.cache.admit(r.prompt, reserve_tokens=len(r.prompt) + r.max_tokens,
                                         namespace=r.namespace, step_tokens=self.config.prefill_chunk)
            except CapacityError:
                break       # head of the line waits; a large job is not starved by small ones
            self.waiting.popleft()
            r.lease = lease
            r.computed = r.cached = lease.cached_tokens
            r.status = "active"
            self.active.append(r)
            self.trace.emit("admit", request_id=r.id, reused_tokens=r.cached,
                            reserved_blocks=math.ceil((len(r.prompt) + r.max_tokens) / self.config.block_size),
                            shared_blocks=r.cached // self.config.block_size, **self.cache.stats())

    # ------------------------------------------------------------------ events / finishing
    def _emit(self, r: Request, event: dict) -> bool:
        try:
            r.events.put_nowait(event)
            return True
        except queue.Full:
            self._finish(r, "error", "Consumer too slow; bounded output queue exhausted")
            return False

    def _finish(self, r: Request, reason: str, error: str | None = None) -> None:
        """Take the request out of every list, give its pages back, deliver the terminal event
        (engine.py:123-146).  Full blocks were already made shareable as they were computed."""
        if r.id not in self.requests:
            return
        if r in self.active:
            self.active.remove(r)
        elif r in self.waiting:
            self.waiting.remove(r)
        if r.lease is not None:
            if self.inflight is not None and r.id in self.inflight.rows:
                self.inflight.deferred.append(r.lease)    # a running step still writes this request's pages
            else:
                self.cache.release(r.lease)
            r.lease = None
        r.status = reason
        del self.requests[r.id]
        self.counters[{"cancelled": "cancelled", "error": "failed"}.get(reason, "finished")] += 1
        end = {"type": "done", "finish_reason": reason, "error": error,
               "usage": {"prompt_tokens": len(r.prompt), "completion_tokens": len(r.output),
                         "total_tokens": len(r.prompt) + len(r.output)},
               "cached_tokens": r.cached, "elapsed_s": time.perf_counter() - r.created}
        if r.events.full():          # a terminal event is always delivered
            while not r.events.empty():
                r.events.get_nowait()
        r.events.put_nowait(end)
        self.trace.emit("finish", request_id=r.id, **{k: v for k, v in end.items() if k != "type"})

    def cancel(self, request_id: str) -> None:
        with self.lock:
            r = self.requests.get(request_id)
            if r:
                self._finish(r, "cancelled")

    def _commit(self, r: Request, token: int) -> bool:
        """Append a sampled token; finish on EOS or on the length budget (engine.py:160-175)."""
        r.tokens.append(token)
        r.output.append(token)
        self.counters["generated_tokens"] += 1
        if r.first_token is None:
            r.first_token = time.perf_counter()
            self.trace.emit("first_token", request_id=r.id, ttft_ms=(r.first_token - r.created) * 1000)
        if not self._emit(r, {"type": "token", "token_id": token}):
            return False
        if not r.ignore_eos and token in self.model.spec.eos_token_ids:
            self._finish(r, "stop")
            return False
        if len(r.output) >= r.max_tokens:
            self._finish(r, "length")
            return False
        return True

    # ------------------------------------------------------------------ one turn
    def plan(self, flight: "Flight | None" = None) -> list[tuple[Request, int]]:
        """Which requests bring how many tokens to the next step: every decoding request one
        token first, then prompt portions in round-robin order while the token budget lasts.

        With ``flight`` (a step that is still running) the plan is made for the step after it:
        positions count from where that step will have left each request, a request whose token
        that step is choosing brings it by reference (it is still on the device), and a request
        that the step will finish by its length budget brings nothing."""
        ahead = flight.rows if flight else {}
        budget = self.config.step_token_budget
        plan: list[tuple[Request, int]] = []
        for r in self.active:
            done = r.computed + ahead.get(r.id, 0)
            if done >= len(r.prompt) and budget > 0:
                if flight and r.id in flight.sampled_index and len(r.output) + 1 >= r.max_tokens:
                    continue
                plan.append((r, 1))
                budget -= 1
        prefill = [r for r in self.active if r.computed + ahead.get(r.id, 0) < len(r.prompt)]
        if prefill:
            start = self.prefill_cursor % len(prefill)
            self.prefill_cursor += 1
            for r in prefill[start:] + prefill[:start]:
                count = min(self.chunk, len(r.prompt) - r.computed - ahead.get(r.id, 0), budget)
                if count <= 0:
                    break
                plan.append((r, count))
                budget -= count
        return plan

    def step(self) -> bool:
        """Admit, run one mixed step, sample, commit.  False when nothing is left to do."""
        with self.lock:
            try:
                return self._step()
            except Exception as exc:
                self._fail(exc)
                raise

    def _launch(self, plan: list[tuple[Request, int]], after: "Flight | None") -> "Flight":
        """Hand one step to the runner without waiting for it."""
        ahead = after.rows if after else {}
        entries, sampling, temps, seeds, counters = [], [], [], [], []
        for r, count in plan:
            start = r.computed + ahead.get(r.id, 0)
            self.cache.ensure(r.lease, start + count)
            if start >= len(r.tokens):
                # the token this row feeds is being chosen by the step in flight: name it by its place there
                tokens = [-(after.sampled_index[r.id] + 1)]
                drawn = len(r.output) + 1
            else:
                tokens = r.tokens[start:start + count]
                drawn = len(r.output)
            finishes_prompt = start + count >= len(r.prompt)
            entries.append(StepEntry(r.lease.slot, tokens, start, [count - 1] if finishes_prompt else []))
            if finishes_prompt:
                sampling.append(r)
                temps.append(r.temperature); seeds.append(r.seed); counters.append(drawn)
        flight = Flight(plan=plan, rows={r.id: c for r, c in plan}, sampling=sampling,
                        sampled_index={r.id: i for i, r in enumerate(sampling)}, started=time.perf_counter())
        if hasattr(self.runner, "launch"):
            flight.pending = self.runner.launch(entries, temps, seeds, counters)
        else:       # a stand-in runner without asynchronous steps
            self.runner.stage_sampling(temps, seeds, counters)
            logits = self.runner.step(entries)
            flight.tokens = self.runner.sample(logits, greedy_only=all(t == 0 for t in temps)) if sampling else []
        return flight

    def _complete(self, flight: "Flight") -> None:
        """Wait for a step, move its requests on, commit its tokens, give back what was held for it."""
        try:
            chosen = flight.tokens if flight.pending is None else self.runner.finish(flight.pending)
        finally:
            for lease in flight.deferred:
                self.cache.release(lease)
            flight.deferred = []
        elapsed = (time.perf_counter() - flight.started) * 1000
        self.counters["steps"] += 1
        prefill_tokens = 0
        for r, count in flight.plan:
            if r.id not in self.requests:
                continue                     # finished or cancelled while the step ran; its row is dropped
            if r.computed < len(r.prompt):
                prefill_tokens += count
            r.computed += count
            self.cache.advance(r.lease, r.tokens, r.computed)
        self.counters["prefill_tokens"] += prefill_tokens
        for r, token in zip(flight.sampling, chosen):
            if r.id in self.requests:
                self._commit(r, int(token))
        if prefill_tokens and self.config.adaptive_chunk:
            self._adapt_chunk(elapsed, prefill_tokens, sum(1 for _, c in flight.plan if c == 1))
        self.trace.emit("step", phase="mixed", request_ids=[r.id for r, _ in flight.plan], batch=len(flight.plan),
                        tokens=sum(c for _, c in flight.plan), prefill_tokens=prefill_tokens, elapsed_ms=elapsed,
                        prefill_chunk=self.chunk, **self.cache.stats())

    @torch.inference_mode()
    def _step(self) -> bool:
        self._admit()
        if self.inflight is None:
            if not self.active:
                return False
            self.inflight = self._launch(self.plan(), None)
        current, self.inflight = self.inflight, None
        if self.lookahead and self.active:
            ahead = self.plan(current)
            if ahead:
                # the step after `current` starts on the device before `current`'s tokens are on the host
                self.inflight = self._launch(ahead, current)
        self._complete(current)
        return True

    def _drain(self) -> None:
        """Wait for a step that is still running; its results are dropped."""
        flight, self.inflight = self.inflight, None
        if flight is not None:
            try:
                if flight.pending is not None:
                    self.runner.finish(flight.pending)
            finally:
                for lease in flight.deferred:
                    self.cache.release(lease)
                flight.deferred = []

    def _adapt_chunk(self, elapsed_ms: float, prefill_tokens: int, decode_rows: int) -> None:
        """The reference's feedback controller (engine.py:261-268): an EMA of milliseconds per
        prompt token steers the next portion towards ``target_step_ms``."""
        sample = elapsed_ms / max(1, prefill_tokens + decode_rows)
        self.prefill_ms_per_token = sample if self.prefill_ms_per_token is None else \
            .8 * self.prefill_ms_per_token + .2 * sample
        budget = max(1.0, self.config.target_step_ms - decode_rows * self.prefill_ms_per_token)
        estimate = int(budget / max(.001, self.prefill_ms_per_token))
        self.chunk = max(self.config.min_prefill_chunk, min(self.config.prefill_chunk, estimate))

    def _fail(self, exc: Exception) -> None:
        """A failed step ends every request with an error and gives all pages back (engine.py:283-289)."""
        self.fatal = f"{type(exc).__name__}: {exc}"
        self.trace.emit("fatal", error=self.fatal)
        try:
            self._drain()
        except Exception:       # noqa: BLE001  (the first failure is the one reported)
            pass
        for r in list(self.requests.values()):
            self._finish(r, "error", self.fatal)
        self.running = False

    # ------------------------------------------------------------------ worker thread
    def start(self) -> None:
        if self.running:
            return
        self.running = True
        self.thread = threading.Thread(target=self._loop, name="tessweave-model-worker", daemon=True)
        self.thread.start()

    def _loop(self) -> None:
        while self.running:
            try:
                if not self.step():
                    self.wake.wait(.05)
                    self.wake.clear()
            except Exception:
                self.running = False     # step() has already failed every request

    def close(self) -> None:
        self.running = False
        self.wake.set()
        if self.thread:
            self.thread.join()           # never free storage while kernels are in flight
            self.thread = None
        with self.lock:
            self._drain()
            for r in list(self.requests.values()):
                self._finish(r, "cancelled")
            self.cache.clear_prefixes()
        self.trace.close()

    def stats(self) -> dict:
        with self.lock:
            return {**self.counters, **self.cache.stats(), "active": len(self.active), "waiting": len(self.waiting),
                    "prefill_chunk": self.chunk, "ready": not self.fatal, "fatal": self.fatal,
                    "device": str(self.device), "dtype": str(self.model.runtime.dtype).replace("torch.", "")}

    # ------------------------------------------------------------------ convenience
    def run_until_done(self, limit: int = 1_000_000) -> None:
        """Step until nothing is left to do, acting as the consumer of every request's events
        (the bounded queues would otherwise end long generations with "Consumer too slow");
        tokens stay available in ``request.output``."""
        for _ in range(limit):
            busy = self.step()
            with self.lock:
                for r in list(self.requests.values()):
                    while not r.events.empty():
                        try:
                            r.events.get_nowait()
                        except queue.Empty:
                            break
            if not busy:
                return
        raise RuntimeError("the engine did not come to rest")
