"""Requests and the book that keeps them.

A ``Request`` is what ``Engine.submit`` hands back: the caller reads ``output``, ``status`` and the
``events`` queue.  The ``RequestBook`` owns the three places a request can be (waiting, active,
gone), the engine's counters, and the one way a request ends: a terminal ``done`` event that is
always delivered, whatever the consumer did with the events before it.  The scheduler decides
*when* something happens to a request; the book records *that* it happened.

Field names, event shapes, counters, finish reasons and messages are those of the reference's
engine (flow_engine/engine.py:15-32 record, :67-69 counters, :115-146 events and terminal event,
:160-175 stop conditions), because callers written against it read exactly these.
"""
from __future__ import annotations

import queue
import time
from collections import deque
from dataclasses import dataclass, field

from ..cache.manager import CapacityError, Lease
from .trace import Trace

EVENT_QUEUE_SIZE = 256
SLOW_CONSUMER = "Consumer too slow; bounded output queue exhausted"


@dataclass
class Request:
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
    status: str = "waiting"                             # waiting, active, then the finish reason
    created: float = field(default_factory=time.perf_counter)
    first_token: float | None = None
    events: queue.Queue = field(default_factory=lambda: queue.Queue(maxsize=EVENT_QUEUE_SIZE))

    @property
    def in_prompt(self) -> bool:
        return self.computed < len(self.prompt)

    def usage(self) -> dict:
        return {"prompt_tokens": len(self.prompt), "completion_tokens": len(self.output),
                "total_tokens": len(self.prompt) + len(self.output)}


class RequestBook:
    def __init__(self, trace: Trace, max_queue: int, eos_token_ids):
        self.trace = trace
        self.max_queue = max_queue
        self.eos = frozenset(eos_token_ids)
        self.waiting: deque[Request] = deque()
        self.active: list[Request] = []
        self.by_id: dict[str, Request] = {}
        self.counters = dict.fromkeys(
            ("submitted", "finished", "cancelled", "failed", "generated_tokens", "prefill_tokens", "steps"), 0)

    # ---- arrival ------------------------------------------------------------------------
    def enqueue(self, request: Request) -> None:
        if len(self.waiting) >= self.max_queue:
            raise CapacityError("Waiting queue is full")
        self.by_id[request.id] = request
        self.waiting.append(request)
        self.counters["submitted"] += 1
        self.trace.emit("submit", request_id=request.id, prompt_tokens=len(request.prompt),
                        max_tokens=request.max_tokens, temperature=request.temperature, seed=request.seed)

    def activate(self, request: Request, lease: Lease, **trace_fields) -> None:
        """The head of the queue got its slot and its pages."""
        assert self.waiting and self.waiting[0] is request
        self.waiting.popleft()
        request.lease = lease
        request.computed = request.cached = lease.cached_tokens
        request.status = "active"
        self.active.append(request)
        self.trace.emit("admit", request_id=request.id, reused_tokens=request.cached, **trace_fields)

    def alive(self, request: Request) -> bool:
        return request.id in self.by_id

    # ---- tokens -------------------------------------------------------------------------
    def add_token(self, request: Request, token: int) -> str | None:
        """Record one generated token and tell the consumer.  Returns how the request ends with
        this token -- "stop", "length", "error" (the consumer's queue is full) -- or None."""
        request.tokens.append(token)
        request.output.append(token)
        self.counters["generated_tokens"] += 1
        if request.first_token is None:
            request.first_token = time.perf_counter()
            self.trace.emit("first_token", request_id=request.id, ttft_ms=(request.first_token - request.created) * 1000)
        try:
            request.events.put_nowait({"type": "token", "token_id": token})
        except queue.Full:
            return "error"
        if token in self.eos and not request.ignore_eos:
            return "stop"
        if len(request.output) >= request.max_tokens:
            return "length"
        return None

    # ---- departure ----------------------------------------------------------------------
    def retire(self, request: Request, reason: str, error: str | None = None) -> Lease | None:
        """Take the request out of the book for ``reason`` (stop, length, cancelled, error) and
        deliver its terminal event.  Returns the lease it still held: the caller decides when the
        pages go back (not while a step that writes them is running).  None if the request was
        gone already."""
        if self.by_id.pop(request.id, None) is None:
            return None
        try:
            self.active.remove(request)
        except ValueError:
            try:
                self.waiting.remove(request)
            except ValueError:
                pass
        lease, request.lease = request.lease, None
        request.status = reason
        if reason == "cancelled":
            self.counters["cancelled"] += 1
        elif reason == "error":
            self.counters["failed"] += 1
        else:
            self.counters["finished"] += 1
        done = {"type": "done", "finish_reason": reason, "error": error, "usage": request.usage(),
                "cached_tokens": request.cached, "elapsed_s": time.perf_counter() - request.created}
        self._deliver_last(request, done)
        self.trace.emit("finish", request_id=request.id,
                        **{key: value for key, value in done.items() if key != "type"})
        return lease

    @staticmethod
    def _deliver_last(request: Request, done: dict) -> None:
        """The terminal event always arrives: a consumer that let the queue fill up loses the
        undelivered token events, not the news that the request is over."""
        while True:
            try:
                request.events.put_nowait(done)
                return
            except queue.Full:
                try:
                    request.events.get_nowait()
                except queue.Empty:
                    pass

    def drain_events(self) -> None:
        """Act as the consumer of every live request (for callers that read ``output`` only)."""
        for request in list(self.by_id.values()):
            while True:
                try:
                    request.events.get_nowait()
                except queue.Empty:
                    break
