"""The step function.

One step takes a batch of (request, its next tokens) -- portions of prompts beside
single decoded tokens, cut anywhere -- runs exactly those tokens as one flat batch
against the cache that earlier steps left, and returns fp32 logits at the wanted
rows.  The reference's forward takes uniform [B, T] batches only (flow_engine/
model.py:167-204) and its scheduler runs decode and prefill as two calls
(flow_engine/engine.py:249-260); here both are rows of one call.

All per-step metadata travels in one pinned host buffer and one host-to-device
copy.  The device copy lives at a fixed address, as do the workspace buffers, so a
decode-only step of a given size can be captured once as a CUDA graph and replayed.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..cache.manager import CacheManager
from ..csrc import ops
from ..models.model import Model
from ..parts.base import StepContext, Workspace
from ..parts.linear import configure_matmul_precision, verify_true_fp32
from ..sampling import select_tokens


@dataclass
class StepEntry:
    """The next tokens of one request in a step."""
    slot: int                      # request slot (from the cache manager's lease)
    tokens: list[int]              # consecutive tokens, the first at position ``start``
    start: int                     # tokens of this request already in the cache
    want: list[int] = field(default_factory=list)   # indices into ``tokens`` whose logits are wanted


GRAPH_BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


class StepError(RuntimeError):
    """A kernel reported a bad token id or a missing page."""


_STATUS_TEXT = {1: "a token id lies outside the vocabulary", 2: "a block table holds no page where one is needed",
                4: "a bounded wait in a kernel ran out"}


class ModelRunner:
    def __init__(self, model: Model, cache: CacheManager, max_step_tokens: int, max_step_seqs: int,
                 max_logit_rows: int | None = None, cuda_graphs: bool = True):
        if model.runtime.device.type != "cuda":
            raise RuntimeError("the step function runs on a CUDA device only; there is no CPU path")
        configure_matmul_precision()
        if model.runtime.dtype == torch.float32:
            verify_true_fp32(model.runtime.device)
        self.model, self.cache = model, cache
        self.device = model.runtime.device
        self.max_tokens = int(max_step_tokens)
        self.max_seqs = int(max_step_seqs)
        # batch sizes for which decode-only steps are captured: powers of two below the largest batch, and that batch
        self.buckets = tuple(b for b in GRAPH_BUCKETS if b < self.max_seqs) + (self.max_seqs,)
        self.max_rows = max(int(max_logit_rows or max_step_tokens), self.max_seqs)
        self.workspace = Workspace(self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.vocab = model.spec.vocab_size
        # ---- one staging buffer for all metadata of a step (int32 units)
        n, s, m = self.max_tokens, self.max_seqs, self.max_rows
        sizes = [("seed", 2 * m), ("counter", 2 * m), ("temperature", m), ("token_ids", n), ("positions", n),
                 ("seq_of_token", n), ("seq_slot", s), ("seq_q_start", s), ("seq_q_len", s), ("seq_kv_len", s),
                 ("logit_rows", m)]
        self._offsets, total = {}, 0
        for name, size in sizes:
            self._offsets[name] = (total, size)
            total += size + (-size % 4)          # keep every field 16-byte aligned
        self._host = torch.zeros(total, dtype=torch.int32, pin_memory=True)
        self._dev = torch.zeros(total, dtype=torch.int32, device=self.device)
        self._h = {k: self._host[o:o + sz] for k, (o, sz) in self._offsets.items()}
        host_np = self._host.numpy()              # same memory; numpy assigns Python lists much faster
        self._n = {k: host_np[o:o + sz] for k, (o, sz) in self._offsets.items()}
        self._n["temperature"] = self._n["temperature"].view("float32")
        self._n["seed"] = self._n["seed"].view("int64")
        self._n["counter"] = self._n["counter"].view("int64")
        self._d = {k: self._dev[o:o + sz] for k, (o, sz) in self._offsets.items()}
        self.sampled = torch.zeros(m + 1, dtype=torch.int32, device=self.device)   # ids, then the status word
        self._sampled_host = torch.zeros(m + 1, dtype=torch.int32, pin_memory=True)
        self._sampled_hosts = [torch.zeros(m + 1, dtype=torch.int32, pin_memory=True) for _ in range(2)]
        self._launched = 0
        self._staged = torch.cuda.Event()
        self._staged.record()
        self.use_graphs = bool(cuda_graphs and model.graph_safe)
        self._graphs: dict[int, tuple] = {}
        self.graph_kernels: dict[int, int] = {}      # bucket -> this engine's kernels inside the captured graph
        self.launches = 0
        self._graph_chose: int | None = None         # set by a graph step that chose a token of every row itself

    # ------------------------------------------------------------------ batch building
    def _stage(self, entries: list[StepEntry], pad_to: int = 0, all_rows: bool = False,
               device_refs: bool = False) -> tuple[StepContext, int]:
        """Fill the staging buffer for ``entries`` and copy it to the device.  ``pad_to`` pads the
        batch with rows that belong to no request; ``all_rows`` asks for the logits of every row.
        ``device_refs``: a token id -(i + 1) names the i-th token the step before chose (``launch``
        says so for a step it launches behind another); otherwise a negative id is refused here."""
        h = self._n
        self._staged.synchronize()       # the previous step's copy has read the pinned buffer
        n = sum(len(e.tokens) for e in entries)
        s = len(entries)
        if n == 0:
            raise ValueError("a step needs at least one token")
        rows_total = max(n, pad_to)
        seqs_total = max(s, pad_to) if pad_to else s
        if rows_total > self.max_tokens or seqs_total > self.max_seqs:
            raise ValueError(f"step of {n} tokens / {s} requests exceeds the runner's limits "
                             f"({self.max_tokens} tokens, {self.max_seqs} requests)")
        ids, pos, sot, rows = [], [], [], []
        slot, qs, ql, kl = [], [], [], []
        cursor = 0
        for si, e in enumerate(entries):
            t = len(e.tokens)
            if t == 0:
                raise ValueError("an entry without tokens cannot be part of a step")
            ids.extend(e.tokens)
            pos.extend(range(e.start, e.start + t))
            sot.extend([si] * t)
            self.cache.check_writable(e.slot, e.start, e.start + t)
            slot.append(e.slot); qs.append(cursor); ql.append(t); kl.append(e.start + t)
            for w in e.want:
                if not 0 <= w < t:
                    raise ValueError(f"wanted place {w} lies outside the {t} tokens of the entry")
                rows.append(cursor + w)
            cursor += t
        if all_rows:
            rows = list(range(rows_total))
        m = len(rows)
        if m > self.max_rows:
            raise ValueError(f"{m} wanted rows exceed the runner's limit of {self.max_rows}")
        h["token_ids"][:n] = ids
        lowest = int(h["token_ids"][:n].min())
        if lowest < (-self.max_rows if device_refs else 0):
            raise ValueError(f"token id {lowest} is negative" + (" and names no token of the step before" if device_refs else ""))
        h["positions"][:n] = pos
        h["seq_of_token"][:n] = sot
        if rows_total > n:
            h["token_ids"][n:rows_total] = 0
            h["positions"][n:rows_total] = 0
            h["seq_of_token"][n:rows_total] = -1
        h["seq_slot"][:s] = slot
        h["seq_q_start"][:s] = qs
        h["seq_q_len"][:s] = ql
        h["seq_kv_len"][:s] = kl
        if seqs_total > s:
            for key in ("seq_slot", "seq_q_start", "seq_q_len", "seq_kv_len"):
                h[key][s:seqs_total] = 0
        if m:
            h["logit_rows"][:m] = rows
        self._dev.copy_(self._host, non_blocking=True)
        self._staged.record()
        self.cache.sync_tables()
        d = self._d
        ctx = StepContext(
            runtime=self.model.runtime, workspace=self.workspace, n_tokens=rows_total, n_seqs=seqs_total,
            token_ids=d["token_ids"][:rows_total], positions=d["positions"][:rows_total],
            seq_of_token=d["seq_of_token"][:rows_total], seq_slot=d["seq_slot"][:seqs_total],
            seq_q_start=d["seq_q_start"][:seqs_total], seq_q_len=d["seq_q_len"][:seqs_total],
            seq_kv_len=d["seq_kv_len"][:seqs_total], status=self.status,
            host_slot=slot, host_q_start=qs, host_q_len=ql, host_kv_len=kl,
            max_q_len=max(ql), max_kv_len=max(kl), decode_only=all(t == 1 for t in ql), fixed_shape=bool(pad_to),
            device_tokens=self.sampled if (device_refs or pad_to) else None)
        return ctx, m

    def _padding_context(self, rows: int, logit_rows: int) -> StepContext:
        """A step of ``rows`` padding rows: every kernel runs, none touches the cache."""
        h = self._n
        self._staged.synchronize()
        h["token_ids"][:rows] = 0
        h["positions"][:rows] = 0
        h["seq_of_token"][:rows] = -1
        seqs = min(rows, self.max_seqs)
        for key in ("seq_slot", "seq_q_start", "seq_q_len", "seq_kv_len"):
            h[key][:seqs] = 0
        h["logit_rows"][:logit_rows] = [i % rows for i in range(logit_rows)]
        self._dev.copy_(self._host, non_blocking=True)
        self._staged.record()
        d = self._d
        return StepContext(
            runtime=self.model.runtime, workspace=self.workspace, n_tokens=rows, n_seqs=seqs,
            token_ids=d["token_ids"][:rows], positions=d["positions"][:rows], seq_of_token=d["seq_of_token"][:rows],
            seq_slot=d["seq_slot"][:seqs], seq_q_start=d["seq_q_start"][:seqs], seq_q_len=d["seq_q_len"][:seqs],
            seq_kv_len=d["seq_kv_len"][:seqs], status=self.status, host_slot=[0] * seqs, host_q_start=[0] * seqs,
            host_q_len=[0] * seqs, host_kv_len=[0] * seqs, max_q_len=1,
            max_kv_len=self.cache.max_blocks * self.cache.page_size, decode_only=(rows <= self.max_seqs),
            fixed_shape=True, device_tokens=self.sampled)

    # ------------------------------------------------------------------ the step
    @torch.inference_mode()
    def step(self, entries: list[StepEntry], device_refs: bool = False) -> torch.Tensor:
        """Run the tokens of ``entries`` and return fp32 logits ``[wanted rows, vocab]`` on the
        device, in the order of the entries and of their ``want`` lists."""
        if self.use_graphs and entries and all(len(e.tokens) == 1 for e in entries):
            bucket = next((b for b in self.buckets if len(entries) <= b), None)
            if bucket is not None:
                return self._graph_step(entries, bucket, device_refs)
        ctx, m = self._stage(entries, device_refs=device_refs)
        logits = self.workspace.get("runner.logits", (max(m, 1), self.vocab), torch.float32)
        self.model.forward(ctx, self.cache.views(), self._d["logit_rows"], m, logits)
        return logits[:m]

    # ------------------------------------------------------------------ CUDA graphs for decode-only steps
    def reserve(self) -> None:
        """Run one step of padding rows at the largest size, so that every workspace buffer
        has its final address, then forbid growth: captured graphs hold these addresses."""
        if self.workspace.frozen:
            return
        logits = self.workspace.get("runner.logits", (self.max_rows, self.vocab), torch.float32)
        ctx = self._padding_context(self.max_tokens, self.max_rows)
        self.model.forward(ctx, self.cache.views(), self._d["logit_rows"], self.max_rows, logits)
        for bucket in self.buckets:           # decode-only kernels may use buffers of their own
            ctx = self._padding_context(bucket, bucket)
            self.model.forward(ctx, self.cache.views(), self._d["logit_rows"], bucket, logits)
        torch.cuda.current_stream().synchronize()
        self.status.zero_()
        self.workspace.frozen = True

    def _capture(self, bucket: int):
        self.reserve()
        rows = bucket
        logits = self.workspace.get("runner.logits", (self.max_rows, self.vocab), torch.float32)
        ctx = self._padding_context(bucket, rows)
        views = self.cache.views()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            spare = torch.empty_like(self.sampled)      # `sampled` may hold tokens that the step being prepared refers to
            for _ in range(2):
                self.model.forward(ctx, views, self._d["logit_rows"], rows, logits)
                self._select_in_graph(logits, rows, spare)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES[0]
        with torch.cuda.graph(graph):
            self.model.forward(ctx, views, self._d["logit_rows"], rows, logits)
            # the graph also chooses a token for every row (by each row's own temperature, seed and counter, which
            # travel in the step's staging copy) and puts the status word behind them: a step that wants a token of
            # every row launches nothing after the graph but the copy to the host
            self._select_in_graph(logits, rows)
        self.graph_kernels[bucket] = ops.LAUNCHES[0] - before
        self.status.zero_()
        self._graphs[bucket] = (graph, logits)
        return self._graphs[bucket]

    def _select_in_graph(self, logits: torch.Tensor, rows: int, into: torch.Tensor | None = None) -> None:
        into = self.sampled if into is None else into
        select_tokens(into, logits, rows, self._d["temperature"].view(torch.float32),
                      self._d["seed"].view(torch.int64), self._d["counter"].view(torch.int64))
        into[rows:rows + 1].copy_(self.status)

    def _graph_step(self, entries: list[StepEntry], bucket: int, device_refs: bool = False) -> torch.Tensor:
        if not self._graphs:
            # capture every bucket at the first decode step, so that a batch that shrinks or grows
            # later does not pay for a capture in the middle of generation
            for b in self.buckets:
                self._capture(b)
        graph, logits = self._graphs.get(bucket) or self._capture(bucket)
        wanted = [i for i, e in enumerate(entries) if e.want]
        for e in entries:
            e_want = e.want
            if e_want and e_want != [0]:
                raise ValueError("a single-token entry can only want place 0")
        self._stage([StepEntry(e.slot, e.tokens, e.start, []) for e in entries], pad_to=bucket, all_rows=True,
                    device_refs=device_refs)
        graph.replay()
        if len(wanted) == len(entries):
            self._graph_chose = bucket          # `sampled` holds a token of every row and, at [bucket], the status
        if wanted == list(range(len(wanted))):
            return logits[:len(wanted)]
        return logits.index_select(0, torch.tensor(wanted, dtype=torch.long, device=self.device))

    # ------------------------------------------------------------------ sampling
    def stage_sampling(self, temperature: list[float], seed: list[int], counter: list[int]) -> None:
        """Per wanted row: temperature (0 = greedy), seed and draw counter.  Must be called
        before ``step`` of the same batch, as it travels in the same copy."""
        m = len(temperature)
        self._staged.synchronize()
        self._n["temperature"][:m] = temperature
        self._n["seed"][:m] = seed
        self._n["counter"][:m] = counter

    @torch.inference_mode()
    def sample(self, logits: torch.Tensor, greedy_only: bool = False) -> list[int]:
        """Choose one token per row of ``logits`` on the device; one copy brings the ids and
        the kernels' status word to the host."""
        m = logits.shape[0]
        if greedy_only:
            select_tokens(self.sampled, logits, m)
        else:
            select_tokens(self.sampled, logits, m, self._d["temperature"].view(torch.float32),
                          self._d["seed"].view(torch.int64), self._d["counter"].view(torch.int64))
        self.sampled[m:m + 1].copy_(self.status)
        self._sampled_host[:m + 1].copy_(self.sampled[:m + 1], non_blocking=True)
        torch.cuda.current_stream().synchronize()
        out = self._sampled_host[:m + 1].tolist()
        self._raise_on_status(out[m])
        return out[:m]

    # ------------------------------------------------------------------ steps in flight
    @torch.inference_mode()
    def launch(self, entries: list[StepEntry], temperature: list[float], seed: list[int], counter: list[int],
               device_refs: bool = False):
        """Launch a whole step -- forward, token selection, copy of the chosen ids to the host --
        and return without waiting.  With ``device_refs`` a token id -(i + 1) in an entry stands for the
        i-th token chosen by the step launched just before, which is still on the device; so the next
        step can be launched before this one's tokens have reached the host.  ``finish`` waits."""
        self.stage_sampling(temperature, seed, counter)
        self._graph_chose = None
        logits = self.step(entries, device_refs)
        m = logits.shape[0]
        host = self._sampled_hosts[self._launched % 2]
        self._launched += 1
        at = m                                  # where the status word lies behind the chosen ids
        if self._graph_chose is not None:
            at = self._graph_chose              # the captured graph has chosen the tokens already
        else:
            if m:
                if all(t == 0 for t in temperature):
                    select_tokens(self.sampled, logits, m)
                else:
                    select_tokens(self.sampled, logits, m, self._d["temperature"].view(torch.float32),
                                  self._d["seed"].view(torch.int64), self._d["counter"].view(torch.int64))
            self.sampled[m:m + 1].copy_(self.status)
        host[:at + 1].copy_(self.sampled[:at + 1], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        return (done, host, m, at)

    def finish(self, pending) -> list[int]:
        """Wait for a launched step; its chosen token ids, in the order of the wanted rows."""
        done, host, m, at = pending
        done.synchronize()
        out = host[:at + 1].tolist()
        self._raise_on_status(out[at])
        return out[:m]

    # ------------------------------------------------------------------ errors
    def _raise_on_status(self, code: int) -> None:
        if code:
            self.status.zero_()
            what = "; ".join(text for bit, text in _STATUS_TEXT.items() if code & bit) or f"code {code}"
            raise StepError(f"a kernel refused part of the step: {what}")

    def check_status(self) -> None:
        """Read the kernels' status word (synchronises) and raise if a kernel refused something."""
        self._raise_on_status(int(self.status.item()))
