"""The cache manager: pages of keys and values, block tables, prefix sharing, state slots.

Layers are sorted into *groups* by what they need: all keys of a request, or a
window of them (per head count and head size).  Every group has its own pool of
pages, its own reference counts and free list, and its own block table per
request; a page of a group holds the keys and values of *every* layer of that
group for ``page_size`` consecutive tokens.  Pages go back to the free list when a
request ends or when a window has moved past them, and are handed out again.
Beside the pages there are slots of fixed size for per-request state (one row per
request slot for each layer that declares such a state), zeroed at admission.

Ownership follows flow_engine/cache.py:17-117: a page is referenced by the
requests whose tables hold it and by the prefix index; it is free when nobody
references it.  Prefix keys chain ``sha256(parent || tokens of the block)`` from
``sha256(namespace)`` (cache.py:60-65), only full blocks are shared, a hit never
covers the last prompt token (cache.py:67-78), and the least recently used index
entries are evicted when an allocation is short (cache.py:49-52).  Differences:
pages are promised at admission and taken when first written, and a block is
published as soon as the step that completed it has run, so that requests running
side by side can share a prefix.
"""
from __future__ import annotations

import hashlib
import math
import struct
from collections import OrderedDict
from dataclasses import dataclass, field

import torch

from ..parts.base import FixedState, PagedKV, PagedView, StateView


class CapacityError(RuntimeError):
    """Pages, request slots or queue places ran out."""


@dataclass
class Lease:
    """What one live request holds: a slot, and per group a block table."""
    slot: int
    namespace: str
    tables: list[list[int]]                 # per group: logical block -> page, -1 = none
    promised: list[int]                     # per group: pages promised but not yet taken
    first_live_block: list[int]             # per group: blocks before this were given back
    ensured_blocks: list[int] = field(default_factory=list)   # per group: every block below this has been handled
    cached_tokens: int = 0                  # tokens covered by shared prefix pages at admission
    published_blocks: int = 0
    reserved: bool = False                  # pages were promised at admission
    chain: list[bytes] = field(default_factory=list)   # prefix keys of this request's full blocks
    released: bool = False


class PageGroup:
    """Pool of one group: storage, reference counts, free list, device block table."""

    def __init__(self, need: PagedKV, entries: list[int], num_pages: int, page_size: int, max_requests: int,
                 max_blocks: int, dtype: torch.dtype, device: torch.device):
        self.need, self.entries = need, entries
        self.num_pages, self.page_size = num_pages, page_size
        self.window = need.window
        shape = (len(entries), num_pages, need.kv_heads, page_size, need.head_dim)
        self.k = torch.zeros(shape, dtype=dtype, device=device)
        self.v = torch.zeros(shape, dtype=dtype, device=device)
        self.refs = [0] * num_pages
        self.free = list(reversed(range(num_pages)))    # pop() hands out low ids first
        self.promised = 0
        self.host_table = torch.full((max_requests, max_blocks), -1, dtype=torch.int32,
                                     pin_memory=(device.type == "cuda"))
        self.device_table = torch.full((max_requests, max_blocks), -1, dtype=torch.int32, device=device)
        self.dirty: set[int] = set()
        self.layer_of_entry = {e: i for i, e in enumerate(entries)}

    @property
    def bytes(self) -> int:
        return 2 * self.k.numel() * self.k.element_size()

    def unpromised_free(self) -> int:
        return len(self.free) - self.promised


class CacheManager:
    def __init__(self, needs: list, page_size: int, num_pages: int, max_requests: int, max_context: int,
                 dtype: torch.dtype, device, prefix_cache: bool = True, poison_freed: bool = False):
        """``needs``: for every schedule entry ``(need, cache_of)`` as ``Model.cache_needs()`` gives it."""
        if min(page_size, num_pages, max_requests, max_context) <= 0:
            raise ValueError("page_size, num_pages, max_requests and max_context must be positive")
        self.device = torch.device(device)
        self.dtype = dtype
        self.page_size, self.num_pages, self.max_requests = page_size, num_pages, max_requests
        self.max_blocks = math.ceil(max_context / page_size)
        self.poison_freed = poison_freed
        self.needs = needs
        # ---- sort the schedule entries into groups
        self.groups: list[PageGroup] = []
        self.group_of_entry: dict[int, int] = {}
        self.state: dict[int, torch.Tensor] = {}
        by_need: dict[PagedKV, list[int]] = {}
        for i, (need, cache_of) in enumerate(needs):
            if isinstance(need, PagedKV):
                by_need.setdefault(need, []).append(i)
            elif isinstance(need, FixedState):
                self.state[i] = torch.zeros((max_requests, need.numel), dtype=need.dtype, device=self.device)
            elif need is not None:
                raise TypeError(f"schedule entry {i}: unknown cache need {need!r}")
        for need, entries in by_need.items():
            gi = len(self.groups)
            self.groups.append(PageGroup(need, entries, num_pages, page_size, max_requests, self.max_blocks,
                                         dtype, self.device))
            for e in entries:
                self.group_of_entry[e] = gi
        self.owner_of_entry = {i: (i if cache_of is None else cache_of) for i, (_, cache_of) in enumerate(needs)}
        # ---- request slots and the prefix index
        self.free_slots = list(reversed(range(max_requests)))
        self.leases: dict[int, Lease] = {}
        shareable = bool(self.groups) and not self.state and all(g.window is None for g in self.groups)
        self.prefix_cache = bool(prefix_cache and shareable)
        self.prefixes: "OrderedDict[bytes, tuple[int, ...]]" = OrderedDict()   # key -> page per group
        self.hits = 0
        self.evictions = 0

    # ------------------------------------------------------------------ views
    def view(self, entry: int):
        """The cache a mixer sees for schedule entry ``entry`` (its owner's, if it reads another's)."""
        owner = self.owner_of_entry[entry]
        if owner in self.state:
            return StateView(self.state[owner])
        gi = self.group_of_entry.get(owner)
        if gi is None:
            return None
        g = self.groups[gi]
        li = g.layer_of_entry[owner]
        return PagedView(g.k[li], g.v[li], g.device_table, self.page_size, g.window,
                         host_tables=lambda slot, _g=gi: list(self.leases[slot].tables[_g]))

    def views(self) -> list:
        return [self.view(i) for i in range(len(self.needs))]

    @property
    def allocated_bytes(self) -> int:
        return sum(g.bytes for g in self.groups) + sum(t.numel() * t.element_size() for t in self.state.values())

    # ------------------------------------------------------------------ pages
    def _release_page(self, gi: int, page: int) -> None:
        g = self.groups[gi]
        if not 0 <= page < g.num_pages or g.refs[page] <= 0:
            raise RuntimeError(f"page {page} of group {gi} released more often than it was taken")
        g.refs[page] -= 1
        if g.refs[page] == 0:
            if self.poison_freed:
                g.k[:, page].fill_(float("nan"))
                g.v[:, page].fill_(float("nan"))
            g.free.append(page)

    def _evict_one(self) -> bool:
        if not self.prefixes:
            return False
        _, pages = self.prefixes.popitem(last=False)
        for gi, page in enumerate(pages):
            self._release_page(gi, page)
        self.evictions += 1
        return True

    def _take_pages(self, gi: int, count: int, from_promise: int) -> list[int]:
        """Hand out ``count`` pages of group ``gi``; ``from_promise`` of them were promised before."""
        g = self.groups[gi]
        fresh = count - from_promise
        while g.unpromised_free() < fresh and self._evict_one():
            pass
        if g.unpromised_free() < fresh or len(g.free) < count:
            raise CapacityError("cache pages exhausted; the request must wait or ask for fewer tokens")
        g.promised -= from_promise
        pages = [g.free.pop() for _ in range(count)]
        for p in pages:
            g.refs[p] = 1
        return pages

    def _promise(self, gi: int, count: int) -> None:
        g = self.groups[gi]
        while g.unpromised_free() < count and self._evict_one():
            pass
        if g.unpromised_free() < count:
            raise CapacityError("cache pages exhausted; the request must wait or ask for fewer tokens")
        g.promised += count

    # ------------------------------------------------------------------ prefix keys
    def _keys(self, tokens, namespace: str, start_block: int = 0, parent: bytes | None = None):
        """Keys of the full blocks of ``tokens`` from ``start_block`` on (cache.py:60-65)."""
        ps = self.page_size
        if parent is None:
            parent = hashlib.sha256(namespace.encode()).digest()
        for b in range(start_block, len(tokens) // ps):
            chunk = tokens[b * ps:(b + 1) * ps]
            parent = hashlib.sha256(parent + struct.pack(f"<{ps}q", *chunk)).digest()
            yield parent

    # ------------------------------------------------------------------ request life cycle
    def pages_needed(self, total_tokens: int, step_tokens: int = 1) -> list[int]:
        """Worst number of pages a request of ``total_tokens`` holds at a time, per group.
        A windowed group never needs more than its window plus one step's tokens."""
        out = []
        for g in self.groups:
            full = math.ceil(total_tokens / self.page_size)
            if g.window is not None:
                full = min(full, math.ceil((g.window + step_tokens) / self.page_size) + 1)
            out.append(full)
        return out

    def admit(self, prompt, reserve_tokens: int = 0, namespace: str = "local", step_tokens: int = 1) -> Lease:
        """Give a request a slot, the shared pages of its known prefix, and a promise of the
        pages it can need for ``reserve_tokens`` tokens (0 = no promise; pages are then taken
        as they are needed and may run out).  All or nothing: on CapacityError nothing is held."""
        if not self.free_slots:
            raise CapacityError("no free request slot")
        if reserve_tokens and math.ceil(reserve_tokens / self.page_size) > self.max_blocks:
            raise ValueError("the request is longer than the configured context")
        shared: list[tuple[int, ...]] = []
        chain: list[bytes] = []
        if self.prefix_cache and prompt is not None:
            # at least the last prompt token must run to give its logits (cache.py:70)
            for key in self._keys(prompt[:-1], namespace):
                pages = self.prefixes.get(key)
                if pages is None:
                    break
                self.prefixes.move_to_end(key)
                for gi, page in enumerate(pages):
                    self.groups[gi].refs[page] += 1
                shared.append(pages)
                chain.append(key)
        promised = [0] * len(self.groups)
        try:
            if reserve_tokens:
                for gi, need in enumerate(self.pages_needed(reserve_tokens, step_tokens)):
                    extra = max(0, need - len(shared))
                    self._promise(gi, extra)
                    promised[gi] = extra
        except CapacityError:
            for gi, count in enumerate(promised):
                self.groups[gi].promised -= count
            for pages in shared:
                for gi, page in enumerate(pages):
                    self._release_page(gi, page)
            raise
        slot = self.free_slots.pop()
        tables = [[pages[gi] for pages in shared] for gi in range(len(self.groups))]
        lease = Lease(slot, namespace, tables, promised, [0] * len(self.groups),
                      cached_tokens=len(shared) * self.page_size, published_blocks=len(shared), chain=chain,
                      reserved=bool(reserve_tokens))
        self.leases[slot] = lease
        self.hits += lease.cached_tokens
        for gi, g in enumerate(self.groups):
            g.host_table[slot].fill_(-1)
            if tables[gi]:
                g.host_table[slot, :len(tables[gi])] = torch.tensor(tables[gi], dtype=torch.int32)
            g.dirty.add(slot)
        for t in self.state.values():
            t[slot].zero_()
        return lease

    def ensure(self, lease: Lease, n_tokens: int) -> None:
        """Make sure every group has pages for positions below ``n_tokens`` (those a window has
        already passed excepted).  Pages come out of the lease's promise first."""
        if lease.released:
            raise RuntimeError("the request has already given its pages back")
        blocks = math.ceil(n_tokens / self.page_size)
        if blocks > self.max_blocks:
            raise CapacityError("the request has outgrown the configured context")
        if not lease.ensured_blocks:
            lease.ensured_blocks = [0] * len(self.groups)
        for gi, g in enumerate(self.groups):
            if blocks <= lease.ensured_blocks[gi]:
                continue
            table = lease.tables[gi]
            if len(table) < blocks:
                table.extend([-1] * (blocks - len(table)))
            start = max(lease.first_live_block[gi], lease.ensured_blocks[gi])
            want = [b for b in range(start, blocks) if table[b] < 0]
            lease.ensured_blocks[gi] = blocks
            if not want:
                continue
            from_promise = min(lease.promised[gi], len(want))
            pages = self._take_pages(gi, len(want), from_promise)
            lease.promised[gi] -= from_promise
            for b, p in zip(want, pages):
                table[b] = p
                g.host_table[lease.slot, b] = p
            g.dirty.add(lease.slot)

    def check_writable(self, slot: int, start: int, end: int) -> None:
        """A step is about to write the keys and values of positions ``start .. end - 1`` of the request
        in ``slot``: every page it touches must be held by that request alone.  Shared pages are immutable
        (flow_engine/cache.py:3-5): only full blocks are ever shared and a hit never covers a position that
        is still to be computed, so a page with another holder here means the bookkeeping went wrong, and
        the step must not run."""
        lease = self.leases.get(slot)
        if lease is None:
            raise RuntimeError(f"request slot {slot} holds no lease")
        ps = self.page_size
        for gi, g in enumerate(self.groups):
            table = lease.tables[gi]
            for b in range(max(start // ps, lease.first_live_block[gi]), -(-end // ps)):
                page = table[b] if b < len(table) else -1
                if page < 0:
                    raise RuntimeError(f"slot {slot}: block {b} of group {gi} has no page for positions {start}..{end - 1}")
                if g.refs[page] != 1:
                    raise RuntimeError(f"slot {slot}: page {page} of group {gi} (block {b}) has {g.refs[page]} holders "
                                       f"and would be written at positions {start}..{end - 1}; shared pages are immutable")

    def advance(self, lease: Lease, tokens, computed: int) -> None:
        """Tell the manager that ``computed`` tokens of the request are now in the cache:
        full blocks become shareable, and pages that every later token's window has left
        behind go back to the free list."""
        ps = self.page_size
        if self.prefix_cache and tokens is not None:
            full = min(computed, len(tokens)) // ps
            if full > lease.published_blocks:
                parent = lease.chain[-1] if lease.chain else None
                for i, key in enumerate(self._keys(tokens[:full * ps], lease.namespace,
                                                   start_block=len(lease.chain), parent=parent)):
                    b = len(lease.chain)
                    lease.chain.append(key)
                    if key not in self.prefixes:
                        pages = tuple(lease.tables[gi][b] for gi in range(len(self.groups)))
                        if all(p >= 0 for p in pages):
                            self.prefixes[key] = pages
                            for gi, page in enumerate(pages):
                                self.groups[gi].refs[page] += 1
                lease.published_blocks = full
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            # the next token sits at position `computed` and sees keys > computed - window
            dead_before = max(0, computed - g.window + 1) // ps
            table = lease.tables[gi]
            for b in range(lease.first_live_block[gi], min(dead_before, len(table))):
                if table[b] >= 0:
                    self._release_page(gi, table[b])
                    table[b] = -1
                    g.host_table[lease.slot, b] = -1
                    if lease.reserved:               # the promise covers the pages held at a time
                        lease.promised[gi] += 1
                        g.promised += 1
                    g.dirty.add(lease.slot)
            lease.first_live_block[gi] = max(lease.first_live_block[gi], dead_before)

    def release(self, lease: Lease) -> None:
        """Give back everything the request holds (its references only; shared pages that the
        prefix index still references stay cached)."""
        if lease.released:
            raise RuntimeError("the request's pages were given back twice")
        lease.released = True
        for gi, g in enumerate(self.groups):
            for page in lease.tables[gi]:
                if page >= 0:
                    self._release_page(gi, page)
            lease.tables[gi] = []
            g.promised -= lease.promised[gi]
            lease.promised[gi] = 0
            g.host_table[lease.slot].fill_(-1)
            g.dirty.add(lease.slot)
        del self.leases[lease.slot]
        self.free_slots.append(lease.slot)

    def clear_prefixes(self) -> None:
        """Drop every index entry (cache.py:88-91); pages nobody else holds become free."""
        while self.prefixes:
            _, pages = self.prefixes.popitem(last=False)
            for gi, page in enumerate(pages):
                self._release_page(gi, page)

    # ------------------------------------------------------------------ device side
    def sync_tables(self) -> None:
        """Upload the block-table rows that changed since the last step."""
        for g in self.groups:
            for slot in g.dirty:
                g.device_table[slot].copy_(g.host_table[slot], non_blocking=True)
            g.dirty.clear()

    # ------------------------------------------------------------------ accounting
    def stats(self) -> dict:
        g0 = self.groups[0] if self.groups else None
        return {"physical_blocks": self.num_pages,
                "free_blocks": len(g0.free) if g0 else 0,
                "cached_prefix_blocks": len(self.prefixes),
                "prefix_hit_tokens": self.hits,
                "evictions": self.evictions,
                "kv_allocated_bytes": self.allocated_bytes,
                "groups": len(self.groups),
                "free_request_slots": len(self.free_slots)}

    def check_invariants(self) -> None:
        """Every page is either free or referenced, never both; reference counts equal the
        number of tables and index entries that hold the page; promises fit the free list."""
        for gi, g in enumerate(self.groups):
            held = [0] * g.num_pages
            for lease in self.leases.values():
                for page in lease.tables[gi]:
                    if page >= 0:
                        held[page] += 1
            for pages in self.prefixes.values():
                held[pages[gi]] += 1
            free = set(g.free)
            if len(free) != len(g.free):
                raise AssertionError(f"group {gi}: a page is on the free list twice")
            for page in range(g.num_pages):
                if held[page] != g.refs[page]:
                    raise AssertionError(f"group {gi}: page {page} has {g.refs[page]} references but {held[page]} holders")
                if (page in free) == (g.refs[page] > 0):
                    raise AssertionError(f"group {gi}: page {page} is both free and held, or neither")
            promised = sum(lease.promised[gi] for lease in self.leases.values())
            if promised != g.promised or g.promised > len(g.free) or g.promised < 0:
                raise AssertionError(f"group {gi}: promises {g.promised} do not match leases {promised} / free {len(g.free)}")
        slots = set(self.free_slots)
        if len(slots) != len(self.free_slots) or slots & set(self.leases) or len(slots) + len(self.leases) != self.max_requests:
            raise AssertionError("request slots are lost or held twice")
