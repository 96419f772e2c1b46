"""The cache manager: pages of keys and values with a block table per request, and state slots.

The reference keeps, per layer and per sequence slot, one contiguous ring sized at plan time
(crates/kf-core/src/plan.rs:59-64, crates/kf-backend-cuda/src/exec.rs:1466-1498) and learns what a layer
keeps only from its `StateNeed` (crates/kf-core/src/layer.rs:29-43).  This manager keeps that
declaration-driven shape but stores tokens in fixed-size pages:

* cache slots whose needs have the same lifetime rule (the same window, or none) form a *group*;
  a group has one page pool (page ids) and one block table per request, shared by all its slots:
  page id `i` names the i-th page of every slot's own storage;
* a request's block table maps absolute page index (position // page_size) to a page id, -1 where
  the request holds no page (not yet reached, or slid out of the window);
* pages return to the pool when the request is released, and in a windowed group as soon as every
  position they hold is out of reach of any later query: a query at position p reads keys
  j >= p - window + 1, so after a step that leaves the request at length n the pages that end at or
  before n - window + 1 go back;
* every live request also owns one state slot (an index into dense per-request state arrays) for
  mixers that keep a state of fixed size; it is zeroed at admission.

All bookkeeping is on the host; device memory is allocated once at construction.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..parts.base import FixedState, PagedKV


class OutOfPages(RuntimeError):
    """A reservation needs more pages than the group's pool has free."""


class CacheError(RuntimeError):
    """Misuse of the manager: unknown request, double release, a page freed twice."""


class PagePool:
    """Page ids 0..n-1 with a free list; refuses to free a page twice or one it never gave out."""

    def __init__(self, n_pages: int):
        self.n_pages = int(n_pages)
        self._free = list(range(self.n_pages - 1, -1, -1))      # pop() hands out low ids first
        self._held = [False] * self.n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        p = self._free.pop()
        self._held[p] = True
        return p

    def give_back(self, page: int) -> None:
        if not (0 <= page < self.n_pages) or not self._held[page]:
            raise CacheError(f"page {page} is not held")
        self._held[page] = False
        self._free.append(page)

    def held_pages(self) -> list[int]:
        return [i for i, h in enumerate(self._held) if h]


@dataclass
class _Group:
    window: int | None
    pool: PagePool
    slots: list[int]                                   # cache slots in this group
    tables: dict = field(default_factory=dict)         # request -> list[int] (absolute page index -> page id or -1)
    first_live: dict = field(default_factory=dict)     # request -> first page index still held


class PagedKVView:
    """What a mixer sees of its cache slot during one step."""

    def __init__(self, pages: torch.Tensor, page_size: int, group: int, writes: bool):
        self.pages = pages              # [n_pages, 2 (key, value), n_kv_heads, page_size, head_dim]
        self.page_size = page_size
        self.group = group
        self.writes = writes


class FixedStateView:
    def __init__(self, state: torch.Tensor, writes: bool):
        self.state = state              # [max_requests, *shape]; row = the request's state slot
        self.writes = writes


class CacheManager:
    def __init__(self, needs: list, *, page_size: int, n_pages: int, max_requests: int, max_context: int,
                 dtype: torch.dtype, device, n_pages_windowed: int | None = None):
        """`needs[s]` is the `StateNeed` of cache slot s (or None).  `n_pages` is the size of each group's
        pool (`n_pages_windowed` for groups with a window, when given)."""
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_context = int(max_context)
        self.max_pages_per_request = -(-self.max_context // self.page_size)
        self.dtype, self.device = dtype, torch.device(device)
        self.needs = list(needs)
        self.groups: list[_Group] = []
        self._group_of_slot: dict[int, int] = {}
        self.storage: dict[int, torch.Tensor] = {}
        by_window: dict = {}
        for s, need in enumerate(self.needs):
            if isinstance(need, PagedKV):
                g = by_window.get(need.window)
                if g is None:
                    n = n_pages_windowed if (need.window is not None and n_pages_windowed is not None) else n_pages
                    g = len(self.groups)
                    by_window[need.window] = g
                    self.groups.append(_Group(need.window, PagePool(n), []))
                self.groups[g].slots.append(s)
                self._group_of_slot[s] = g
                self.storage[s] = torch.zeros((self.groups[g].pool.n_pages, 2, need.n_kv_heads, self.page_size,
                                               need.head_dim), dtype=dtype, device=self.device)
            elif isinstance(need, FixedState):
                self.storage[s] = torch.zeros((self.max_requests, *need.shape), dtype=need.dtype, device=self.device)
            elif need is not None:
                raise TypeError(f"cache slot {s}: unknown state need {need!r}")
        # host mirror of every block table, one row per state slot, ready to be copied into a step's integer block
        self._table_np = [np.full((self.max_requests, (self.max_pages_per_request + 3) & ~3), -1, dtype=np.int32)
                          for _ in self.groups]          # width padded to a multiple of 4, as the step's block is
        self._length: dict = {}                 # request -> tokens committed
        self._reserved: dict = {}               # request -> tokens reserved beyond the committed length
        self._state_slot: dict = {}
        self._free_state_slots = list(range(self.max_requests - 1, -1, -1))

    # ---- requests ---------------------------------------------------------------------------------
    def __contains__(self, request) -> bool:
        return request in self._length

    @property
    def n_live(self) -> int:
        return len(self._length)

    def length(self, request) -> int:
        return self._length[request]

    def state_slot(self, request) -> int:
        return self._state_slot[request]

    def add_request(self, request) -> int:
        """Admit a request: gives it a state slot (zeroed) and empty block tables."""
        if request in self._length:
            raise CacheError(f"request {request!r} is already live")
        if not self._free_state_slots:
            raise CacheError(f"more than {self.max_requests} live requests")
        slot = self._free_state_slots.pop()
        self._state_slot[request] = slot
        self._length[request] = 0
        self._reserved[request] = 0
        for gi, g in enumerate(self.groups):
            g.tables[request] = []
            g.first_live[request] = 0
            self._table_np[gi][slot, :] = -1
        for s, need in enumerate(self.needs):
            if isinstance(need, FixedState):
                self.storage[s][slot].zero_()
        return slot

    def pages_needed(self, request, n_new: int) -> list[int]:
        """Pages each group must still take so the request can hold `n_new` more tokens."""
        end = self._length[request] + self._reserved[request] + n_new
        want = -(-end // self.page_size)
        return [max(0, want - len(g.tables[request])) for g in self.groups]

    def can_reserve(self, request, n_new: int) -> bool:
        if self._length[request] + self._reserved[request] + n_new > self.max_context:
            return False
        return all(n <= g.pool.n_free for n, g in zip(self.pages_needed(request, n_new), self.groups))

    def reserve(self, request, n_new: int) -> None:
        """Take the pages for `n_new` more tokens in every group, or none at all (raises OutOfPages)."""
        if request not in self._length:
            raise CacheError(f"request {request!r} is not live")
        if self._length[request] + self._reserved[request] + n_new > self.max_context:
            raise OutOfPages(f"request {request!r} would exceed the context of {self.max_context} tokens")
        needed = self.pages_needed(request, n_new)
        for n, g in zip(needed, self.groups):
            if n > g.pool.n_free:
                raise OutOfPages(f"group with window {g.window}: {n} pages needed, {g.pool.n_free} free")
        slot = self._state_slot[request]
        for gi, (n, g) in enumerate(zip(needed, self.groups)):
            table = g.tables[request]
            for _ in range(n):
                page = g.pool.take()
                self._table_np[gi][slot, len(table)] = page
                table.append(page)
        self._reserved[request] += n_new

    def cancel_reservation(self, request) -> None:
        """Give back the pages taken for tokens that were reserved but never committed."""
        self._reserved[request] = 0
        keep = -(-self._length[request] // self.page_size)
        slot = self._state_slot[request]
        for gi, g in enumerate(self.groups):
            table = g.tables[request]
            while len(table) > keep:
                p = table.pop()
                self._table_np[gi][slot, len(table)] = -1
                if p >= 0:
                    g.pool.give_back(p)

    def commit(self, request, n_new: int) -> None:
        """The step that wrote `n_new` reserved tokens succeeded: advance, and give back slid-out pages."""
        if n_new > self._reserved[request]:
            raise CacheError(f"commit of {n_new} tokens, only {self._reserved[request]} reserved")
        self._reserved[request] -= n_new
        self._length[request] += n_new
        n = self._length[request]
        slot = self._state_slot[request]
        for gi, g in enumerate(self.groups):
            if g.window is None:
                continue
            # positions < n - window + 1 are out of reach of every later query
            dead_pages = max(0, n - g.window + 1) // self.page_size
            table = g.tables[request]
            for i in range(g.first_live[request], min(dead_pages, len(table))):
                if table[i] >= 0:
                    g.pool.give_back(table[i])
                    table[i] = -1
                    self._table_np[gi][slot, i] = -1
            g.first_live[request] = max(g.first_live[request], min(dead_pages, len(table)))

    def release(self, request) -> None:
        """The request is finished (or preempted): everything it holds goes back."""
        if request not in self._length:
            raise CacheError(f"request {request!r} is not live")
        slot = self._state_slot[request]
        for gi, g in enumerate(self.groups):
            for p in g.tables.pop(request):
                if p >= 0:
                    g.pool.give_back(p)
            g.first_live.pop(request)
            self._table_np[gi][slot, :] = -1
        self._free_state_slots.append(self._state_slot.pop(request))
        del self._length[request]
        del self._reserved[request]

    # ---- what a step needs ----------------------------------------------------------------------
    def block_table(self, group: int, request) -> list[int]:
        return self.groups[group].tables[request]

    def table_rows(self, group: int, state_slots) -> np.ndarray:
        """Block-table rows (full width, -1 where no page is held) of the requests in the given state slots."""
        return self._table_np[group][state_slots]

    def group_of(self, cache_slot: int) -> int | None:
        return self._group_of_slot.get(cache_slot)

    def view(self, cache_slot: int, writes: bool):
        need = self.needs[cache_slot]
        if isinstance(need, PagedKV):
            return PagedKVView(self.storage[cache_slot], self.page_size, self._group_of_slot[cache_slot], writes)
        if isinstance(need, FixedState):
            return FixedStateView(self.storage[cache_slot], writes)
        return None

    # ---- accounting and self-check -----------------------------------------------------------------
    def free_pages(self) -> list[int]:
        return [g.pool.n_free for g in self.groups]

    def bytes_per_token(self) -> int:
        n = 0
        for s, need in enumerate(self.needs):
            if isinstance(need, PagedKV):
                n += 2 * need.n_kv_heads * need.head_dim * self.storage[s].element_size()
        return n

    def check(self) -> None:
        """Every page is either free or in exactly one table; raises CacheError otherwise."""
        for gi, g in enumerate(self.groups):
            seen: dict[int, object] = {}
            for req, table in g.tables.items():
                for p in table:
                    if p < 0:
                        continue
                    if p in seen:
                        raise CacheError(f"group {gi}: page {p} held by {seen[p]!r} and {req!r}")
                    seen[p] = req
            for req, table in g.tables.items():
                row = self._table_np[gi][self._state_slot[req]]
                if list(row[:len(table)]) != list(table) or (row[len(table):] != -1).any():
                    raise CacheError(f"group {gi}: host mirror of {req!r}'s block table is stale")
            held = set(g.pool.held_pages())
            if held != set(seen):
                raise CacheError(f"group {gi}: pool holds {sorted(held)}, tables hold {sorted(seen)}")
            if len(held) + g.pool.n_free != g.pool.n_pages:
                raise CacheError(f"group {gi}: {len(held)} held + {g.pool.n_free} free != {g.pool.n_pages}")
