"""The cache manager: pages of keys and values with a block table for each request, and state slots.

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

The bookkeeping itself (pools, tables, the host mirror of the tables that steps copy from) is native code,
`csrc/host_runtime.cpp`; this class owns the device storage and turns its status codes into exceptions.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .kinds import FixedStateView, PagedKVView, kind_of       # the views are re-exported from here

_OK, _E_NOT_LIVE, _E_ALREADY_LIVE, _E_NO_SLOT, _E_OUT_OF_PAGES, _E_CONTEXT, _E_COMMIT, _E_PAGE, _E_INCONSISTENT = range(9)


class OutOfPages(RuntimeError):
    """A reservation needs more pages than the group's pool has free."""


class CacheError(RuntimeError):
    """Misuse of the manager: unknown request, double release, a page freed twice."""


_host = None


def host_library():
    """The native host runtime (compiled with the C++ compiler at first use)."""
    global _host
    if _host is None:
        from ..csrc import build as _build
        lib = ctypes.CDLL(_build.build_host())
        lib.kf_pool_create.restype = ctypes.c_void_p
        lib.kf_cache_create.restype = ctypes.c_void_p
        lib.kf_cache_mirror.restype = ctypes.POINTER(ctypes.c_int)
        lib.kf_cache_pool_n_taken.restype = ctypes.c_long
        lib.kf_cache_pool_n_taken.argtypes = [ctypes.c_void_p, ctypes.c_int]
        for name in ("kf_pool_destroy", "kf_pool_take", "kf_pool_give_back", "kf_pool_n_free", "kf_pool_is_held",
                     "kf_cache_destroy", "kf_cache_width", "kf_cache_n_live", "kf_cache_pool_n_free",
                     "kf_cache_pool_is_held", "kf_cache_mirror", "kf_cache_check"):
            getattr(lib, name).argtypes = [ctypes.c_void_p] + [ctypes.c_int] * {"kf_pool_give_back": 1, "kf_pool_is_held": 1,
                                                                                  "kf_cache_pool_n_free": 1, "kf_cache_pool_is_held": 2,
                                                                                  "kf_cache_mirror": 1}.get(name, 0)
        i64 = ctypes.c_int64
        for name, extra in (("kf_cache_contains", []), ("kf_cache_length", []), ("kf_cache_state_slot", []),
                            ("kf_cache_add_request", []), ("kf_cache_cancel_reservation", []), ("kf_cache_release", []),
                            ("kf_cache_reserve", [ctypes.c_int]), ("kf_cache_commit", [ctypes.c_int]),
                            ("kf_cache_pages_needed", [ctypes.c_int, ctypes.c_void_p])):
            getattr(lib, name).argtypes = [ctypes.c_void_p, i64] + extra
        lib.kf_cache_table.argtypes = [ctypes.c_void_p, ctypes.c_int, i64, ctypes.c_void_p, ctypes.c_int]
        lib.kf_step_layout.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                       ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
        lib.kf_step_fill.argtypes = [ctypes.c_void_p, ctypes.c_int] + [ctypes.c_void_p] * 5 + [ctypes.c_int] * 3 + [ctypes.c_void_p,
                                                                                                   ctypes.c_void_p]
        vp, ci = ctypes.c_void_p, ctypes.c_int
        lib.kf_sched_create.restype = vp
        lib.kf_sched_create.argtypes = [vp, ci, ci]
        lib.kf_sched_destroy.argtypes = [vp]
        lib.kf_sched_pad_decode_rows.argtypes = [vp, ci]
        lib.kf_sched_add.argtypes = [vp, i64, ci, ci, ci]
        lib.kf_sched_adopt.argtypes = [vp, i64, ci, ci, ci, ci]
        lib.kf_sched_forget.argtypes = [vp, i64]
        lib.kf_sched_schedule.argtypes = [vp, vp, ci, vp, ci, vp]
        lib.kf_sched_advance.argtypes = [vp, i64, ci]
        lib.kf_sched_on_token.argtypes = [vp, i64, ci]
        lib.kf_sched_finish.argtypes = [vp, i64]
        lib.kf_sched_preempt_last.argtypes = [vp, i64]
        lib.kf_sched_preempt_last.restype = i64
        lib.kf_sched_n_preemptions.argtypes = [vp]
        lib.kf_sched_n_preemptions.restype = ctypes.c_long
        lib.kf_sched_counts.argtypes = [vp, vp, vp]
        lib.kf_sched_lists.argtypes = [vp, vp, vp]
        lib.kf_sched_state.argtypes = [vp, i64, vp]
        _host = lib
    return _host


class PagePool:
    """Page ids 0..n-1 with a free list; refuses to free a page twice or one it never gave out."""

    def __init__(self, n_pages: int):
        self.n_pages = int(n_pages)
        self._lib = host_library()
        self._h = ctypes.c_void_p(self._lib.kf_pool_create(self.n_pages))

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.kf_pool_destroy(self._h)
            self._h = None

    @property
    def n_free(self) -> int:
        return self._lib.kf_pool_n_free(self._h)

    def take(self) -> int:
        p = self._lib.kf_pool_take(self._h)
        if p < 0:
            raise OutOfPages("no free page")
        return p

    def give_back(self, page: int) -> None:
        if self._lib.kf_pool_give_back(self._h, int(page)) != _OK:
            raise CacheError(f"page {page} is not held")

    def held_pages(self) -> list[int]:
        return [i for i in range(self.n_pages) if self._lib.kf_pool_is_held(self._h, i)]


class _GroupPool:
    """Read-only view of one group's pool inside the native manager."""

    def __init__(self, manager, g: int, n_pages: int):
        self._m, self._g, self.n_pages = manager, g, n_pages

    @property
    def n_free(self) -> int:
        return self._m._lib.kf_cache_pool_n_free(self._m._h, self._g)

    def held_pages(self) -> list[int]:
        return [i for i in range(self.n_pages) if self._m._lib.kf_cache_pool_is_held(self._m._h, self._g, i)]


class _GroupTables:
    def __init__(self, manager, g: int):
        self._m, self._g = manager, g

    def __getitem__(self, request) -> list[int]:
        return self._m.block_table(self._g, request)

    def items(self):
        return [(r, self._m.block_table(self._g, r)) for r in list(self._m._key)]


class _Group:
    def __init__(self, manager, g: int, window: int | None, n_pages: int):
        self.window = window
        self.slots: list[int] = []                       # cache slots in this group
        self.pool = _GroupPool(manager, g, n_pages)
        self.tables = _GroupTables(manager, g)


class CacheManager:
    def __init__(self, needs: list, *, page_size: int, n_pages: int | dict, max_requests: int, max_context: int,
                 dtype: torch.dtype, device, n_pages_windowed: int | None = None):
        """`needs[s]` is the `StateNeed` of cache slot s (or None); what the manager must know about it comes from the
        state kind registered for its class (`cache/kinds.py`).  `n_pages` is the size of each group's pool, or a
        dictionary {window or None: pages} as `plan_cache` gives it (`n_pages_windowed`: the size for groups with a
        window when `n_pages` is one number)."""
        self.page_size = int(page_size)
        self.max_requests = int(max_requests)
        self.max_context = int(max_context)
        self.max_pages_per_request = -(-self.max_context // self.page_size)
        self.dtype, self.device = dtype, torch.device(device)
        self.needs = list(needs)
        self._kinds = [None if n is None else kind_of(n) for n in self.needs]
        self._lib = host_library()
        self.groups: list[_Group] = []
        self._group_of_slot: dict[int, int] = {}
        self.storage: dict[int, torch.Tensor] = {}
        by_window: dict = {}
        pool_sizes: list[int] = []
        for s, (need, kind) in enumerate(zip(self.needs, self._kinds)):
            if need is None:
                continue
            if kind.paged:
                window = kind.window(need)
                g = by_window.get(window)
                if g is None:
                    if isinstance(n_pages, dict):
                        n = n_pages[window]
                    else:
                        n = n_pages_windowed if (window is not None and n_pages_windowed is not None) else n_pages
                    g = len(self.groups)
                    by_window[window] = g
                    self.groups.append(_Group(self, g, window, int(n)))
                    pool_sizes.append(int(n))
                self.groups[g].slots.append(s)
                self._group_of_slot[s] = g
                self.storage[s] = torch.zeros((pool_sizes[g], *kind.page_shape(need, self.page_size)),
                                              dtype=kind.dtype(need, dtype), device=self.device)
            else:
                self.storage[s] = torch.zeros((self.max_requests, *kind.shape(need)), dtype=kind.dtype(need, dtype),
                                              device=self.device)
        G = len(self.groups)
        windows = (ctypes.c_int * max(G, 1))(*[(-1 if g.window is None else int(g.window)) for g in self.groups])
        sizes = (ctypes.c_int * max(G, 1))(*pool_sizes)
        self._h = ctypes.c_void_p(self._lib.kf_cache_create(G, windows, sizes, self.page_size, self.max_requests,
                                                            self.max_context))
        self.table_width = self._lib.kf_cache_width(self._h)
        # the native block-table mirrors, [max_requests, table_width] per group, as numpy views (no copy)
        self._table_np = [np.ctypeslib.as_array(self._lib.kf_cache_mirror(self._h, g), shape=(self.max_requests, self.table_width))
                          for g in range(G)]
        self._key: dict = {}                    # request (any hashable) -> the 64-bit key the native side knows it by
        self._next_key = 1
        self._scratch = (ctypes.c_int * max(G, 1))()

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.kf_cache_destroy(self._h)
            self._h = None

    # ---- requests ---------------------------------------------------------------------------------------
    def key_of(self, request) -> int:
        try:
            return self._key[request]
        except KeyError:
            raise CacheError(f"request {request!r} is not live") from None

    def __contains__(self, request) -> bool:
        return request in self._key

    @property
    def n_live(self) -> int:
        return len(self._key)

    def length(self, request) -> int:
        return self._lib.kf_cache_length(self._h, self.key_of(request))

    def state_slot(self, request) -> int:
        return self._lib.kf_cache_state_slot(self._h, self.key_of(request))

    def add_request(self, request) -> int:
        """Admit a request: gives it a state slot (zeroed) and empty block tables."""
        if request in self._key:
            raise CacheError(f"request {request!r} is already live")
        key = self._next_key
        slot = self._lib.kf_cache_add_request(self._h, key)
        if slot == -_E_NO_SLOT:
            raise CacheError(f"more than {self.max_requests} live requests")
        if slot < 0:
            raise CacheError(f"request {request!r}: native manager refused admission (code {-slot})")
        self._next_key += 1
        self._key[request] = key
        self._zero_fixed(slot)
        return slot

    def new_key(self) -> int:
        """A fresh 64-bit key for a request that the native scheduler will admit by itself later."""
        key = self._next_key
        self._next_key += 1
        return key

    def adopt(self, request, key: int, slot: int) -> None:
        """The native side has admitted `request` under `key` into state slot `slot`: record it here (and zero its
        fixed-size state)."""
        if request in self._key:
            raise CacheError(f"request {request!r} is already live")
        self._key[request] = int(key)
        self._zero_fixed(slot)

    def _zero_fixed(self, slot: int) -> None:
        for s, kind in enumerate(self._kinds):
            if kind is not None and not kind.paged:
                self.storage[s][slot].zero_()

    def forget(self, request) -> None:
        """The native side has released `request` (finished or preempted): drop it here."""
        self._key.pop(request, None)

    def pages_needed(self, request, n_new: int) -> list[int]:
        """Pages each group must still take so the request can hold `n_new` more tokens."""
        self._lib.kf_cache_pages_needed(self._h, self.key_of(request), int(n_new), self._scratch)
        return list(self._scratch[:len(self.groups)])

    def can_reserve(self, request, n_new: int) -> bool:
        if self.length(request) + n_new > self.max_context:      # (reservations in flight are counted natively)
            return False
        return all(n <= g.pool.n_free for n, g in zip(self.pages_needed(request, n_new), self.groups))

    def reserve(self, request, n_new: int) -> None:
        """Take the pages for `n_new` more tokens in every group, or none at all (raises OutOfPages)."""
        rc = self._lib.kf_cache_reserve(self._h, self.key_of(request), int(n_new))
        if rc == _E_CONTEXT:
            raise OutOfPages(f"request {request!r} would exceed the context of {self.max_context} tokens")
        if rc == _E_OUT_OF_PAGES:
            raise OutOfPages(f"request {request!r}: {self.pages_needed(request, n_new)} pages needed, {self.free_pages()} free")
        if rc != _OK:
            raise CacheError(f"reserve for {request!r} failed (code {rc})")

    def cancel_reservation(self, request) -> None:
        """Give back the pages taken for tokens that were reserved but never committed."""
        if self._lib.kf_cache_cancel_reservation(self._h, self.key_of(request)) != _OK:
            raise CacheError(f"cancel_reservation for {request!r} failed")

    def commit(self, request, n_new: int) -> None:
        """The step that wrote `n_new` reserved tokens succeeded: advance, and give back slid-out pages."""
        rc = self._lib.kf_cache_commit(self._h, self.key_of(request), int(n_new))
        if rc == _E_COMMIT:
            raise CacheError(f"commit of {n_new} tokens for {request!r}: more than were reserved")
        if rc != _OK:
            raise CacheError(f"commit for {request!r} failed (code {rc})")

    def release(self, request) -> None:
        """The request is finished (or preempted): everything it holds goes back."""
        rc = self._lib.kf_cache_release(self._h, self.key_of(request))
        del self._key[request]
        if rc != _OK:
            raise CacheError(f"release of {request!r} failed (code {rc})")

    # ---- what a step needs ----------------------------------------------------------------------------
    def block_table(self, group: int, request) -> list[int]:
        buf = (ctypes.c_int * self.table_width)()
        n = self._lib.kf_cache_table(self._h, group, self.key_of(request), buf, self.table_width)
        return list(buf[:n])

    def table_rows(self, group: int, state_slots) -> np.ndarray:
        """Block-table rows (full width, -1 where no page is held) of the requests in the given state slots."""
        return self._table_np[group][state_slots]

    def group_of(self, cache_slot: int) -> int | None:
        return self._group_of_slot.get(cache_slot)

    def view(self, cache_slot: int, writes: bool):
        need, kind = self.needs[cache_slot], self._kinds[cache_slot]
        if kind is None:
            return None
        if kind.paged:
            return kind.view(self.storage[cache_slot], self.page_size, self._group_of_slot[cache_slot], writes, need)
        return kind.view(self.storage[cache_slot], writes, need)

    # ---- accounting and self-check -----------------------------------------------------------------------
    def free_pages(self) -> list[int]:
        return [g.pool.n_free for g in self.groups]

    def pages_handed_out(self) -> list[int]:
        """Per group, how many pages the pool has handed out so far; more than the pool holds means pages were given
        back and used again."""
        return [int(self._lib.kf_cache_pool_n_taken(self._h, g)) for g in range(len(self.groups))]

    def bytes_per_token(self) -> int:
        """Bytes one token adds over all paged cache slots (windowed slots included, as long as it is in reach)."""
        n = 0
        for s, (need, kind) in enumerate(zip(self.needs, self._kinds)):
            if kind is not None and kind.paged:
                n += kind.page_bytes(need, self.page_size, self.storage[s].element_size()) // self.page_size
        return n

    def storage_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.storage.values())

    def check(self) -> None:
        """Every page is either free or in exactly one table; raises CacheError otherwise."""
        if self._lib.kf_cache_check(self._h) != _OK:
            raise CacheError("page accounting is inconsistent: a page is lost, held twice, or a table entry is stale")
