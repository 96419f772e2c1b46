"""What the cache manager has to know about a kind of per-request state, registered per `StateNeed` class.

The reference's planner reads only a layer's `StateNeed` (crates/kf-core/src/layer.rs:29-43: `KvCache`, `Recurrent`,
`TokenShift`, `Latent`, ...) and never the layer type; each variant brings its own row width and lifetime.  Here a
state kind is an object with the few answers the manager and the sizing need, and a new kind is registered from
wherever its mixer is defined (a test file is enough): the manager has no list of kinds of its own.

A *paged* kind stores something for every token, in pages that the manager hands out; its answers:
  window(need)                          -> tokens that stay readable (None: all); needs with equal windows share a
                                           group, i.e. a pool of page ids and one block table per request
  page_shape(need, page_size)           -> shape of one page of one cache slot
  page_bytes(need, page_size, elsize)   -> its bytes (elsize: bytes of the cache's element type)
  dtype(need, cache_dtype)              -> element type of the storage
  view(storage, page_size, group, writes, need) -> what the mixer's forward() is given
A *fixed* kind stores one state of fixed shape per live request, zeroed at admission:
  shape(need), dtype(need, cache_dtype), fixed_bytes(need), view(storage, writes, need)
"""
from __future__ import annotations

import math

import torch

from ..parts.base import FixedState, PagedKV


class PagedKVView:
    """What a mixer sees of a cache slot of keys and values during one step."""

    def __init__(self, pages: torch.Tensor, page_size: int, group: int, writes: bool):
        self.pages = pages              # [n_pages, 2 (key, value), n_kv_heads, page_size, head_dim]
        self.page_size = page_size
        self.group = group
        self.writes = writes


class FixedStateView:
    def __init__(self, state: torch.Tensor, writes: bool):
        self.state = state              # [max_requests, *shape]; row = the request's state slot
        self.writes = writes


class PagedKVKind:
    paged = True

    def window(self, need):
        return need.window

    def page_shape(self, need, page_size):
        return (2, need.n_kv_heads, page_size, need.head_dim)

    def page_bytes(self, need, page_size, elsize):
        return 2 * need.n_kv_heads * page_size * need.head_dim * elsize

    def dtype(self, need, cache_dtype):
        return cache_dtype

    def view(self, storage, page_size, group, writes, need):
        return PagedKVView(storage, page_size, group, writes)


class FixedStateKind:
    paged = False

    def shape(self, need):
        return tuple(need.shape)

    def dtype(self, need, cache_dtype):
        return need.dtype

    def fixed_bytes(self, need):
        return int(math.prod(need.shape)) * torch.empty(0, dtype=need.dtype).element_size()

    def view(self, storage, writes, need):
        return FixedStateView(storage, writes)


_KINDS: dict = {}


def register_state_kind(need_class: type, kind) -> None:
    """Make the manager able to hold what `need_class` declares.  `kind` answers the questions in this module's
    header (see `PagedKVKind` and `FixedStateKind`)."""
    if need_class in _KINDS and type(_KINDS[need_class]) is not type(kind):
        raise ValueError(f"a state kind for {need_class.__name__} is already registered")
    _KINDS[need_class] = kind


def kind_of(need):
    for cls in type(need).__mro__:
        if cls in _KINDS:
            return _KINDS[cls]
    raise TypeError(f"unknown state need {need!r}: no state kind is registered for {type(need).__name__} "
                    f"(known: {sorted(c.__name__ for c in _KINDS)})")


register_state_kind(PagedKV, PagedKVKind())
register_state_kind(FixedState, FixedStateKind())
