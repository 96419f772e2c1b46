"""Sizing the cache pools: how many pages each group gets, from what its requests can ever hold and from the
memory that is left after the weights.

The reference sizes each layer's ring at plan time: `n_ctx` rows for layers that see everything, `window + n_batch`
rows for sliding layers (crates/kf-core/src/plan.rs:59-64), and refuses (`no_fit`) or shrinks the context when the
device cannot hold it (crates/kf-engine/src/plan.rs:199-228,319-343).  With pages the same two rules read:

* a request can hold at most `ctx` tokens in a group without a window, and at most `window + batch + page` tokens in
  a windowed group (the keys the earliest row of its next portion still reads, the portion itself, and one page of
  slack because pages are given back whole); a pool never needs more than `parallel` times that;
* the pools of all groups together must fit the memory budget; if they do not, every group is cut by the same
  factor, but never below what ONE request of full context needs (below that nothing can run: `NoFit`).

The plan is data (`CachePlan`), printed as a `plan` event by the engine and turned into storage by `CacheManager`.
"""
from __future__ import annotations

from dataclasses import dataclass, field


class NoFit(RuntimeError):
    """The cache for even one request of the asked context does not fit the memory budget."""


@dataclass
class GroupPlan:
    window: int | None
    tokens_per_request: int          # the most tokens one request can hold in this group
    pages: int                       # pages in the group's pool
    bytes_per_page: int              # summed over the cache slots of the group
    slots: list = field(default_factory=list)


@dataclass
class CachePlan:
    page_size: int
    parallel: int
    ctx: int
    batch: int
    groups: list                     # GroupPlan per group, in the order the manager creates them
    fixed_bytes: int                 # fixed-size state of all slots, for `parallel` requests
    budget_bytes: int | None
    shrunk: bool = False

    @property
    def paged_bytes(self) -> int:
        return sum(g.pages * g.bytes_per_page for g in self.groups)

    @property
    def total_bytes(self) -> int:
        return self.paged_bytes + self.fixed_bytes

    def pages_by_window(self) -> dict:
        return {g.window: g.pages for g in self.groups}

    def fields(self) -> dict:
        """Flat key/values for the `plan` event line."""
        out = {"page_size": self.page_size, "parallel": self.parallel, "ctx": self.ctx, "batch": self.batch,
               "cache_bytes": self.total_bytes, "budget_bytes": self.budget_bytes if self.budget_bytes is not None else "none",
               "shrunk": int(self.shrunk)}
        for i, g in enumerate(self.groups):
            out[f"group{i}"] = f"window:{g.window if g.window is not None else 'none'},pages:{g.pages},tokens_per_request:{g.tokens_per_request},slots:{len(g.slots)}"
        return out


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def plan_cache(needs: list, *, page_size: int, parallel: int, ctx: int, batch: int, element_size: int,
               budget_bytes: int | None = None, pool_tokens: int | None = None) -> CachePlan:
    """`needs[s]`: the state need of cache slot s (or None).  `pool_tokens`, when given, replaces `parallel * ctx` as
    the size of a group without a window (a caller that knows its requests are short).  `budget_bytes`: what the
    cache may take (None: no limit)."""
    from .kinds import kind_of
    groups: dict = {}
    order: list = []
    fixed = 0
    for s, need in enumerate(needs):
        if need is None:
            continue
        kind = kind_of(need)
        if not kind.paged:
            fixed += parallel * kind.fixed_bytes(need)
            continue
        window = kind.window(need)
        g = groups.get(window)
        if g is None:
            if window is None:
                per_req = _ceil_div(ctx, page_size) * page_size
            else:
                per_req = min(_ceil_div(ctx, page_size) * page_size,
                              _ceil_div(window + min(batch, ctx) + page_size, page_size) * page_size)
            g = groups[window] = GroupPlan(window, per_req, 0, 0)
            order.append(window)
        g.slots.append(s)
        g.bytes_per_page += kind.page_bytes(need, page_size, element_size)
    full_tokens = pool_tokens if pool_tokens is not None else parallel * _ceil_div(ctx, page_size) * page_size
    for g in groups.values():
        want = parallel * g.tokens_per_request
        g.pages = _ceil_div(min(want, full_tokens), page_size)
    plan = CachePlan(page_size, parallel, ctx, batch, [groups[w] for w in order], fixed, budget_bytes)
    if budget_bytes is not None and plan.total_bytes > budget_bytes:
        floor = sum(_ceil_div(g.tokens_per_request, page_size) * g.bytes_per_page for g in plan.groups) + fixed
        if floor > budget_bytes:
            raise NoFit(f"no_fit: the cache of one request of {ctx} tokens needs {floor} bytes, {budget_bytes} are left "
                        f"after the weights")
        factor = (budget_bytes - fixed) / max(plan.paged_bytes, 1)
        for g in plan.groups:
            g.pages = max(_ceil_div(g.tokens_per_request, page_size), int(g.pages * factor))
        while plan.total_bytes > budget_bytes:                       # the floors may have pushed it over again
            big = max(plan.groups, key=lambda g: g.pages - _ceil_div(g.tokens_per_request, page_size))
            if big.pages <= _ceil_div(big.tokens_per_request, page_size):
                raise NoFit(f"no_fit: the cache does not fit {budget_bytes} bytes")
            big.pages -= 1
        plan.shrunk = True
    return plan
