"""The cache manager and the scheduler's decisions, on the host only."""
import random

import pytest
import torch

from kungfu_b200.cache import CacheError, CacheManager, OutOfPages, PagePool
from kungfu_b200.engine.scheduler import Request, Scheduler
from kungfu_b200.parts import FixedState, PagedKV
from kungfu_b200.sampling import Sampling


def make_cache(n_pages=16, page=4, window=8, max_requests=4, max_context=64, n_pages_windowed=None, state=True):
    needs = [PagedKV(2, 8, window), PagedKV(2, 8, None), PagedKV(1, 16, window), PagedKV(2, 8, None)]
    if state:
        needs.append(FixedState((3,), torch.float32))
    return CacheManager(needs, page_size=page, n_pages=n_pages, max_requests=max_requests, max_context=max_context,
                        dtype=torch.float32, device="cpu", n_pages_windowed=n_pages_windowed)


def test_pool_refuses_double_free():
    pool = PagePool(3)
    a, b = pool.take(), pool.take()
    pool.give_back(a)
    with pytest.raises(CacheError):
        pool.give_back(a)
    with pytest.raises(CacheError):
        pool.give_back(2)                 # never handed out
    pool.take(), pool.take()
    with pytest.raises(OutOfPages):
        pool.take()
    assert b == 1


def test_groups_follow_the_needs():
    c = make_cache()
    assert [g.window for g in c.groups] == [8, None]
    assert [g.slots for g in c.groups] == [[0, 2], [1, 3]]
    assert c.storage[2].shape == (16, 2, 1, 4, 16) and c.storage[4].shape == (4, 3)
    assert c.view(0, True).group == 0 and c.view(3, False).group == 1 and c.view(4, True).state.shape == (4, 3)


def test_window_pages_go_back_and_tables_keep_absolute_index():
    c = make_cache(n_pages=16, page=4, window=8)
    c.add_request("a")
    c.reserve("a", 10)
    c.commit("a", 10)                    # next query at 10 reads keys >= 3: page 0 (positions 0..3) still holds 3
    assert c.block_table(0, "a")[0] >= 0
    c.reserve("a", 1)
    c.commit("a", 1)                     # next query at 11 reads keys >= 4: page 0 is dead
    assert c.block_table(0, "a")[0] == -1 and c.block_table(0, "a")[1] >= 0
    assert c.block_table(1, "a")[0] >= 0           # the group without a window keeps everything
    assert c.free_pages() == [16 - 2, 16 - 3]
    c.check()
    c.release("a")
    assert c.free_pages() == [16, 16]
    with pytest.raises(CacheError):
        c.release("a")


def test_reserve_is_all_or_nothing_and_cancel_gives_back():
    c = make_cache(n_pages=4, page=4, window=None)
    c.add_request("a")
    c.add_request("b")
    c.reserve("a", 9)                    # 3 pages in the single group
    with pytest.raises(OutOfPages):
        c.reserve("b", 5)                # needs 2, only 1 free
    assert c.free_pages() == [1] and c.block_table(0, "b") == []
    c.reserve("b", 4)
    c.cancel_reservation("b")
    assert c.free_pages() == [1]
    c.cancel_reservation("a")
    assert c.free_pages() == [4]
    with pytest.raises(OutOfPages):
        c.reserve("a", 65)               # beyond the context
    c.check()


def test_state_slots_are_zeroed_and_reused():
    c = make_cache()
    s = c.add_request("a")
    c.storage[4][s] = 5.0
    c.release("a")
    assert c.add_request("b") == s and float(c.storage[4][s].abs().sum()) == 0.0
    for r in ("c", "d", "e"):
        c.add_request(r)
    with pytest.raises(CacheError):
        c.add_request("f")               # more live requests than state slots


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    c = make_cache(n_pages=12, page=4, window=8, max_requests=4, max_context=40)
    live = {}
    for step in range(400):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{step}"
            c.add_request(rid)
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 2, 3, 7])
            try:
                c.reserve(rid, n)
            except OutOfPages:
                assert not c.can_reserve(rid, n)
            else:
                if rng.random() < 0.1:
                    c.cancel_reservation(rid)
                else:
                    c.commit(rid, n)
                    live[rid] += n
                    assert c.length(rid) == live[rid]
                    # every position a later query may read still has a page
                    for g in c.groups:
                        lo = 0 if g.window is None else max(0, live[rid] - g.window + 1)
                        tab = g.tables[rid]
                        assert all(tab[p // 4] >= 0 for p in range(lo, live[rid]))
        elif live:
            rid = rng.choice(list(live))
            c.release(rid)
            del live[rid]
        c.check()
    for rid in list(live):
        c.release(rid)
    assert c.free_pages() == [12, 12] and c.n_live == 0


# ---- scheduler ---------------------------------------------------------------------------------------------

def greedy():
    return Sampling(temperature=0.0)


def run_plan(s, plan, token=7):
    """Pretend the step ran: reserve+commit pages, advance, produce a token where logits were wanted."""
    out = []
    for p in plan:
        s.cache.reserve(p.request.id, p.n)
        s.cache.commit(p.request.id, p.n)
        s.advance(p)
    for p in plan:
        if p.wants_logits:
            out.append((p.request.id, s.on_token(p.request, token)))
    s.cache.check()
    return out


def test_budget_cuts_prompts_and_decodes_first():
    c = make_cache(n_pages=64, page=4, window=8, max_context=200)
    s = Scheduler(c, max_batch_tokens=16, max_requests=4)
    s.add(Request("a", list(range(20)), greedy(), max_tokens=3))
    s.add(Request("b", list(range(30)), greedy(), max_tokens=3))
    p1 = s.schedule()
    assert [(p.request.id, p.start, p.n, p.wants_logits) for p in p1] == [("a", 0, 16, False)]
    run_plan(s, p1)
    p2 = s.schedule()
    assert [(p.request.id, p.start, p.n, p.wants_logits) for p in p2] == [("a", 16, 4, True), ("b", 0, 12, False)]
    run_plan(s, p2)
    p3 = s.schedule()                    # a decodes (1 token) before b gets the rest of the budget
    assert [(p.request.id, p.start, p.n, p.wants_logits) for p in p3] == [("a", 20, 1, True), ("b", 12, 15, False)]
    run_plan(s, p3)
    p4 = s.schedule()
    assert [(p.request.id, p.n, p.wants_logits) for p in p4] == [("a", 1, True), ("b", 3, True)]
    assert run_plan(s, p4) == [("a", "length"), ("b", None)]
    assert "a" not in c and s.finished[0].id == "a"
    while not s.idle:
        run_plan(s, s.schedule())
    assert c.free_pages() == [64, 64] and [r.finish_reason for r in s.finished] == ["length", "length"]


@pytest.mark.parametrize("n_short,padded", [(1, 1), (3, 4), (4, 4), (5, 8)])
def test_padded_decode_rows_count_as_their_power_of_two(n_short, padded):
    """A step function that replays captured graphs pads a step's decode rows to a power of two; a scheduler told so
    (`pad_decode_rows`) leaves that many rows out of the prompts' budget, so that decode and prompt rows together are the
    budget: three decoding requests cost four rows, five cost eight."""
    for pad in (False, True):
        c = make_cache(n_pages=256, page=4, window=8, max_requests=8, max_context=400)
        s = Scheduler(c, max_batch_tokens=32, max_requests=8, pad_decode_rows=pad)
        for k in range(n_short):
            s.add(Request(f"s{k}", [1, 2, 3], greedy(), max_tokens=50))
        run_plan(s, s.schedule())                       # the short prompts; from now on they decode
        s.add(Request("long", list(range(200)), greedy(), max_tokens=2))
        for _ in range(3):
            plan = s.schedule()
            got = [(p.request.id, p.n) for p in plan]
            assert got[:n_short] == [(f"s{k}", 1) for k in range(n_short)]
            assert got[n_short:] == [("long", 32 - (padded if pad else n_short))], (pad, got)
            run_plan(s, plan)


def test_padding_never_starves_prompts():
    """Five decoding requests under a budget of 8 would be padded to 8 rows and leave nothing: padding then stands back."""
    c = make_cache(n_pages=256, page=4, window=8, max_requests=8, max_context=400)
    s = Scheduler(c, max_batch_tokens=8, max_requests=8, pad_decode_rows=True)
    for k in range(5):
        s.add(Request(f"s{k}", [1, 2], greedy(), max_tokens=50))
    run_plan(s, s.schedule())
    run_plan(s, s.schedule())
    run_plan(s, s.schedule())                           # all five decode by now
    s.add(Request("long", list(range(100)), greedy(), max_tokens=2))
    plan = s.schedule()
    assert [(p.request.id, p.n) for p in plan][-1] == ("long", 3)


def test_admission_waits_for_slots_and_pages():
    c = make_cache(n_pages=6, page=4, window=None, max_requests=2, max_context=64, state=False)
    s = Scheduler(c, max_batch_tokens=64, max_requests=2)
    for rid, n in (("a", 10), ("b", 10), ("c", 4)):
        s.add(Request(rid, list(range(n)), greedy(), max_tokens=2))
    plan = s.schedule()
    assert [(p.request.id, p.n) for p in plan] == [("a", 10), ("b", 10)]     # 3 + 3 pages; c waits for a slot
    run_plan(s, plan)
    plan = s.schedule()                  # both decode at position 10: still inside their third page
    assert [(p.request.id, p.n) for p in plan] == [("a", 1), ("b", 1)]
    assert run_plan(s, plan) == [("a", "length"), ("b", "length")]
    plan = s.schedule()
    assert [(p.request.id, p.n) for p in plan] == [("c", 4)]


def test_out_of_pages_preempts_the_youngest_and_recomputes():
    c = make_cache(n_pages=4, page=4, window=None, max_requests=4, max_context=64, state=False)
    s = Scheduler(c, max_batch_tokens=64)
    s.add(Request("old", list(range(8)), greedy(), max_tokens=6))
    s.add(Request("young", list(range(7)), greedy(), max_tokens=6))
    run_plan(s, s.schedule())            # 2 + 2 pages: the pool is full; both produced their first token
    assert c.free_pages() == [0]
    plan = s.schedule()                  # old needs a third page -> young is preempted; young (8 tokens now) cannot come back yet
    assert [(p.request.id, p.n) for p in plan] == [("old", 1)] and s.n_preemptions == 1
    young = s.waiting[0]
    assert young.id == "young" and young.n_cached == 0 and young.tokens() == list(range(7)) + [7] and "young" not in c
    run_plan(s, plan)
    seen_young_again = False
    for _ in range(40):
        if s.idle:
            break
        plan = s.schedule()
        for p in plan:
            if p.request.id == "young" and p.start == 0:
                assert p.n == len(p.request.tokens()) and p.wants_logits      # recomputed whole, prompt + its own output
                seen_young_again = True
        run_plan(s, plan)
    assert s.idle and seen_young_again
    assert {r.id: r.finish_reason for r in s.finished} == {"old": "length", "young": "length"}
    assert len(s.finished[0].output) == 6 and len(young.output) == 6
    assert c.free_pages() == [4]


def test_a_request_that_can_never_fit_fails_with_no_fit():
    c = make_cache(n_pages=3, page=4, window=None, max_requests=2, max_context=64, state=False)
    s = Scheduler(c, max_batch_tokens=64)
    s.add(Request("big", list(range(20)), greedy(), max_tokens=4))
    s.add(Request("ok", list(range(5)), greedy(), max_tokens=2))
    plan = s.schedule()
    assert [p.request.id for p in plan] == ["ok"]
    assert s.finished[0].id == "big" and s.finished[0].finish_reason == "no_fit"


def test_eos_and_context_finish():
    c = make_cache(n_pages=32, page=4, window=None, max_context=12, state=False)
    s = Scheduler(c, max_batch_tokens=64)
    s.add(Request("e", [1, 2, 3], greedy(), max_tokens=50, eos=(7,)))
    s.add(Request("i", [1, 2, 3], greedy(), max_tokens=50, eos=(7,), ignore_eos=True))
    assert run_plan(s, s.schedule(), token=7) == [("e", "eos"), ("i", None)]
    reasons = []
    while not s.idle:
        reasons += [r for _, r in run_plan(s, s.schedule(), token=7) if r]
    assert reasons == ["context"] and len(s.finished[1].output) == 9


def test_adopted_request_decodes_from_where_its_cache_ends():
    """A request whose prompt the caller has put into the cache by hand joins the running requests as it is."""
    c = make_cache(n_pages=32, page=4, window=None, max_context=64, state=False)
    s = Scheduler(c, max_batch_tokens=64)
    c.add_request("r")
    c.reserve("r", 9)
    c.commit("r", 9)
    req = Request("r", list(range(10)), greedy(), max_tokens=3)
    req.n_cached = 9
    s.adopt(req)
    plan = s.schedule()
    assert [(p.request.id, p.start, p.n, p.wants_logits) for p in plan] == [("r", 9, 1, True)]
    assert run_plan(s, plan) == [("r", None)]
    while not s.idle:
        run_plan(s, s.schedule())
    assert req.finish_reason == "length" and len(req.output) == 3 and c.free_pages() == [32] and "r" not in c


# ---- sizing of the pools ------------------------------------------------------------------------------------------

def test_plan_gives_windowed_groups_only_what_they_can_hold():
    from kungfu_b200.cache.plan import NoFit, plan_cache
    from kungfu_b200.parts.base import FixedState, PagedKV
    # 4 cache slots: two windowed (window 4096), two global; 8 requests of 8192 tokens, portions of 512, pages of 64
    needs = [PagedKV(4, 256, 4096), PagedKV(4, 256, None), PagedKV(4, 256, 4096), PagedKV(4, 256, None), FixedState((10,), torch.float32)]
    plan = plan_cache(needs, page_size=64, parallel=8, ctx=8192, batch=512, element_size=2)
    by = plan.pages_by_window()
    assert by[None] == 8 * 8192 // 64
    assert by[4096] == 8 * (4096 + 512 + 64) // 64 and by[4096] < by[None]
    page_bytes = 2 * 4 * 64 * 256 * 2
    assert plan.paged_bytes == 2 * page_bytes * (by[None] + by[4096]) and plan.fixed_bytes == 8 * 40
    assert not plan.shrunk
    # a window as long as the context changes nothing
    same = plan_cache([PagedKV(4, 256, 8192), PagedKV(4, 256, None)], page_size=64, parallel=8, ctx=8192, batch=512, element_size=2)
    assert same.pages_by_window()[8192] == same.pages_by_window()[None]
    # a budget below the plan cuts every pool, never below one request's need
    small = plan_cache(needs, page_size=64, parallel=8, ctx=8192, batch=512, element_size=2, budget_bytes=plan.total_bytes // 2)
    assert small.shrunk and small.total_bytes <= plan.total_bytes // 2
    sb = small.pages_by_window()
    assert sb[None] >= 8192 // 64 and sb[4096] >= (4096 + 512 + 64) // 64 and sb[None] < by[None]
    with pytest.raises(NoFit, match="no_fit"):
        plan_cache(needs, page_size=64, parallel=8, ctx=8192, batch=512, element_size=2, budget_bytes=1 << 20)
    # an explicit pool size is taken as it is (replay makes pools so small that pages are used again)
    tiny = plan_cache(needs, page_size=64, parallel=8, ctx=8192, batch=8192, element_size=2, pool_tokens=640)
    assert tiny.pages_by_window() == {4096: 10, None: 10}
    fields = plan.fields()
    assert fields["group0"].startswith("window:4096,pages:") and fields["parallel"] == 8


def test_manager_takes_the_plans_pool_sizes_and_the_scheduler_lives_with_them():
    """Pools sized by the plan: the windowed group is smaller than the global one, and requests far longer than the
    window still run to their end because slid-out pages come back."""
    from kungfu_b200.cache.plan import plan_cache
    from kungfu_b200.parts.base import PagedKV
    needs = [PagedKV(1, 4, 8), PagedKV(1, 4, None)]
    plan = plan_cache(needs, page_size=4, parallel=2, ctx=64, batch=6, element_size=4)
    assert plan.pages_by_window() == {8: 2 * 5, None: 2 * 16}
    cache = CacheManager(needs, page_size=4, n_pages=plan.pages_by_window(), max_requests=2, max_context=64,
                         dtype=torch.float32, device="cpu")
    assert [g.pool.n_pages for g in cache.groups] == [10, 32]
    assert cache.storage[0].shape[0] == 10 and cache.storage[1].shape[0] == 32
    for rid in ("a", "b"):
        cache.add_request(rid)
    fed = {"a": 0, "b": 0}
    while min(fed.values()) < 64:
        for rid in ("a", "b"):
            n = min(6, 64 - fed[rid])
            if n:
                cache.reserve(rid, n)
                cache.commit(rid, n)
                fed[rid] += n
        cache.check()
    cache.release("a")
    cache.release("b")
    assert cache.free_pages() == [10, 32]
