"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes, finishes, frees.

The reference's loop is admit -> one prefill chunk -> sample -> one decode pass -> retire
(crates/kf-serve/src/engine.rs:396-430, admit :505-552, prefill_chunk :555-622, step :1041-1070, retire
:1144-1191); its prompt rows and decode rows never share a pass.  Here one `schedule()` call plans one mixed step:

1. every request that is decoding gets its one token;
2. the rest of the token budget goes to prompt portions, requests in order of admission, a portion being
   whatever still fits (any size >= 1);
3. waiting requests are admitted, first come first served, while a state slot is free and the pages for
   their whole pending prompt are free now (so that half-fed prompts cannot starve one another); no request
   is admitted in a step that had to preempt.

When pages run out: a decoding request that cannot get its next page makes the scheduler preempt the request
admitted last (it gives back everything and returns to the front of the waiting queue with the tokens it has
produced so far, to be recomputed); prompt portions are simply shortened or postponed.  A request that could
not fit even with the whole pool to itself is failed with reason `no_fit` (the reference refuses such a
context at plan time, crates/kf-engine/src/plan.rs:213-215).

The scheduler only decides; it reads page accounting from the cache manager and changes nothing there except
through `add_request`/`release`.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Hashable

from ..sampling.sampler import Rng, Sampling

WAITING, RUNNING, FINISHED = "waiting", "running", "finished"


@dataclass
class Request:
    id: Hashable
    prompt: list
    sampling: Sampling = field(default_factory=Sampling)
    max_tokens: int = 64
    eos: tuple = ()
    ignore_eos: bool = False
    seed: int = 42
    # state
    status: str = WAITING
    output: list = field(default_factory=list)
    n_cached: int = 0                  # tokens of `tokens()` whose keys/values are in the cache
    finish_reason: str | None = None
    n_preempted: int = 0
    rng: Rng | None = None

    def __post_init__(self):
        self.prompt = [int(t) for t in self.prompt]
        if self.rng is None:
            self.rng = Rng(self.seed)

    def tokens(self) -> list:
        return self.prompt + self.output

    def slice(self, start: int, n: int) -> list:
        """tokens()[start:start+n] without building the whole list."""
        np_ = len(self.prompt)
        if start + n <= np_:
            return self.prompt[start:start + n]
        if start >= np_:
            return self.output[start - np_:start - np_ + n]
        return self.prompt[start:] + self.output[:start + n - np_]

    @property
    def n_pending(self) -> int:
        """Tokens not yet run through the model."""
        return len(self.prompt) + len(self.output) - self.n_cached

    @property
    def decoding(self) -> bool:
        return self.status == RUNNING and self.n_pending == 1 and len(self.output) > 0


@dataclass
class Portion:
    request: Request
    start: int                         # index into request.tokens()
    n: int
    wants_logits: bool                 # the portion ends at the request's last pending token


class Scheduler:
    def __init__(self, cache, *, max_batch_tokens: int = 512, max_requests: int | None = None):
        self.cache = cache
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_requests = int(max_requests if max_requests is not None else cache.max_requests)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []          # in order of admission
        self.finished: list[Request] = []
        self.n_preemptions = 0

    # ---- queue ---------------------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError(f"request {req.id!r} has an empty prompt")
        req.status = WAITING
        self.waiting.append(req)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    # ---- page arithmetic --------------------------------------------------------------------------------
    def _pages_for(self, req: Request, n_new: int, live: bool) -> list[int]:
        if live:
            return self.cache.pages_needed(req.id, n_new)
        want = -(-n_new // self.cache.page_size)
        return [want for _ in self.cache.groups]

    def _fits_at_all(self, req: Request) -> bool:
        """Could the request run with the whole pool to itself?  Worst case per group: its full length, or for a
        windowed group the window plus one portion."""
        total = len(req.prompt) + req.max_tokens
        if total > self.cache.max_context:
            total = self.cache.max_context
        if len(req.prompt) >= self.cache.max_context:
            return False
        P = self.cache.page_size
        for g in self.cache.groups:
            need = total
            if g.window is not None:
                need = min(total, g.window + P + min(self.max_batch_tokens, len(req.prompt)))
            if -(-need // P) > g.pool.n_pages:
                return False
        return True

    def _admission_pages(self, req: Request) -> list[int]:
        """Pages per group that must be free to admit `req`: its whole pending prompt (a windowed group never
        holds more than the window, a page of slack and one portion)."""
        P = self.cache.page_size
        out = []
        for g in self.cache.groups:
            need = req.n_pending
            if g.window is not None:
                need = min(need, g.window + P + min(self.max_batch_tokens, req.n_pending))
            out.append(-(-need // P))
        return out

    # ---- decisions ---------------------------------------------------------------------------------------
    def preempt_last(self, keep: Request | None = None) -> Request | None:
        """Take the most recently admitted running request (other than `keep`) out, to be recomputed later."""
        for req in reversed(self.running):
            if req is keep:
                continue
            self.running.remove(req)
            self.cache.release(req.id)
            req.status = WAITING
            req.n_cached = 0
            req.n_preempted += 1
            self.n_preemptions += 1
            self.waiting.appendleft(req)
            return req
        return None

    def finish(self, req: Request, reason: str) -> None:
        req.finish_reason = reason
        req.status = FINISHED
        if req in self.running:
            self.running.remove(req)
            self.cache.release(req.id)
        elif req in self.waiting:
            self.waiting.remove(req)
        self.finished.append(req)

    def schedule(self) -> list[Portion]:
        """Plan one step.  Returns the portions to run (possibly none if nothing can run right now)."""
        free = list(self.cache.free_pages())
        budget = self.max_batch_tokens
        plan: list[Portion] = []
        preempted = False

        def take(need: list[int]) -> bool:
            if any(n > f for n, f in zip(need, free)):
                return False
            for i, n in enumerate(need):
                free[i] -= n
            return True

        # 1. decoding requests, oldest first; out of pages -> preempt the youngest and try again
        i = 0
        while i < len(self.running):
            req = self.running[i]
            if not req.decoding:
                i += 1
                continue
            if budget <= 0:
                break
            need = self.cache.pages_needed(req.id, 1)
            if take(need):
                plan.append(Portion(req, req.n_cached, 1, True))
                budget -= 1
                i += 1
                continue
            victim = self.preempt_last(keep=req)
            if victim is None:
                # alone and still no page: the pool cannot hold this request
                self.finish(req, "no_fit")
                continue
            preempted = True
            planned = [p for p in plan if p.request is victim]
            for p in planned:                       # it had been planned in this very call: undo
                plan.remove(p)
                budget += p.n
            free = list(self.cache.free_pages())
            for p in plan:                          # re-apply what is already planned
                for gi, n in enumerate(self.cache.pages_needed(p.request.id, p.n)):
                    free[gi] -= n
            # `i` stays: retry the same request (the victim sat after it or before it in the list)
            i = self.running.index(req)

        # 2. prompt portions of running requests, in order of admission
        for req in self.running:
            if budget <= 0:
                break
            if req.decoding or req.n_pending == 0 or any(p.request is req for p in plan):
                continue
            n = self._largest_portion(req, min(budget, req.n_pending), free, live=True)
            if n <= 0:
                continue
            take(self.cache.pages_needed(req.id, n))
            plan.append(Portion(req, req.n_cached, n, n == req.n_pending))
            budget -= n

        # 3. admission, first come first served
        while self.waiting and budget > 0 and len(self.running) < self.max_requests:
            req = self.waiting[0]
            if not self._fits_at_all(req):
                self.waiting.popleft()
                self.finish(req, "no_fit")
                continue
            if preempted or any(a > b for a, b in zip(self._admission_pages(req), free)):
                break
            n = min(budget, req.n_pending)
            self.waiting.popleft()
            self.cache.add_request(req.id)
            req.status = RUNNING
            self.running.append(req)
            take(self._pages_for(req, n, live=True))
            plan.append(Portion(req, 0, n, n == req.n_pending))
            budget -= n

        if not plan and self.running and not any(r.decoding for r in self.running):
            # every running request is mid-prompt and none can get a page: free the youngest so the oldest moves
            if len(self.running) > 1:
                self.preempt_last(keep=self.running[0])
                return self.schedule()
            self.finish(self.running[0], "no_fit")
        return plan

    def _largest_portion(self, req: Request, n_max: int, free: list[int], live: bool) -> int:
        """The most tokens (<= n_max) whose pages the free counts still cover."""
        P = self.cache.page_size
        n = n_max
        while n > 0:
            need = self._pages_for(req, n, live)
            if all(a <= b for a, b in zip(need, free)):
                return n
            # drop to the largest count that needs one page fewer in the tightest group
            have = (self.cache.length(req.id) if live else 0)
            n = min(n - 1, ((have + n - 1) // P) * P - have)
        return 0

    # ---- after the step ------------------------------------------------------------------------------------
    def advance(self, portion: Portion) -> None:
        portion.request.n_cached += portion.n

    def on_token(self, req: Request, token: int) -> str | None:
        """Record a sampled token; returns the finish reason if the request is done (and frees it)."""
        req.output.append(int(token))
        reason = None
        if not req.ignore_eos and int(token) in req.eos:
            reason = "eos"
        elif len(req.output) >= req.max_tokens:
            reason = "length"
        elif len(req.prompt) + len(req.output) >= self.cache.max_context:
            reason = "context"
        if reason is not None:
            self.finish(req, reason)
        return reason
