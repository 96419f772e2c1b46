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
by admitting and releasing requests.  The decisions themselves are native code (see `Scheduler`).
"""
from __future__ import annotations

import ctypes
from collections import deque
from dataclasses import dataclass, field
from typing import Hashable

from ..sampling.sampler import Sampling

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
    sampler_epoch: int = -1            # the admission (count of preemptions) for which the device holds its sampler state

    def __post_init__(self):
        self.prompt = [int(t) for t in self.prompt]

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
    """The decisions are taken by the native scheduler (`kungfu_b200/csrc/host_runtime.cpp`, which also owns the page
    accounting it reads); this class keeps the `Request` objects (token values, sampling state) in step with it and
    offers the queues as lists of those objects."""

    _FINISH = {1: "eos", 2: "length", 3: "context"}

    def __init__(self, cache, *, max_batch_tokens: int = 512, max_requests: int | None = None, pad_decode_rows: bool = False):
        self.cache = cache
        self.max_batch_tokens = int(max_batch_tokens)
        self.max_requests = int(max_requests if max_requests is not None else cache.max_requests)
        self.waiting: deque[Request] = deque()
        self.running: list[Request] = []          # in order of admission
        self.finished: list[Request] = []
        self._lib = cache._lib
        self._h = ctypes.c_void_p(self._lib.kf_sched_create(cache._h, self.max_batch_tokens, self.max_requests))
        # decode rows count as their next power of two: what a step function that replays captured graphs pads them to, so
        # that a step's rows (decode + prompt) stay within the budget and its products within the budget's tiles
        self.pad_decode_rows = bool(pad_decode_rows)
        self._lib.kf_sched_pad_decode_rows(self._h, int(self.pad_decode_rows))
        self._by_key: dict[int, Request] = {}
        self._key_of: dict[int, int] = {}         # id(request object) -> key
        cap = 4 * (self.max_requests + 8)
        self._portions = (ctypes.c_int64 * (4 * cap))()
        self._events = (ctypes.c_int64 * (3 * 4 * cap))()
        self._cap_portions, self._cap_events = cap, 4 * cap
        self._counts = (ctypes.c_int * 2)()
        self._state = (ctypes.c_int * 4)()

    def __del__(self):
        if getattr(self, "_h", None) and getattr(self.cache, "_h", None):
            self._lib.kf_sched_destroy(self._h)
        self._h = None

    # ---- queue ---------------------------------------------------------------------------------------
    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError(f"request {req.id!r} has an empty prompt")
        key = self.cache.new_key()
        if self._lib.kf_sched_add(self._h, key, len(req.prompt), len(req.output), int(req.max_tokens)) != 0:
            raise ValueError(f"request {req.id!r} is already known to the scheduler")
        req.status = WAITING
        self._by_key[key] = req
        self._key_of[id(req)] = key
        self.waiting.append(req)

    def adopt(self, req: Request) -> None:
        """A request whose prompt (all but `n_pending` tokens) the caller has already put into the cache under
        `req.id`: it joins the running requests as it is (measurement set-ups use this to start at a long context)."""
        key = self.cache.key_of(req.id)
        if self._lib.kf_sched_adopt(self._h, key, len(req.prompt), len(req.output), int(req.n_cached), int(req.max_tokens)) != 0:
            raise ValueError(f"request {req.id!r} cannot be adopted: it must be live in the cache and new to the scheduler")
        req.status = RUNNING
        self._by_key[key] = req
        self._key_of[id(req)] = key
        self.running.append(req)

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running

    @property
    def n_preemptions(self) -> int:
        return int(self._lib.kf_sched_n_preemptions(self._h))

    def _key(self, req: Request) -> int:
        try:
            return self._key_of[id(req)]
        except KeyError:
            raise ValueError(f"request {req.id!r} is not known to the scheduler") from None

    def _sync(self) -> None:
        """Bring the lists and the requests' counters in line with the native state."""
        nw, nr = ctypes.c_int(0), ctypes.c_int(0)
        self._lib.kf_sched_counts(self._h, ctypes.byref(nw), ctypes.byref(nr))
        w = (ctypes.c_int64 * max(nw.value, 1))()
        r = (ctypes.c_int64 * max(nr.value, 1))()
        self._lib.kf_sched_lists(self._h, w, r)
        self.waiting = deque(self._by_key[k] for k in w[:nw.value])
        self.running = [self._by_key[k] for k in r[:nr.value]]

    def _apply_events(self, n_events: int) -> None:
        for i in range(n_events):
            code, key, arg = self._events[3 * i], self._events[3 * i + 1], self._events[3 * i + 2]
            req = self._by_key[key]
            if code == 1:                                   # admitted: the native cache gave it a state slot
                self.cache.adopt(req.id, key, int(arg))
                req.status = RUNNING
            elif code == 2:                                 # preempted: everything given back, to be recomputed
                self.cache.forget(req.id)
                req.status = WAITING
                req.n_cached = 0
                req.n_preempted += 1
            elif code == 3:                                 # cannot fit even alone
                self._retire(req, key, "no_fit")

    def _retire(self, req: Request, key: int, reason: str) -> None:
        req.finish_reason = reason
        req.status = FINISHED
        if req.id in self.cache and self.cache.key_of(req.id) == key:
            self.cache.forget(req.id)
        self.finished.append(req)
        self._lib.kf_sched_forget(self._h, key)
        del self._by_key[key]
        del self._key_of[id(req)]

    # ---- decisions ---------------------------------------------------------------------------------------
    def preempt_last(self, keep: Request | None = None) -> Request | None:
        """Take the most recently admitted running request (other than `keep`) out, to be recomputed later."""
        key = self._lib.kf_sched_preempt_last(self._h, self._key(keep) if keep is not None else 0)
        if key == 0:
            return None
        req = self._by_key[key]
        self.cache.forget(req.id)
        req.status = WAITING
        req.n_cached = 0
        req.n_preempted += 1
        self._sync()
        return req

    def finish(self, req: Request, reason: str) -> None:
        key = self._key(req)
        self._lib.kf_sched_finish(self._h, key)
        self._retire(req, key, reason)
        self._sync()

    def schedule(self) -> list[Portion]:
        """Plan one step.  Returns the portions to run (possibly none if nothing can run right now)."""
        rc = self._lib.kf_sched_schedule(self._h, self._portions, self._cap_portions, self._events, self._cap_events, self._counts)
        if rc != 0:
            raise RuntimeError(f"the native scheduler returned more portions or events than fit ({self._counts[0]}, {self._counts[1]})")
        n_portions, n_events = self._counts[0], self._counts[1]
        if n_events:
            self._apply_events(n_events)
            self._sync()
        plan = []
        for i in range(n_portions):
            key, start, n, wants = self._portions[4 * i:4 * i + 4]
            plan.append(Portion(self._by_key[key], int(start), int(n), bool(wants)))
        return plan

    # ---- after the step ------------------------------------------------------------------------------------
    def advance(self, portion: Portion) -> None:
        portion.request.n_cached += portion.n
        self._lib.kf_sched_advance(self._h, self._key(portion.request), int(portion.n))

    def on_token(self, req: Request, token: int) -> str | None:
        """Record a sampled token; returns the finish reason if the request is done (and frees it)."""
        req.output.append(int(token))
        key = self._key(req)
        is_eos = (not req.ignore_eos) and int(token) in req.eos
        code = self._lib.kf_sched_on_token(self._h, key, int(is_eos))
        if code <= 0:
            return None
        reason = self._FINISH[code]
        self._retire(req, key, reason)
        self.running = [r for r in self.running if r is not req]
        return reason

    def on_token_pending(self, req: Request) -> str | None:
        """Count a token that a step has produced but the host has not read yet: a placeholder takes its place in
        `req.output` (the caller puts the value there later), and the request is retired if the count alone ends it
        (length, context).  Whether the token ends the request by its value is for the caller to see when it arrives."""
        req.output.append(0)
        key = self._key(req)
        code = self._lib.kf_sched_on_token(self._h, key, 0)
        if code <= 0:
            return None
        reason = self._FINISH[code]
        self._retire(req, key, reason)
        self.running = [r for r in self.running if r is not req]
        return reason
