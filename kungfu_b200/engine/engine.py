"""The engine a user drives: requests in (token ids), tokens out.

`Engine` wraps a model, a cache manager, the step runner, the scheduler and the sampler.  The reference's
counterpart is a `Session` under a `Scheduler` (crates/kf-engine/src/session.rs:84-103,
crates/kf-serve/src/engine.rs:375-430); its `generate` command is `Engine.generate` here
(crates/kungfu/src/main.rs:611-645: seed 42, greedy at temperature 0).
"""
from __future__ import annotations

import time
from typing import Hashable, Sequence

import numpy as np
import torch

from .. import events as _events
from .. import ops
from ..sampling.sampler import STATE_WORDS, Sampling, pack_state
from .scheduler import Request, Scheduler
from .step import Runner, StepEntry


def emit_event(name: str, **fields) -> None:
    """One structured line on stderr, `kungfu event=<name> k=v ...` (reference: crates/kf-core/src/event.rs:31-44)."""
    was, _events.enabled = _events.enabled, True
    try:
        _events.emit(name, **fields)
    finally:
        _events.enabled = was


class Engine:
    def __init__(self, model_dir: str | None = None, *, config=None, seed: int = 0, dtype="bfloat16", device="cuda:0",
                 ctx: int | str = 4096, batch: int = 512, parallel: int = 8, page_size: int | None = None,
                 max_tokens_in_cache: int | None = None, events: bool = False, runner: Runner | None = None,
                 cuda_graphs: bool = True, pipeline: bool = True):
        """`model_dir`: folder with config.json and model.safetensors; or `config` (typed configuration, dictionary
        or config.json path) with `seed` for random weights.  `ctx`: context length per request ('auto' = the
        model's trained length); `batch`: most tokens one step runs; `parallel`: most live requests.
        `max_tokens_in_cache`: size of a cache group's pool in tokens (default: parallel * ctx; a windowed group never
        gets more than parallel * (window + batch + page), and all pools are cut to fit the memory left after the weights).
        `pipeline`: decode steps are launched before the tokens of the step before them have been read (tokens are
        drawn on the device and stay there as the next step's input), so `step()` returns a step's tokens one call
        later and the GPU does not wait for the host between steps."""
        from .. import api
        self.events = events
        if runner is not None:
            self.runner = runner
            self.cfg = None
        else:
            self.device = api.require_cuda(device)
            ops.library()
            t0 = time.time()
            if model_dir is not None:
                self.cfg, model = api.load_model(model_dir, dtype=dtype, device=self.device)
            elif config is not None:
                self.cfg, model = api.random_model(config, seed, dtype=dtype, device=self.device)
            else:
                raise ValueError("Engine needs a model folder or a configuration")
            trained = getattr(self.cfg, "max_position_embeddings", 8192)
            n_ctx = trained if ctx == "auto" else min(int(ctx), trained) if ctx else trained
            page = page_size or api.DEFAULT_PAGE_SIZE
            if events:
                _events.enabled = True
            pool = f"cuda{self.device.index or 0}"
            _events.alloc(pool, "weights", model.weight_bytes())
            # what the cache may take: the memory that is free now, less a reserve for the step's own buffers
            # (activations of `batch` rows, logits of the wanted rows, split sums) and the allocator's slack
            free, total = torch.cuda.mem_get_info(self.device)
            budget = max(0, int(free) - max(2 << 30, int(total) // 16))
            self.runner = api.make_runner(self.cfg, model, dtype=dtype, device=self.device, page_size=page,
                                          max_tokens=max_tokens_in_cache, max_requests=parallel, max_context=n_ctx,
                                          cuda_graphs=cuda_graphs, batch=batch, budget_bytes=budget)
            plan = self.runner.cache.plan
            _events.emit("plan", **plan.fields())
            _events.alloc(pool, "cache", plan.paged_bytes)
            if plan.fixed_bytes:
                _events.alloc(pool, "state", plan.fixed_bytes)
            _events.emit("ready", model=self.cfg.architecture, dtype=str(api.parse_dtype(dtype)).split(".")[-1],
                         weight_bytes=model.weight_bytes(), cache_bytes_per_token=self.runner.cache.bytes_per_token(),
                         pool_pages=",".join(str(g.pages) for g in plan.groups), ctx=n_ctx,
                         load_s=f"{time.time() - t0:.2f}")
        self.scheduler = Scheduler(self.runner.cache, max_batch_tokens=batch, max_requests=parallel,
                                   pad_decode_rows=bool(getattr(self.runner, "cuda_graphs", False)))
        self._next_id = 0
        self.requests: dict[Hashable, Request] = {}
        self._t_start: dict = {}
        # what the device needs to draw a request's tokens (rules, generator, recent tokens), one block per state slot
        self._states = torch.zeros((self.runner.cache.max_requests, STATE_WORDS), dtype=torch.int32, device=self.runner.device)
        self.pipeline = bool(pipeline)
        self._inflight = None                  # (requests and their output places, picked ids on the device, fetch)

    # ---- requests ---------------------------------------------------------------------------------------
    def add_request(self, ids: Sequence[int], sampling: Sampling | None = None, *, max_tokens: int = 64,
                    eos: Sequence[int] | None = None, ignore_eos: bool = False, seed: int = 42,
                    request_id: Hashable | None = None) -> Hashable:
        if request_id is None:
            request_id = self._next_id
            self._next_id += 1
        if request_id in self.requests and self.requests[request_id].status != "finished":
            raise ValueError(f"request id {request_id!r} is in use")
        vocab = self.runner.vocab
        for t in ids:
            if not (0 <= int(t) < vocab):
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        if eos is None:
            eos = tuple(getattr(self.cfg, "eos_token_id", ()) or ()) if self.cfg is not None else ()
        req = Request(request_id, list(ids), sampling or Sampling(temperature=0.0), max_tokens=max_tokens,
                      eos=tuple(eos), ignore_eos=ignore_eos, seed=seed)
        self.requests[request_id] = req
        self._t_start[request_id] = time.time()
        self.scheduler.add(req)
        return request_id

    def cancel(self, request_id: Hashable) -> list[tuple]:
        """End a request now.  Returns the events of the step that was in flight (tokens of every request, this one
        included, and finish reasons that only that step's tokens reveal) followed by (request_id, None, 'cancelled')
        if the request had not ended by itself; a caller that streams from `step()` must handle them like `step()`'s."""
        events = self.flush()
        req = self.requests[request_id]
        if req.status != "finished":
            self.scheduler.finish(req, "cancelled")
            events.append((request_id, None, "cancelled"))
            if self.events:
                self._request_event(req)
        return events

    @property
    def idle(self) -> bool:
        return self.scheduler.idle and self._inflight is None

    # ---- tokens that a launched step has not delivered yet ---------------------------------------------------
    def flush(self) -> list[tuple]:
        """Wait for the step in flight, if any, and return its events."""
        return self._collect() if self._inflight is not None else []

    def _collect(self, flight=None) -> list[tuple]:
        """Read the tokens of a launched step, put them where their placeholders stand and see which of them end a
        request by their value."""
        if flight is None:
            flight, self._inflight = self._inflight, None
        items, _picked, fetch = flight
        events = []
        for (r, at), tok in zip(items, fetch()):
            if at >= len(r.output):                      # produced after the token that ended the request: dropped
                continue
            r.output[at] = int(tok)
            reason = None
            if not r.ignore_eos and int(tok) in r.eos:
                del r.output[at + 1:]                    # the placeholder of a step launched since
                if r.status != "finished":
                    self.scheduler.finish(r, "eos")
                else:
                    r.finish_reason = "eos"
                reason = "eos"
            elif r.status == "finished" and at == len(r.output) - 1:
                reason = r.finish_reason
            events.append((r.id, int(tok), reason))
            if reason is not None and self.events:
                self._request_event(r)
        return events

    def _tokens_needed_first(self) -> bool:
        """True if the coming plan must not be made on counts alone: a request may be admitted or preempted (its
        tokens are then read back as a prompt), which needs every token's value."""
        sched = self.scheduler
        if sched.waiting:
            return True
        running = len(sched.running)
        return any(g.pool.n_free < running for g in self.runner.cache.groups)

    # ---- one step -----------------------------------------------------------------------------------------
    def step(self) -> list[tuple]:
        """Plan and run one step.  Returns (request id, token, finish reason or None) for every token produced,
        and (request id, None, reason) for requests that ended without one (no_fit).  With `pipeline`, the tokens of
        a greedy decode step are returned by the next call (or by `flush()`); a request that one of them ends by its
        value (an end-of-sequence id) has then already run one more step, whose token is dropped."""
        events = []
        if self._inflight is not None and self._tokens_needed_first():
            events += self._collect()
        n_fin = len(self.scheduler.finished)
        plan = self.scheduler.schedule()
        events += [(r.id, None, r.finish_reason) for r in self.scheduler.finished[n_fin:]]
        wanting = [p for p in plan if p.wants_logits]
        # a step of one token per request: its tokens can stay on the device for the step after it
        decode_only = self.pipeline and bool(wanting) and len(wanting) == len(plan) and all(p.n == 1 for p in plan)
        feedback = None
        if self._inflight is not None:
            if decode_only and [id(p.request) for p in plan] == [id(r) for r, _ in self._inflight[0]]:
                feedback = self._inflight[1]
            else:                                        # another step than the one in flight was counted on
                events += self._collect()
                plan = [p for p in plan if p.request.status != "finished"]    # ended by a token that was in flight
                wanting = [p for p in plan if p.wants_logits]
        if not plan:
            return events
        entries = []
        for p in plan:
            toks = p.request.slice(p.start, p.n)
            entries.append(StepEntry(p.request.id, toks, [p.n - 1] if p.wants_logits else []))
        if wanting:                                      # tokens are drawn in the step's own pass, on the device
            self._upload_sampler_states(wanting)
            whole = any(p.request.sampling.needs_whole_ranking for p in wanting)
            logits, picked = self.runner.step(entries, sample=(self._states, whole), feedback=feedback)
        else:
            logits, picked = self.runner.step(entries), None
        for p in plan:
            self.scheduler.advance(p)
        if decode_only and picked is not None:
            fetch = self.runner.fetch_async(picked, len(wanting))
            items = []
            for p in wanting:
                self.scheduler.on_token_pending(p.request)
                items.append((p.request, len(p.request.output) - 1))
            before, self._inflight = self._inflight, (items, picked, fetch)
            if before is not None:                       # the step before this one: its tokens are read while this one runs
                events += self._collect(before)
            return events
        if wanting:
            drawn = picked.cpu().tolist()
            tokens = [drawn[i] for i in self.runner.last_logit_index]
            for p, tok in zip(wanting, tokens):
                reason = self.scheduler.on_token(p.request, tok)
                events.append((p.request.id, tok, reason))
                if reason is not None and self.events:
                    self._request_event(p.request)
        return events

    def _upload_sampler_states(self, wanting) -> None:
        """Write the sampler state of every request that is about to draw its first token since it was (re)admitted:
        its rules, its generator advanced past the draws it has already made, and the tokens it has produced."""
        for p in wanting:
            r = p.request
            if r.sampler_epoch == r.n_preempted:
                continue
            st = pack_state(r.sampling, r.seed, recent=r.output)
            if r.sampling.temperature > 0.0 and r.output:        # after a preemption: one draw per token so far
                x = max(int(r.seed), 1) & ((1 << 64) - 1)
                for _ in r.output:
                    x ^= (x << 13) & ((1 << 64) - 1)
                    x ^= x >> 7
                    x ^= (x << 17) & ((1 << 64) - 1)
                st[0:2] = np.array([x & 0xFFFFFFFF, x >> 32], dtype=np.uint32).view(np.int32)
            slot = self.runner.cache.state_slot(r.id)
            self._states[slot].copy_(torch.from_numpy(st))
            r.sampler_epoch = r.n_preempted

    def _request_event(self, r: Request) -> None:
        dt = max(time.time() - self._t_start.get(r.id, time.time()), 1e-9)
        emit_event("request", id=r.id, prompt_tokens=len(r.prompt), completion_tokens=len(r.output),
                   finish=r.finish_reason, preempted=r.n_preempted, seconds=f"{dt:.3f}")

    # ---- whole generations --------------------------------------------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], sampling: Sampling | None = None, *, max_tokens: int = 64,
                 eos: Sequence[int] | None = None, ignore_eos: bool = False, seed: int = 42) -> list[list[int]]:
        """Token ids in, generated token ids out, one list per prompt (host lists both ways)."""
        ids = [self.add_request(p, sampling, max_tokens=max_tokens, eos=eos, ignore_eos=ignore_eos, seed=seed + i)
               for i, p in enumerate(prompts)]
        while any(self.requests[i].status != "finished" for i in ids) or self._inflight is not None:
            before = sum(len(self.requests[i].output) for i in ids)
            ev = self.step()
            if not ev and before == sum(len(self.requests[i].output) for i in ids) and self.idle:
                break
        if self.runner.device.type == "cuda":
            ops.raise_on_device_error(self.runner.device)
        return [list(self.requests[i].output) for i in ids]

    def warm_up(self) -> None:
        """Run a few tokens of 1, 2, 4, ... up to `parallel` one-token requests, greedy and with a temperature, so that the
        decode steps of every batch bucket are captured as CUDA graphs before the first real request (a layout's first step
        is launched kernel by kernel and its second is captured; from the third on it is one replay).  Optional; call it
        when the engine is idle."""
        if not self.idle:
            raise RuntimeError("warm_up() wants an idle engine")
        limit = self.runner.cache.max_requests
        n = 1
        while True:
            for s in (Sampling(temperature=0.0), Sampling(temperature=0.8)):
                self.generate([[1 % self.runner.vocab]] * n, s, max_tokens=4, ignore_eos=True)
            if n >= limit:
                break
            n = min(2 * n, limit)

    def finish_reason(self, request_id: Hashable) -> str | None:
        return self.requests[request_id].finish_reason
