"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere, runs exactly
those tokens as one batch and returns the logits at the wanted places.  The reference's backend
takes the same shape of input, rows of several sequences in one pass with per-row tokens,
positions and sequence ids (crates/kf-core/src/backend.rs:113-129, runs :190-203), though its scheduler
never mixes prompt rows with decode rows; here that is the normal case.

Per step the host builds one block of 32-bit integers (tokens, positions, the request of each row,
per request its rows / length / state slot, the block tables of every cache group, the rows whose
logits are wanted) and sends it to the device in one copy; every kernel of the step reads from it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager, OutOfPages


@dataclass
class StepEntry:
    request: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)      # places among `tokens` whose logits are wanted
    # further integers per token, by stream name, for parts that declare `step_streams` (a second position axis, a
    # segment id); a stream the entry does not give holds the tokens' positions
    streams: dict | None = None


class StepError(ValueError):
    pass


class BufferPool:
    """Named device buffers that keep their address from step to step (grown when a step needs more)."""

    def __init__(self, device):
        self.device = device
        self._flat: dict[str, torch.Tensor] = {}
        self.generation = 0                                   # bumps whenever a buffer moves

    def get(self, tag: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = max(n * torch.empty(0, dtype=dtype).element_size(), 16)
        flat = self._flat.get(tag)
        if flat is None or flat.numel() < nbytes:
            grow = nbytes if flat is None else max(nbytes, 2 * flat.numel())
            flat = torch.empty(grow, dtype=torch.uint8, device=self.device)
            self._flat[tag] = flat
            self.generation += 1
        return flat[: n * torch.empty(0, dtype=dtype).element_size()].view(dtype).view(*shape)

    def nbytes(self) -> int:
        return sum(t.numel() for t in self._flat.values())


def _align4(n: int) -> int:
    return (n + 3) & ~3


class StepContext:
    """Everything parts may read during one step.  Integer arrays live on the device."""

    def __init__(self, runner: "Runner"):
        self._runner = runner
        self.act_dtype = runner.act_dtype
        self.device = runner.device
        self.memo: dict = {}
        self.n_rows = 0
        self.n_reqs = 0
        self.n_logits = 0
        self.decode_only = False
        self.max_rows_per_req = 0
        self.dec_rows = self.pre_rows = None      # rows of single-row requests / of the others (device int32)
        self.n_dec_rows = self.n_pre_rows = 0
        self.max_kv_len = 0
        self.tile_row0 = self.tile_nrows = None   # prompt-portion tiles: first row and row count (device int32)
        self.n_tiles = 0
        self.wide_row0 = self.wide_nrows = None   # the same rows cut into tiles of up to 128
        self.n_wide = 0
        # device views, set by Runner._fill
        self.tokens = self.positions = self.row_req = self.logit_rows = self.logit_req = None
        self.req_row_start = self.req_n_rows = self.req_kv_len = self.req_state_slot = None
        self.block_tables: list[torch.Tensor] = []
        self.streams: dict[str, torch.Tensor] = {}    # extra per-row integers that parts declared (device int32 [rows])
        # host copies
        self.host: dict[str, np.ndarray] = {}

    def buf(self, tag: str, shape: tuple, dtype: torch.dtype) -> torch.Tensor:
        return self._runner.buffers.get(tag, shape, dtype)

    def cache_view(self, cache_slot: int, writes: bool):
        return self._runner.cache.view(cache_slot, writes)


class Runner:
    """Owns the model, the cache manager and the device buffers, and runs steps."""

    def __init__(self, model, cache: CacheManager, *, act_dtype: torch.dtype, device):
        self.model = model
        self.cache = cache
        self.act_dtype = act_dtype
        self.device = torch.device(device)
        self.buffers = BufferPool(self.device)
        self.vocab = model.vocab
        self._staging: list = []                  # ring of (pinned host block, event of its last copy)
        self._staging_next = 0
        self._meta_dev: torch.Tensor | None = None
        self.steps_run = 0
        self.last_meta_ints = 0
        self.last_logit_index: list[int] = []             # where in the last step's logits each wanted place stands
        self.cuda_graphs = False
        self._graphs: dict = {}
        self._graph_safe = model.all_graph_safe() if hasattr(model, "all_graph_safe") else False
        self.stream_names = tuple(model.step_stream_names()) if hasattr(model, "step_stream_names") else ()
        self.launch_count_hint = 0

    # ---- metadata -----------------------------------------------------------------------------------
    def _meta_buffers(self, n_ints: int):
        """A pinned host block whose last copy has finished, and the device block it is copied to."""
        cuda = self.device.type == "cuda"
        if self._meta_dev is None or self._meta_dev.numel() < n_ints:
            cap = max(n_ints, 1024)
            cap = 1 << (cap - 1).bit_length()
            if cuda:
                torch.cuda.current_stream().synchronize()
            self._staging = [[torch.empty(cap, dtype=torch.int32, pin_memory=cuda), None] for _ in range(3)]
            self._meta_dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            self.buffers.generation += 1
        slot = self._staging[self._staging_next]
        self._staging_next = (self._staging_next + 1) % len(self._staging)
        if slot[1] is not None:
            slot[1].synchronize()
        return slot, self._meta_dev

    _SECTIONS = ("tokens", "positions", "row_req", "logit_rows", "dec_rows", "pre_rows", "tile_row0", "tile_nrows",
                 "wide_row0", "wide_nrows", "req_row_start", "req_n_rows", "req_kv_len", "req_state_slot", "logit_req")

    def _build_block(self, entries: Sequence[StepEntry], bucket: int | None, feedback: torch.Tensor | None = None):
        """The step's integer block, built by the native host runtime (`kf_step_layout` / `kf_step_fill` in
        csrc/host_runtime.cpp) straight into a pinned staging block, and its copy to the device.
        `feedback` (a device tensor of token ids, one per entry, for steps of single tokens) then overwrites the
        block's tokens on the device: the host need not know them yet.
        Returns (info, device block): info[0] total ints, [1] rows, [2] requests, [3] wanted rows, [4] table width,
        [5] decode rows, [6] prompt rows, [7] tiles of 64, [8] tiles of 128, [9] longest kv length, [10] most rows of
        one request, then the offset of every section."""
        cache = self.cache
        lib = cache._lib
        n = len(entries)
        reqs = np.fromiter((cache.key_of(e.request) for e in entries), dtype=np.int64, count=n)
        n_tokens = np.fromiter((len(e.tokens) for e in entries), dtype=np.int32, count=n)
        n_want = np.fromiter((len(e.want) for e in entries), dtype=np.int32, count=n)
        mixed = isinstance(bucket, tuple)                  # ("mixed", decode rows, prompt rows, prompt portions)
        b, pre, pre_reqs = (int(bucket[1]), int(bucket[2]), int(bucket[3])) if mixed else (int(bucket or 0), 0, 0)
        if (not mixed and b > 0) or int(n_tokens.max(initial=0)) == 1:
            tokens = np.fromiter((e.tokens[0] for e in entries), dtype=np.int32, count=n)
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries]) if n else np.zeros(0, np.int32)
        wants = np.fromiter((w for e in entries for w in e.want), dtype=np.int32, count=int(n_want.sum()))
        info = np.zeros(32 + len(cache.groups), dtype=np.int32)
        total = lib.kf_step_layout(cache._h, n, reqs.ctypes.data, n_tokens.ctypes.data, n_want.ctypes.data, b, pre, pre_reqs,
                                   info.ctypes.data)
        if total < 0:
            raise StepError("a request of the step is not live" if total == -1 else f"the step does not fit its layout (code {-total})")
        T = int(info[1])
        base = _align4(total)                              # the extra streams follow the native sections, T ints each
        total = base + len(self.stream_names) * _align4(T) if self.stream_names else total
        slot, dev = self._meta_buffers(total)
        self.last_meta_ints = total
        host = slot[0]
        rc = lib.kf_step_fill(cache._h, n, reqs.ctypes.data, n_tokens.ctypes.data, tokens.ctypes.data, n_want.ctypes.data,
                              wants.ctypes.data, b, pre, pre_reqs, info.ctypes.data, host.data_ptr())
        if rc != 0:
            raise StepError(f"building the step's integer block failed (code {rc})")
        if self.stream_names:
            h = host.numpy()
            pos0 = int(info[12])                           # the positions' section
            row = 0
            rows_of = []
            for e in entries:
                rows_of.append((row, len(e.tokens)))
                row += len(e.tokens)
            for i, name in enumerate(self.stream_names):
                at = base + i * _align4(T)
                h[at:at + T] = h[pos0:pos0 + T]
                for e, (r0, cnt) in zip(entries, rows_of):
                    vals = (e.streams or {}).get(name)
                    if vals is not None:
                        if len(vals) != cnt:
                            raise StepError(f"request {e.request!r}: stream '{name}' has {len(vals)} values for {cnt} tokens")
                        h[at + r0:at + r0 + cnt] = np.asarray(vals, dtype=np.int32)
            info = np.concatenate([info, np.asarray([base], dtype=np.int32)])
        dev[:total].copy_(host[:total], non_blocking=True)
        if self.device.type == "cuda":
            if slot[1] is None:
                slot[1] = torch.cuda.Event()
            slot[1].record()
        if feedback is not None:
            at = int(info[11])                            # the tokens' section; row i is entry i in a step of single tokens
            dev[at:at + n].copy_(feedback[:n])
        return info, dev, host

    def _fill(self, entries: Sequence[StepEntry], bucket: int | None = None, feedback=None) -> StepContext:
        """Build the step's integer block and the context that names its sections.  With `bucket` (decode-only
        steps replayed from a CUDA graph) the layout is the one of `bucket` single-row requests with full-width
        block tables, whatever the step holds: rows beyond the real ones are padding (request index -1) that every
        kernel skips."""
        info, dev, host = self._build_block(entries, bucket, feedback)
        ctx = StepContext(self)
        total, T, B, n_out, width, n_dec, n_pre, n_tiles, n_wide, max_kv, max_rows = (int(v) for v in info[:11])
        off = info[11:]
        h = host.numpy()
        sizes = {"tokens": T, "positions": T, "row_req": T, "logit_rows": max(n_out, 1), "dec_rows": T, "pre_rows": T,
                 "tile_row0": T // 64 + B + 1, "tile_nrows": T // 64 + B + 1, "wide_row0": T // 128 + B + 1,
                 "wide_nrows": T // 128 + B + 1, "req_row_start": B, "req_n_rows": B, "req_kv_len": B, "req_state_slot": B,
                 "logit_req": max(n_out, 1)}
        where = {name: (int(off[i]), sizes[name]) for i, name in enumerate(self._SECTIONS)}

        def dview(name):
            a, n = where[name]
            return dev[a:a + n]

        ctx.n_rows, ctx.n_reqs, ctx.n_logits = T, B, n_out
        ctx.max_rows_per_req = max_rows
        ctx.decode_only = max_rows == 1
        ctx.tokens, ctx.positions, ctx.row_req = dview("tokens"), dview("positions"), dview("row_req")
        ctx.logit_rows = dview("logit_rows")[:n_out] if n_out else dview("logit_rows")[:0]
        ctx.logit_req = dview("logit_req")[:n_out] if n_out else dview("logit_req")[:0]
        ctx.dec_rows, ctx.n_dec_rows = dview("dec_rows"), n_dec
        ctx.pre_rows, ctx.n_pre_rows = dview("pre_rows"), n_pre
        ctx.max_kv_len = max_kv
        ctx.tile_row0, ctx.tile_nrows, ctx.n_tiles = dview("tile_row0"), dview("tile_nrows"), n_tiles
        ctx.wide_row0, ctx.wide_nrows, ctx.n_wide = dview("wide_row0"), dview("wide_nrows"), n_wide
        ctx.req_row_start, ctx.req_n_rows = dview("req_row_start"), dview("req_n_rows")
        ctx.req_kv_len, ctx.req_state_slot = dview("req_kv_len"), dview("req_state_slot")
        n_sec = len(self._SECTIONS)
        ctx.block_tables = [dev[int(off[n_sec + g]):int(off[n_sec + g]) + B * width].view(B, width)
                            for g in range(len(self.cache.groups))]
        if self.stream_names:
            base = int(info[-1])
            ctx.streams = {name: dev[base + i * _align4(T):base + i * _align4(T) + T] for i, name in enumerate(self.stream_names)}
        ctx.host = {name: h[where[name][0]:where[name][0] + where[name][1]].copy()
                    for name in ("positions", "row_req", "req_row_start", "req_n_rows", "req_kv_len", "req_state_slot")}
        return ctx

    # ---- the step -------------------------------------------------------------------------------------
    def validate(self, entries: Sequence[StepEntry]) -> None:
        seen = set()
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            if e.request not in self.cache:
                raise StepError(f"request {e.request!r} is not live")
            n = len(e.tokens)
            if n == 0:
                raise StepError(f"request {e.request!r} brings no tokens")
            for t in e.tokens:
                if not (0 <= int(t) < self.vocab):
                    raise StepError(f"request {e.request!r}: token id {t} is outside the vocabulary of {self.vocab}")
            for w in e.want:
                if not (0 <= int(w) < n):
                    raise StepError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")

    def step(self, entries: Sequence[StepEntry], sample=None, feedback: torch.Tensor | None = None):
        """Run the tokens of `entries` as one batch.  Returns 32-bit logits [wanted, vocab] on the device,
        in the order of the entries and of each entry's `want`, or None when nothing is wanted.  The result
        lives in a buffer the next step overwrites.  Raises OutOfPages before touching anything when the
        pages for the new tokens cannot all be had.
        `sample`: (sampler states [max_requests, STATE_WORDS] int32 on the device, whole_ranking); the token of every
        wanted row is then drawn in the same pass under its request's rules (inside the replayed graph when the step has
        one) and the result is (logits, int32 token ids), both with one row per wanted place EXCEPT under a padded mixed
        layout, where `last_logit_index` says which row holds which wanted place.
        `feedback`: for a step in which every entry brings one token, a device tensor with those tokens in the order
        of the entries (the ids an earlier step drew, which the host has not read yet); the entries' own token values
        are then ignored."""
        entries = list(entries)
        greedy = sample is not None
        if not entries:
            return (None, None) if greedy else None
        self.validate(entries)
        if feedback is not None and any(len(e.tokens) != 1 for e in entries):
            raise StepError("tokens can only be fed back on the device to a step of single tokens")
        reserved = []
        try:
            for e in entries:
                self.cache.reserve(e.request, len(e.tokens))
                reserved.append(e)
        except OutOfPages:
            for e in reserved:
                self.cache.cancel_reservation(e.request)
            raise
        try:
            bucket = self._graph_bucket(entries, greedy)
            self.last_logit_index = self._logit_index(entries, bucket)
            picked = None
            if bucket is None:
                ctx = self._fill(entries, None, feedback)
                logits = self._forward(ctx)
                if greedy and logits is not None:
                    picked = self._sample(logits, ctx, sample)
            elif greedy:
                logits, picked = self._step_graphed(entries, ("sample", bucket, bool(sample[1])), feedback, sample)
            else:
                logits = self._step_graphed(entries, bucket, feedback)
        except BaseException:
            for e in entries:                              # nothing was committed: the pages taken for this step go back
                self.cache.cancel_reservation(e.request)
            raise
        for e in entries:
            self.cache.commit(e.request, len(e.tokens))
        self.steps_run += 1
        return (logits, picked) if greedy else logits

    def fetch_async(self, ids: torch.Tensor, n: int):
        """Start the copy of `ids[:n]` (token ids on the device) to pinned host memory, in stream order after the step
        that wrote them and before anything that overwrites them; returns a function that waits for the copy and gives
        the ids as a list."""
        if self.device.type != "cuda":
            vals = ids[:n].tolist()
            return lambda: vals
        ring = getattr(self, "_fetch_ring", None)
        if ring is None or ring[0][0].numel() < n:
            cap = max(64, 1 << (max(n, 1) - 1).bit_length())
            ring = self._fetch_ring = [[torch.empty(cap, dtype=torch.int32, pin_memory=True), torch.cuda.Event()] for _ in range(4)]
            self._fetch_next = 0
        buf, ev = ring[self._fetch_next]
        self._fetch_next = (self._fetch_next + 1) % len(ring)
        buf[:n].copy_(ids[:n], non_blocking=True)
        ev.record()

        def wait():
            ev.synchronize()
            return buf[:n].tolist()
        return wait

    def _sample(self, logits, ctx, sample):
        """Draw the token of every wanted row on the device (ops.sample) from its request's sampler state."""
        from .. import ops
        states, whole = sample
        out = self.buffers.get("sampled_ids", (max(logits.shape[0], 1),), torch.int32)
        # row i of the logits belongs to request ctx.logit_req[i] of the step (-1: a row of a padded layout that nobody wants)
        ops.sample(logits, states, out, row_req=ctx.logit_req, req_slot=ctx.req_state_slot, whole_ranking=bool(whole))
        return out[:logits.shape[0]]

    # ---- steps replayed from CUDA graphs -------------------------------------------------------------------------
    MAX_MIXED_GRAPHS = 24

    def _graph_bucket(self, entries, sampled: bool):
        """The layout under which this step can be replayed from a CUDA graph, or None if it runs eagerly.
        A pure decode step: the padded batch size (an int).  A step that holds prompt portions, with or without decode
        rows before them (what the scheduler plans while prompts are being fed under a token budget): ("mixed", decode
        rows, prompt rows, portions), each rounded up to a bucket; such steps repeat with the same shape, and launching
        their two hundred kernels one by one takes the host longer than the GPU needs to run them.  Mixed layouts have
        one output row per request, so they serve steps whose tokens are drawn on the device (`sampled`) and whose
        portions want their last row or none."""
        if not self.cuda_graphs or self.device.type != "cuda" or not self._graph_safe:
            return None
        from .. import ops
        if ops.tracing():                                  # per-kernel timing needs eager launches
            return None
        nd = 0
        while nd < len(entries) and len(entries[nd].tokens) == 1 and list(entries[nd].want) == [0]:
            nd += 1
        rest = entries[nd:]
        if not rest:
            b = 1
            while b < nd:
                b *= 2
            return b if b <= max(self.cache.max_requests, 1) * 2 else None
        if not sampled or self.stream_names or len(rest) > 4:
            return None
        rows = 0
        for e in rest:
            n = len(e.tokens)
            if n < 2 or list(e.want) not in ([], [n - 1]):
                return None
            rows += n
        if rows > 2048:
            return None
        d = 0
        if nd:
            d = 1
            while d < nd:
                d *= 2
        # decode and prompt rows TOGETHER are rounded up to the unit (a scheduler that pads its decode rows the same way hands
        # out budget - d prompt rows, and the step's products then see exactly the budget's rows)
        unit = 64 if rows <= 512 else 128 if rows <= 1024 else 256
        key = ("mixed", d, -(-(d + rows) // unit) * unit - d, 1 if len(rest) == 1 else 2 if len(rest) == 2 else 4)
        held = {k[1] for k in self._graphs if isinstance(k, tuple) and isinstance(k[1], tuple)}
        return key if (key in held or len(held) < self.MAX_MIXED_GRAPHS) else None

    @staticmethod
    def _logit_index(entries, bucket) -> list[int]:
        """For every wanted place of the step, in the order of the entries, the row of the step's logits that holds it."""
        if not isinstance(bucket, tuple):
            return list(range(sum(len(e.want) for e in entries)))
        d, out, j = bucket[1], [], 0
        for i, e in enumerate(entries):
            if len(e.tokens) == 1:
                out.append(i)
            else:
                if e.want:
                    out.append(d + j)
                j += 1
        return out

    def _forward(self, ctx):
        """The model's pass over the step, every launch on the stream that is current now."""
        if self.device.type == "cuda":
            from .. import ops
            with ops.pinned_stream():
                return self.model.forward(ctx)
        return self.model.forward(ctx)

    def _step_graphed(self, entries, key, feedback=None, sample=None):
        """First time a key is seen the step runs eagerly (that also sizes every buffer); the second time the
        launches are captured into a graph; from then on the step is one copy of integers and one replay."""
        from .. import ops
        pick = isinstance(key, tuple) and key[0] == "sample"   # a graph that also holds the draw of the tokens
        bucket = key[1] if pick else key
        if isinstance(bucket, tuple):                      # a mixed layout: one output row per request of the bucket
            n = bucket[1] + bucket[3]
        else:
            n = len(entries)
        state = self._graphs.get(key)
        if state is not None and state["generation"] != self.buffers.generation:
            state = None                                   # a buffer moved: the old graph points at freed memory
            self._graphs.pop(key)
        if state is not None and pick and state.get("states_ptr") != sample[0].data_ptr():
            state = None                                   # another engine's sampler states
            self._graphs.pop(key)

        def result(logits, picked=None):
            out = None if (logits is None or n == 0) else logits[:n]
            return (out, None if picked is None else picked[:n]) if pick else out

        def run(ctx):
            logits = self._forward(ctx)
            return (logits, self._sample(logits, ctx, sample)) if (pick and logits is not None) else (logits, None)

        if state is not None and state["graph"] is not None:
            self._build_block(entries, bucket, feedback)  # same layout as at capture; a replay needs no context object
            state["graph"].replay()
            ops.add_launches(state["kernels"])
            return result(state["logits"], state["picked"])
        ctx = self._fill(entries, bucket, feedback)
        if state is None:
            self._graphs[key] = {"generation": None, "graph": None, "seen": 1,
                                 "states_ptr": sample[0].data_ptr() if pick else None}
            logits, picked = run(ctx)
            self._graphs[key]["generation"] = self.buffers.generation
            return result(logits, picked)
        if state["graph"] is None:
            before = ops.launch_count()
            graph = torch.cuda.CUDAGraph()
            torch.cuda.current_stream().synchronize()
            with torch.cuda.graph(graph):
                logits, picked = run(ctx)
            if self.buffers.generation != state["generation"]:
                self._graphs.pop(key)                      # capture itself grew a buffer: run this step eagerly
                return result(*run(ctx))
            state.update(graph=graph, logits=logits, picked=picked, kernels=ops.launch_count() - before)
            ops.add_launches(-state["kernels"])            # capture launched nothing
        state["graph"].replay()
        ops.add_launches(state["kernels"])
        return result(state["logits"], state["picked"])
