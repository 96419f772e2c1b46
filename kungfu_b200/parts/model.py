"""A decoder: embedding, blocks run in the order a list gives, output head.

The order in which blocks run is data (`schedule`): a list of `LayerCall`s.  A call
names the block to run and the cache slot it uses.  A block may be named twice (each
call then has its own cache slot), and a call may read a slot that an earlier call
wrote (`writes=False`, the reference's `kv_source`, crates/kf-layers/src/attention.rs:106-107).
The model reports what each cache slot must hold (`state_needs`); the cache manager
reads only that (reference: `Layer::states`, crates/kf-core/src/layer.rs:20-27).
Reference for the pass itself: crates/kf-layers/src/model.rs:105-180.
"""
from __future__ import annotations

from dataclasses import dataclass

from .. import ops
from .base import Block, Part, StateNeed
from .embedding import Embedding, LmHead


@dataclass(frozen=True)
class LayerCall:
    layer: int                 # index into `layers`
    cache: int                 # cache slot this call uses
    writes: bool = True        # False: reads a slot another call filled in this step


def default_schedule(n_layers: int) -> list[LayerCall]:
    return [LayerCall(i, i) for i in range(n_layers)]


class DecoderModel(Part):
    def __init__(self, embedding: Embedding, layers: list[Block], head: LmHead,
                 schedule: list[LayerCall] | None = None, name: str = ""):
        self.embedding, self.layers, self.head = embedding, list(layers), head
        self.schedule = list(schedule) if schedule is not None else default_schedule(len(self.layers))
        self.name = name
        self.vocab = head.vocab
        writers: dict[int, int] = {}
        for call in self.schedule:
            if not (0 <= call.layer < len(self.layers)):
                raise ValueError(f"schedule names layer {call.layer}; the model has {len(self.layers)}")
            if call.writes:
                if call.cache in writers:
                    raise ValueError(f"cache slot {call.cache} is written by two calls")
                writers[call.cache] = call.layer
            elif call.cache not in writers:
                raise ValueError(f"cache slot {call.cache} is read before any call writes it")
        if sorted(writers) != list(range(len(writers))):
            raise ValueError("cache slots must be numbered 0..n-1")
        self._writers = writers

    def children(self):
        return [self.embedding, *self.layers, self.head]

    def state_needs(self) -> list[StateNeed | None]:
        """Per cache slot, what the mixer that writes it keeps per request."""
        return [self.layers[self._writers[s]].mixer.state_need() for s in range(len(self._writers))]

    def forward(self, ctx):
        """Runs exactly the rows in `ctx`; returns 32-bit logits for `ctx.logit_rows` (None if none wanted)."""
        with ops.nvtx_range("embedding"):
            x = self.embedding.forward(ctx)
        normed = None
        for i, call in enumerate(self.schedule):
            block = self.layers[call.layer]
            view = ctx.cache_view(call.cache, call.writes)
            with ops.nvtx_range(f"layer {call.layer} ({type(block.mixer).__name__})"):
                if getattr(block, "fuses_next_norm", False):
                    # the last kernel of this block also computes the next block's first norm, when both can
                    nxt = self.layers[self.schedule[i + 1].layer] if i + 1 < len(self.schedule) else None
                    then = nxt.pre_mixer if nxt is not None and getattr(nxt, "fuses_next_norm", False) else None
                    x, normed = block.forward(x, ctx, view, normed=normed, then=then)
                else:
                    x, normed = block.forward(x, ctx, view), None
        if ctx.n_logits == 0:
            return None
        with ops.nvtx_range("head"):
            return self.head.forward(x, ctx)
