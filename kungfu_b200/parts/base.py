"""Interfaces of the parts a model is put together from, and what each part may ask of the cache.

The reference's layer trait is `forward`, `weights`, `states` (crates/kf-core/src/layer.rs:8-27)
and a layer tells the planner what per-sequence state it keeps through `StateNeed`
(layer.rs:29-43); the planner never looks at layer types.  The same split holds here:

* `Norm`, `PositionEncoding`, `Mixer`, `FeedForward` and `Block` are the part kinds;
* a mixer declares a `StateNeed` (paged keys/values with an optional window, or a
  fixed-size per-request state); the cache manager reads only that declaration;
* a part receives its sizes and constants as constructor arguments and a `StepContext`
  at run time; it never sees the configuration or the model that holds it.

New kinds register under a name (`register_mixer` and friends) so an architecture's
builder can choose them by name, layer by layer.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch


# ---- what a mixer keeps per request -------------------------------------------------------------

@dataclass(frozen=True)
class PagedKV:
    """Keys and values for every past token, in pages; `window` keys at most are ever read when set."""
    n_kv_heads: int
    head_dim: int
    window: int | None = None


@dataclass(frozen=True)
class FixedState:
    """A state of fixed shape per live request (a recurrent state, a running sum); zeroed at admission."""
    shape: tuple
    dtype: torch.dtype = torch.float32


StateNeed = PagedKV | FixedState


# ---- part kinds -----------------------------------------------------------------------------------

class Part:
    """Common base: parts report their weight tensors for accounting."""

    # False for a part whose forward does host-side work that depends on the step (loops over requests, reads of
    # ctx.host): steps of a model holding such a part are never captured into CUDA graphs.
    graph_safe = True
    # Names of further per-row integer streams this part reads from `ctx.streams` (a second position axis, a segment
    # id, ...).  The step function carries every declared stream in its integer block; a request gives the values with
    # its tokens (`StepEntry.streams`), and a stream it does not give holds the tokens' positions.
    step_streams: tuple = ()

    def step_stream_names(self) -> list:
        names = list(self.step_streams)
        for c in self.children():
            for n in c.step_stream_names():
                if n not in names:
                    names.append(n)
        return names

    def all_graph_safe(self) -> bool:
        return self.graph_safe and all(c.all_graph_safe() for c in self.children())

    def weights(self) -> list[torch.Tensor]:
        return [v for v in vars(self).values() if isinstance(v, torch.Tensor)]

    def children(self) -> list["Part"]:
        return [v for v in vars(self).values() if isinstance(v, Part)]

    def weight_bytes(self, seen: set | None = None) -> int:
        seen = set() if seen is None else seen
        n = 0
        for w in self.weights():
            if w.data_ptr() not in seen:
                seen.add(w.data_ptr())
                n += w.numel() * w.element_size()
        for c in self.children():
            n += c.weight_bytes(seen)
        return n


class Norm(Part):
    """y = normalise(x) over the last axis.  x is the 32-bit residual stream [rows, width]."""

    def forward(self, x: torch.Tensor, ctx, out_dtype: torch.dtype, rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError

    def add_into(self, branch: torch.Tensor, residual: torch.Tensor, ctx, then: "Norm | None" = None,
                 out_dtype: torch.dtype | None = None) -> torch.Tensor | None:
        """residual += norm(branch); if `then` is given also return then(residual) in `out_dtype`."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Turns the step's positions into whatever the mixer applies to queries and keys."""

    def rotation(self, ctx) -> tuple[torch.Tensor, torch.Tensor]:
        """cos and sin, each [rows, head_dim/2] in 32-bit, for this step's rows (computed once per step)."""
        raise NotImplementedError


class Mixer(Part):
    """Mixes information across the tokens of a request (attention, a recurrence, ...)."""

    def state_need(self) -> StateNeed | None:
        return None

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        """x: normalised input [rows, width] in the step's activation dtype; returns 32-bit [rows, width].
        `cache` is the view of this call's cache slot (`PagedKVView` or `FixedStateView`) or None."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """x: normalised input [rows, width] in the activation dtype; returns 32-bit [rows, width]."""
        raise NotImplementedError


class Block(Part):
    """An arrangement of norms, one mixer and one feed-forward around the residual stream."""

    mixer: Mixer
    # A block that sets this takes forward(x, ctx, cache, normed=None, then=None) and returns (x, normed_for_next):
    # `normed` is its own first norm computed by the block before it, `then` the next block's first norm.
    fuses_next_norm = False

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        raise NotImplementedError


# ---- registries of part kinds ---------------------------------------------------------------------

_KINDS: dict[str, dict[str, Callable]] = {"mixer": {}, "feed_forward": {}, "norm": {}, "position": {}, "block": {}}


def _register(kind: str, name: str, factory: Callable) -> Callable:
    table = _KINDS[kind]
    if name in table and table[name] is not factory:
        raise ValueError(f"{kind} '{name}' is already registered")
    table[name] = factory
    return factory


def register_mixer(name: str, factory: Callable) -> Callable:
    return _register("mixer", name, factory)


def register_feed_forward(name: str, factory: Callable) -> Callable:
    return _register("feed_forward", name, factory)


def register_norm(name: str, factory: Callable) -> Callable:
    return _register("norm", name, factory)


def register_position(name: str, factory: Callable) -> Callable:
    return _register("position", name, factory)


def register_block(name: str, factory: Callable) -> Callable:
    return _register("block", name, factory)


def make(kind: str, name: str, *args, **kwargs):
    """Build the part registered as `name` under `kind` ('mixer', 'feed_forward', 'norm', 'position', 'block')."""
    table = _KINDS[kind]
    if name not in table:
        raise KeyError(f"no {kind} named '{name}'; known: {sorted(table)}")
    return table[name](*args, **kwargs)


def known(kind: str) -> list[str]:
    return sorted(_KINDS[kind])
