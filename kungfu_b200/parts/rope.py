"""Rotary position encoding.

For a token at position p and pair index i < r/2 (r = rotary dims, by default the whole
head): angle = p * base^(-2i/r); the pair is (x_i, x_{i+r/2}) ("NeoX" pairing,
reference: crates/kf-backend-cpu/src/rope.rs:18-37,57-108 and gemma2.rs:19):
  x'_i       = x_i cos - x_{i+r/2} sin
  x'_{i+r/2} = x_i sin + x_{i+r/2} cos
The inverse frequencies are computed once in 64-bit and rounded to 32-bit; the angle,
its cosine and sine are 32-bit and are tabulated once per step for all layers that
share this part.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import PositionEncoding, register_position


class Rope(PositionEncoding):
    def __init__(self, head_dim: int, base: float, device, rotary_dims: int | None = None):
        self.head_dim = int(head_dim)
        self.rotary_dims = int(rotary_dims if rotary_dims is not None else head_dim)
        if self.rotary_dims % 2 or self.rotary_dims > self.head_dim:
            raise ValueError(f"rotary_dims {self.rotary_dims} must be even and at most head_dim {self.head_dim}")
        self.base = float(base)
        half = self.rotary_dims // 2
        idx = torch.arange(half, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.base, dtype=torch.float64), -2.0 * idx / self.rotary_dims)
        self.inv_freq = inv.to(torch.float32).to(device)

    def rotation(self, ctx):
        key = ("rope", id(self))
        hit = ctx.memo.get(key)
        if hit is None:
            half = self.rotary_dims // 2
            cos = ctx.buf(f"rope_cos_{id(self)}", (ctx.n_rows, half), torch.float32)
            sin = ctx.buf(f"rope_sin_{id(self)}", (ctx.n_rows, half), torch.float32)
            ops.rope_table(ctx.positions, self.inv_freq, cos, sin)
            hit = (cos, sin)
            ctx.memo[key] = hit
        return hit


register_position("rope", Rope)
