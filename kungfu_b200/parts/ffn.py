"""Gated feed-forward.

u = x Wup^T, g = x Wgate^T, h = act(g) * u, y = h Wdown^T
(reference: crates/kf-layers/src/ffn.rs:24-47; the activations are those of
crates/kf-backend-cuda/src/kernels/common.cuh:95: gelu_tanh(x) =
0.5 x (1 + tanh(0.79788456 (x + 0.044715 x^3))), gelu_erf, silu).
Gate and up are stacked into one [2*inner, width] matrix when the model is built,
gate rows first, so one product yields both.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, register_feed_forward

ACTIVATIONS = ("gelu_tanh", "gelu_erf", "silu")


class GatedFfn(FeedForward):
    def __init__(self, w_gate_up: torch.Tensor, w_down: torch.Tensor, activation: str = "gelu_tanh"):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation {activation!r} is not one of {ACTIVATIONS}")
        if w_gate_up.shape[0] != 2 * w_down.shape[1]:
            raise ValueError("stacked gate/up matrix must have twice as many rows as the down matrix has columns")
        self.w_gate_up, self.w_down = w_gate_up, w_down
        self.activation = activation
        self.inner = w_down.shape[1]
        self.width = w_down.shape[0]

    def forward(self, x, ctx):
        T = x.shape[0]
        h = ctx.buf("ffn_h", (T, self.inner), ctx.act_dtype)
        ops.linear_gated(x, self.w_gate_up, h, self.activation, ctx)
        y = ctx.buf("branch_out", (T, self.width), torch.float32)
        ops.linear(h, self.w_down, y)
        return y


register_feed_forward("gated", GatedFfn)
