"""Root-mean-square norm.

y_i = x_i / sqrt(mean_j(x_j^2) + eps) * g_i with g = w, or g = 1 + w when `plus_one`
(reference: crates/kf-backend-cuda/src/kernels/norm.cu:4-14 for the norm and :16-27 for
the norm that is added to the residual; Gemma 2 files store w and use 1 + w).
Sums, the reciprocal root and the product run in 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Norm, register_norm


class RmsNorm(Norm):
    def __init__(self, weight: torch.Tensor, eps: float, plus_one: bool = False):
        self.weight = weight
        self.eps = float(eps)
        self.plus_one = bool(plus_one)
        self.width = weight.shape[0]

    def forward(self, x, ctx, out_dtype, rows=None):
        n = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.buf("norm_out" if rows is None else "norm_rows_out", (n, self.width), out_dtype)
        ops.rmsnorm(x, self.weight, self.eps, self.plus_one, out, rows)
        return out

    def add_into(self, branch, residual, ctx, then=None, out_dtype=None):
        """residual += norm(branch); returns then(residual) if `then` is given (one kernel when `then` is an RmsNorm)."""
        if then is None:
            ops.add_rmsnorm(branch, self.weight, self.eps, self.plus_one, residual)
            return None
        if isinstance(then, RmsNorm):
            out = ctx.buf("norm_out", (residual.shape[0], self.width), out_dtype)
            ops.add_rmsnorm(branch, self.weight, self.eps, self.plus_one, residual,
                            next_weight=then.weight, next_eps=then.eps, next_plus_one=then.plus_one, next_out=out)
            return out
        ops.add_rmsnorm(branch, self.weight, self.eps, self.plus_one, residual)
        return then.forward(residual, ctx, out_dtype)


register_norm("rms", RmsNorm)
