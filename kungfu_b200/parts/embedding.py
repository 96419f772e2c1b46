"""Token embedding and the output head.

Embedding: x = E[token] * scale, the scale held in 32-bit (reference:
crates/kf-layers/src/basic.rs:16-50; Gemma 2 sets scale = sqrt(width), gemma2.rs:34).
Head: only the rows whose logits are wanted are normalised and multiplied with the
output matrix (the embedding itself when tied), then capped: logits = cap * tanh(logits / cap)
(reference: crates/kf-layers/src/model.rs:155-175, compose.rs:84-99).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Norm, Part


class Embedding(Part):
    def __init__(self, table: torch.Tensor, scale: float = 1.0):
        self.table = table
        self.scale = float(scale)
        self.vocab, self.width = table.shape

    def forward(self, ctx) -> torch.Tensor:
        x = ctx.buf("residual", (ctx.n_rows, self.width), torch.float32)
        ops.embed(ctx.tokens, self.table, self.scale, x)
        return x


class LmHead(Part):
    def __init__(self, norm: Norm, weight: torch.Tensor, softcap: float = 0.0):
        self.norm = norm
        self.weight = weight            # [vocab, width]; the embedding table itself when tied
        self.softcap = float(softcap)
        self.vocab = weight.shape[0]

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        """32-bit logits [n_wanted, vocab] for the rows `ctx.logit_rows` names."""
        n = ctx.n_logits
        h = self.norm.forward(x, ctx, ctx.act_dtype, rows=ctx.logit_rows)
        logits = ctx.buf("logits", (n, self.vocab), torch.float32)
        ops.linear(h, self.weight, logits, softcap=self.softcap)
        return logits
