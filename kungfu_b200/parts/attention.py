"""Grouped-query attention over paged keys and values.

In order (reference: crates/kf-layers/src/attention.rs:118-150,160-172,211-283 and
crates/kf-backend-cpu/src/attention.rs:33-45,79-147):
  q, k, v = x Wq^T, x Wk^T, x Wv^T (one product over the stacked matrix)
  q, k rotated by the position encoding; k, v written to the request's pages at the token's position
  head h reads kv head h / (n_heads / n_kv_heads)
  s_j = (q . k_j) * scale; if softcap: s_j = cap * tanh(s_j / cap)
  key j is seen from position p iff j <= p and (no window or p - j < window)
  o = sum_j softmax(s)_j v_j (zeros when no key is seen); y = o Wo^T
Scores, the softmax and the weighted sum are 32-bit.  Sizes and constants are arguments:
this part does not know which model it sits in.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, PagedKV, PositionEncoding, register_mixer


class PagedAttention(Mixer):
    def __init__(self, wqkv: torch.Tensor, wo: torch.Tensor, *, n_heads: int, n_kv_heads: int, head_dim: int,
                 scale: float, softcap: float = 0.0, window: int | None = None,
                 position: PositionEncoding | None = None):
        if n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} is not a multiple of n_kv_heads {n_kv_heads}")
        self.wqkv, self.wo = wqkv, wo
        self.n_heads, self.n_kv_heads, self.head_dim = int(n_heads), int(n_kv_heads), int(head_dim)
        self.scale, self.softcap = float(scale), float(softcap)
        self.window = None if window is None else int(window)
        self.position = position
        self.width = wo.shape[0]
        ops.check_attention_sizes(self.n_heads, self.n_kv_heads, self.head_dim)

    def state_need(self):
        return PagedKV(self.n_kv_heads, self.head_dim, self.window)

    def forward(self, x, ctx, cache):
        T = x.shape[0]
        nh, nkv, d = self.n_heads, self.n_kv_heads, self.head_dim
        if self.position is not None:
            cos, sin = self.position.rotation(ctx)
            rot = 2 * cos.shape[1]
        else:
            cos = sin = None
            rot = 0
        o = ctx.buf("attn_o", (T, nh * d), ctx.act_dtype)
        if ops.decode_attention_takes_qkv(ctx, cache, nh, nkv, d):
            # a decode step: the attention kernel rotates, appends and attends in one launch
            qkv = ctx.buf("attn_qkv", (T, (nh + 2 * nkv) * d), torch.float32)
            ops.linear(x, self.wqkv, qkv)
            ops.rope_append_attend(qkv, cos, sin, rot, o, ctx, cache, nh, nkv, d, self.scale, self.softcap, self.window)
        else:
            q = ctx.buf("attn_q", (T, nh * d), ctx.act_dtype)
            # a long prompt: the product rotates and files its own result where it can
            if not ops.linear_rope_kv_append(x, self.wqkv, cos, sin, rot, nh, nkv, d, ctx, cache, q):
                qkv = ctx.buf("attn_qkv", (T, (nh + 2 * nkv) * d), torch.float32)
                ops.linear(x, self.wqkv, qkv)
                ops.rope_kv_append(qkv, cos, sin, rot, nh, nkv, d, ctx, cache, q)
            ops.paged_attention(q, o, ctx, cache, nh, nkv, d, self.scale, self.softcap, self.window)
        y = ctx.buf("branch_out", (T, self.width), torch.float32)
        ops.linear(o, self.wo, y)
        return y


register_mixer("paged_attention", PagedAttention)
