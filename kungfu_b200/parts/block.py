"""How norms, a mixer and a feed-forward stand around the residual stream.

`SandwichBlock` is the arrangement Gemma 2 uses (reference: crates/kf-layers/src/basic.rs:215-265
`Residual` with a post norm, two of them per block, gemma2.rs:39-41):
  h   = x + post_mixer(mixer(pre_mixer(x)))
  out = h + post_ffn(ffn(pre_ffn(h)))
A post norm of None gives the plain pre-norm block other models use.
The residual stream and its sums stay in 32-bit.
"""
from __future__ import annotations

from .. import ops
from .base import Block, FeedForward, Mixer, Norm, register_block


class SandwichBlock(Block):
    # forward() takes `normed` (this block's pre-mixer norm, already computed by the block before) and `then` (the
    # next block's pre-mixer norm, to be fused into this block's last kernel) and returns (x, normed_for_next)
    fuses_next_norm = True

    def __init__(self, pre_mixer: Norm, mixer: Mixer, post_mixer: Norm | None,
                 pre_ffn: Norm, ffn: FeedForward, post_ffn: Norm | None):
        self.pre_mixer, self.mixer, self.post_mixer = pre_mixer, mixer, post_mixer
        self.pre_ffn, self.ffn, self.post_ffn = pre_ffn, ffn, post_ffn

    def forward(self, x, ctx, cache, normed=None, then=None):
        act = ctx.act_dtype
        n = normed if normed is not None else self.pre_mixer.forward(x, ctx, act)
        a = self.mixer.forward(n, ctx, cache)
        if self.post_mixer is not None:
            n = self.post_mixer.add_into(a, x, ctx, then=self.pre_ffn, out_dtype=act)
        else:
            ops.add(a, x)
            n = self.pre_ffn.forward(x, ctx, act)
        f = self.ffn.forward(n, ctx)
        nxt = None
        if self.post_ffn is not None:
            nxt = self.post_ffn.add_into(f, x, ctx, then=then, out_dtype=act if then is not None else None)
        else:
            ops.add(f, x)
            if then is not None:
                nxt = then.forward(x, ctx, act)
        return x, nxt


register_block("sandwich", SandwichBlock)
