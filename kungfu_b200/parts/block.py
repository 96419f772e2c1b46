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

    @staticmethod
    def _add_into(post: Norm, branch, x, ctx, then, out_dtype, consumer):
        """(rows for the consumer, residual).  A norm that can defer its work may hand the consumer a pending norm; the
        residual is then the buffer that the consumer's kernel writes."""
        if consumer is not None and getattr(post, "can_defer", False):
            n = post.add_into(branch, x, ctx, then=then, out_dtype=out_dtype, consumer=consumer)
            if isinstance(n, ops.PendingNorm):
                return n, n.residual_out
            return n, x
        return post.add_into(branch, x, ctx, then=then, out_dtype=out_dtype), x

    def forward(self, x, ctx, cache, normed=None, then=None, then_consumer=None):
        act = ctx.act_dtype
        n = normed if normed is not None else self.pre_mixer.forward(x, ctx, act)
        a = self.mixer.forward(n, ctx, cache)
        if self.post_mixer is not None:
            n, x = self._add_into(self.post_mixer, a, x, ctx, self.pre_ffn, act, self.ffn)
        else:
            ops.add(a, x)
            n = self.pre_ffn.forward(x, ctx, act)
        f = self.ffn.forward(n, ctx)
        nxt = None
        if self.post_ffn is not None:
            nxt, x = self._add_into(self.post_ffn, f, x, ctx, then, act if then is not None else None,
                                    then_consumer if then is not None else None)
        else:
            ops.add(f, x)
            if then is not None:
                nxt = then.forward(x, ctx, act)
        return x, nxt


register_block("sandwich", SandwichBlock)
