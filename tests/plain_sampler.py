"""A plain sampler: the reference's rules restated for one row of logits on the host, for tests only.

Written from nickheyer/kungfu's crates/kf-engine/src/sampler.rs (file:line at each step); it shares no code with the
kernels of kungfu_b200/csrc/sampling.cu, which it checks.  One difference from the reference, on purpose and the same
as in the kernels: masses are summed in 64-bit (the reference adds 32-bit numbers one after the other), so that a
result does not depend on the order of a sum.
"""
from __future__ import annotations

import numpy as np

_MASK64 = (1 << 64) - 1


class Rng:
    """xorshift64; next_f32 = top 24 bits / 2^24; seed max(seed, 1).  sampler.rs:20-34."""

    def __init__(self, seed: int):
        self.state = max(int(seed), 1) & _MASK64

    def next_f32(self) -> float:
        x = self.state
        x ^= (x << 13) & _MASK64
        x ^= x >> 7
        x ^= (x << 17) & _MASK64
        self.state = x
        return float(np.float32(x >> 40) / np.float32(1 << 24))


def penalized(v: np.float32, penalty: float) -> np.float32:
    """Positive logits divided, others multiplied.  sampler.rs:62-65."""
    p = np.float32(penalty)
    return np.float32(v / p) if v > 0 else np.float32(v * p)


def ranking(l: np.ndarray) -> np.ndarray:
    """Ids by falling logit, the lower id first among equals (a stable sort, sampler.rs:52-53)."""
    return np.argsort(-l.astype(np.float64), kind="stable")


def sample(logits, *, temperature, top_k=0, top_p=1.0, min_p=0.0, repeat_penalty=1.0, repeat_window=64, recent=(), rng=None):
    """(token, margin): the token one row yields, and how far (as a fraction of the kept mass) the drawn number lies
    from the nearer end of that token's interval; a draw whose margin is tiny may legitimately fall to a neighbour
    when exponentials differ in their last bit.  `margin` is None when nothing was drawn (greedy).
    Order of the rules: sampler.rs:37-100."""
    l = np.array(logits, dtype=np.float32, copy=True)
    if repeat_penalty != 1.0:                                                     # :42-48
        window = list(recent)[-repeat_window:] if repeat_window > 0 else []
        for t in window:
            if 0 <= t < len(l):
                l[t] = penalized(l[t], repeat_penalty)
    if temperature <= 0.0:                                                        # :38-40,49-51,219-227
        return int(np.argmax(l)), None
    order = ranking(l)
    if top_k > 0:                                                                 # :54-56
        order = order[:top_k]
    vals = l[order]
    w = np.exp(((vals - vals[0]) / np.float32(temperature)).astype(np.float32)).astype(np.float32)   # :70
    mass1 = float(w.astype(np.float64).sum())
    keep = len(w)
    if min_p > 0.0:                                                               # :74-77: p >= p_0 min_p, and w_0 = 1
        below = np.nonzero(w < np.float32(min_p))[0]
        keep = max(int(below[0]) if len(below) else keep, 1)
    if top_p < 1.0:                                                               # :78-89
        acc = np.cumsum(w[:keep].astype(np.float64))
        hit = np.nonzero(acc >= float(np.float32(top_p)) * mass1)[0]
        keep = int(hit[0]) + 1 if len(hit) else keep
    cum = np.cumsum(w[:keep].astype(np.float64))
    r = float(np.float32(rng.next_f32())) * float(cum[-1])                        # :91-92
    at = int(np.searchsorted(cum, r, side="right"))                               # first i with r < cum[i]  (:93-98)
    at = min(at, keep - 1)
    lo = cum[at - 1] if at > 0 else 0.0
    margin = min(r - lo, cum[at] - r) / float(cum[-1])
    return int(order[at]), float(margin)
