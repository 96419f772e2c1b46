"""Sampling: greedy, temperature, top-k, top-p, min-p and the repeat penalty, with the reference's generator.

Pipeline and defaults (reference: crates/kf-engine/src/sampler.rs:4-17,37-100): temperature <= 0 (and no
penalty) is greedy, the first maximum wins (:219-227); otherwise repeat penalty on the last `repeat_window`
tokens (positive logits divided, negative multiplied, :62-65), sort by falling logit, keep `top_k`
(0 keeps all), p = softmax((l - max) / T), min-p cut, top-p cut (smallest prefix whose sum reaches top_p),
renormalise, draw r = rng * sum and walk.  The generator is xorshift64 (x ^= x<<13; x ^= x>>7; x ^= x<<17),
next_f32 = (x >> 40) / 2^24, seed max(seed, 1) (:20-34).

On the device the step ends in `argmax` (greedy) or `topk_lse` (64 candidates and the row's
log-sum-exp); the draw itself runs on the host from the candidates when they settle it
(`sample_sparse`, sampler.rs:177-217) and from the whole row otherwise.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

CANDIDATES = 64          # reference: TOP = 64, crates/kf-engine/src/session.rs:80
_MASK64 = (1 << 64) - 1


@dataclass
class Sampling:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    repeat_window: int = 64

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 and self.repeat_penalty == 1.0


class Rng:
    """xorshift64, deterministic from its seed."""

    def __init__(self, seed: int):
        self.state = max(int(seed), 1) & _MASK64

    def next_f32(self) -> float:
        x = self.state
        x ^= (x << 13) & _MASK64
        x ^= x >> 7
        x ^= (x << 17) & _MASK64
        self.state = x
        return float(np.float32(x >> 40) / np.float32(1 << 24))


def argmax(logits: np.ndarray) -> int:
    return int(np.argmax(logits))            # numpy returns the first maximum


def _penalized(v: np.float32, penalty: float) -> np.float32:
    return np.float32(v / penalty) if v > 0 else np.float32(v * penalty)


def draw(ids: np.ndarray, vals: np.ndarray, s: Sampling, rng: Rng) -> int:
    """One token from ids ordered by falling logit: temperature, min-p, top-p in that order."""
    vals = vals.astype(np.float32)
    probs = np.exp((vals - vals[0]) / np.float32(s.temperature)).astype(np.float32)
    probs /= probs.sum(dtype=np.float32)
    keep = len(probs)
    if s.min_p > 0.0:
        floor = probs[0] * np.float32(s.min_p)
        below = np.nonzero(probs < floor)[0]
        keep = max(int(below[0]) if len(below) else keep, 1)
    if s.top_p < 1.0:
        acc = np.cumsum(probs[:keep], dtype=np.float32)
        hit = np.nonzero(acc >= np.float32(s.top_p))[0]
        keep = int(hit[0]) + 1 if len(hit) else keep
    probs = probs[:keep]
    r = np.float32(rng.next_f32()) * probs.sum(dtype=np.float32)
    for i in range(keep):
        if r < probs[i]:
            return int(ids[i])
        r -= probs[i]
    return int(ids[keep - 1])


def sample(logits: np.ndarray, s: Sampling, recent, rng: Rng) -> int:
    """One token from a whole row of logits."""
    if s.greedy:
        return argmax(logits)
    l = np.array(logits, dtype=np.float32, copy=True)
    if s.repeat_penalty != 1.0:
        for t in list(recent)[-s.repeat_window:] if s.repeat_window > 0 else []:
            if 0 <= t < len(l):
                l[t] = _penalized(l[t], s.repeat_penalty)
    if s.temperature <= 0.0:
        return argmax(l)
    idx = np.argsort(-l, kind="stable")
    if s.top_k > 0:
        idx = idx[: s.top_k]
    return draw(idx, l[idx], s, rng)


@dataclass
class Candidates:
    """The top candidates of one row: ids by falling logit (lower id first among equals), every other token's
    logit at most `floor`, and the row's log-sum-exp (sampler.rs:105-124)."""
    ids: np.ndarray
    logits: np.ndarray
    lse: float
    vocab: int

    @property
    def floor(self) -> float:
        return float(self.logits[-1])

    def logprob(self, token: int) -> float | None:
        hit = np.nonzero(self.ids == token)[0]
        return float(self.logits[hit[0]] - self.lse) if len(hit) else None


def sample_sparse(c: Candidates, s: Sampling, recent, rng: Rng) -> int | None:
    """The token the dense sampler would pick when the candidates settle it, else None (the generator is
    advanced only when a token comes back).  sampler.rs:177-217."""
    k = len(c.ids)
    if k == 0:
        return None
    l = c.logits.astype(np.float32).copy()
    touched = np.zeros(k, dtype=bool)
    if s.repeat_penalty != 1.0:
        for t in list(recent)[-s.repeat_window:] if s.repeat_window > 0 else []:
            if t >= c.vocab or t < 0:
                continue
            hit = np.nonzero(c.ids == t)[0]
            if len(hit):
                l[hit[0]] = _penalized(l[hit[0]], s.repeat_penalty)
                touched[hit[0]] = True
            elif s.repeat_penalty < 1.0:
                return None
    order = sorted(range(k), key=lambda i: (-float(l[i]), int(c.ids[i])))
    certain = 0
    for i in order:
        if touched[i] and not (l[i] > c.floor):
            break
        certain += 1
    if certain == 0:
        return None
    if s.temperature <= 0.0:
        return int(c.ids[order[0]])
    if s.top_k == 0 or s.top_k > certain:
        return None
    sel = order[: s.top_k]
    return draw(c.ids[sel], l[sel], s, rng)
