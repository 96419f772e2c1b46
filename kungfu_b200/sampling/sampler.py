"""Sampling rules of a request and the per-request state the device draws from.

The rules and their defaults are the reference's `Sampling` (crates/kf-engine/src/sampler.rs:4-17): temperature 0.7,
top_k 40, top_p 0.95, min_p 0, repeat penalty 1 over a window of 64 tokens; temperature <= 0 without a penalty is
greedy.  The draw itself runs on the device at the end of the step that produced the logits (`ops.sample`, kernels in
csrc/sampling.cu): nothing of a row of logits travels to the host.  What the kernels need per request lives in one
block of 32-bit words on the device, written here when a request is admitted and kept up to date by the kernels
themselves (they advance the generator and append each token they draw):

  [0,1]  state of the xorshift64 generator, seeded with max(seed, 1) (sampler.rs:20-34)
  [2..5] temperature, top_p, min_p, repeat_penalty (32-bit floats)
  [6,7]  top_k, repeat_window
  [8]    tokens recorded so far     [16..272) the last 256 of them, token i at word 16 + i % 256

A plain restatement of the rules, for tests, is tests/plain_sampler.py; the package ships no host sampler.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

CANDIDATES = 64          # reference: TOP = 64, crates/kf-engine/src/session.rs:80
STATE_WORDS = 272
RING = 256
_RING0 = 16
_MASK64 = (1 << 64) - 1


@dataclass
class Sampling:
    temperature: float = 0.7
    top_k: int = 40
    top_p: float = 0.95
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    repeat_window: int = 64

    def __post_init__(self):
        if self.top_k < 0:
            raise ValueError(f"top_k {self.top_k} must be 0 (all) or positive")
        if not (0.0 < self.top_p <= 1.0):
            raise ValueError(f"top_p {self.top_p} must lie in (0, 1]")
        if not (0.0 <= self.min_p <= 1.0):
            raise ValueError(f"min_p {self.min_p} must lie in [0, 1]")
        if not self.repeat_penalty > 0.0:
            raise ValueError(f"repeat_penalty {self.repeat_penalty} must be positive")
        if not (0 <= self.repeat_window <= RING):
            raise ValueError(f"repeat_window {self.repeat_window} must lie in 0..{RING} (what the device keeps per request)")

    @property
    def greedy(self) -> bool:
        return self.temperature <= 0.0 and self.repeat_penalty == 1.0

    @property
    def needs_whole_ranking(self) -> bool:
        """Whether a draw can reach below the 64th candidate of a row (the device then runs one more kernel)."""
        return self.temperature > 0.0 and (self.top_k == 0 or self.top_k > CANDIDATES)


def pack_state(sampling: Sampling, seed: int, recent=()) -> np.ndarray:
    """The device state of a request: its rules, a generator seeded with `seed`, and the tokens it has produced so far
    (`recent`, e.g. after a preemption)."""
    st = np.zeros(STATE_WORDS, dtype=np.int32)
    x = max(int(seed), 1) & _MASK64
    st[0:2] = np.array([x & 0xFFFFFFFF, x >> 32], dtype=np.uint32).view(np.int32)
    st[2:6] = np.array([sampling.temperature, sampling.top_p, sampling.min_p, sampling.repeat_penalty], dtype=np.float32).view(np.int32)
    st[6], st[7] = int(sampling.top_k), int(sampling.repeat_window)
    recent = [int(t) for t in recent]
    st[8] = len(recent)
    for i in range(max(0, len(recent) - RING), len(recent)):
        st[_RING0 + i % RING] = recent[i]
    return st


def generator_state(state: np.ndarray) -> int:
    w = np.asarray(state[0:2], dtype=np.int32).view(np.uint32)
    return int(w[0]) | (int(w[1]) << 32)
