"""Plain restatement of the reference sampler, in Python lists and floats.

Rests on the formulas of HamadAndrabi/glint's src/sampling/sampler.rs (read,
never run: no Rust toolchain here).  Shares no code with ``glint_b200``.
32-bit float arithmetic is mimicked with numpy.float32 where the order of
operations matters (the running sum of the CDF walk).
"""
from __future__ import annotations

import math

import numpy as np

MASK64 = (1 << 64) - 1


class Xorshift64:
    """s ^= s<<13; s ^= s>>7; s ^= s<<17; seed 0 becomes 1
    (src/sampling/sampler.rs:35-70)."""

    def __init__(self, seed):
        self.state = (seed & MASK64) or 1

    def next_u64(self):
        s = self.state
        s ^= (s << 13) & MASK64
        s ^= s >> 7
        s ^= (s << 17) & MASK64
        self.state = s
        return s

    def next_f32(self):
        """Upper 24 bits over 2^24 (src/sampling/sampler.rs:66-69)."""
        return np.float32(self.next_u64() >> 40) / np.float32(1 << 24)


def argmax(logits):
    """Last of equal maxima wins: ``max_by`` keeps the later element
    (src/sampling/sampler.rs:245-252)."""
    best, idx = None, 0
    for i, v in enumerate(logits):
        if best is None or v >= best:
            best, idx = v, i
    return idx


def sample(logits, past_tokens, rng, temperature=0.0, top_k=0, top_p=1.0, min_p=0.0,
           repeat_penalty=1.0):
    """penalty -> temperature -> top-k -> min-p -> softmax -> top-p -> draw
    (src/sampling/sampler.rs:179-235 with the stages of :254-388)."""
    x = np.asarray(logits, dtype=np.float32).copy()
    if temperature == 0.0:
        return argmax(x)
    if repeat_penalty != 1.0:
        pen = np.float32(repeat_penalty)
        for t in past_tokens:  # once per occurrence, as the reference loops (:262-273)
            if t < len(x):
                x[t] = x[t] / pen if x[t] > 0 else x[t] * pen
    if temperature != 1.0:
        x = x * (np.float32(1.0) / np.float32(temperature))
    if top_k > 0 and top_k < len(x):
        order = np.argsort(-x, kind="stable")
        x[order[top_k:]] = -np.inf
    if min_p > 0.0:
        thr = x.max() + np.float32(math.log(min_p))
        x[x < thr] = -np.inf
    e = np.exp(x - x.max()).astype(np.float32)
    total = e.sum(dtype=np.float32)
    probs = e / total if total > 0 and not np.isnan(total) else np.full_like(e, 1.0 / len(e))
    if top_p < 1.0:
        order = np.argsort(-probs, kind="stable")
        cum = np.float32(0.0)
        cutoff = len(order)
        for rank, i in enumerate(order):
            cum = np.float32(cum + probs[i])
            if cum >= np.float32(top_p):
                cutoff = rank + 1
                break
        kept = np.zeros_like(probs)
        kept[order[:cutoff]] = probs[order[:cutoff]]
        s = kept.sum(dtype=np.float32)
        probs = kept / s if s > 0 else kept
    r = rng.next_f32()
    cum = np.float32(0.0)
    for i, p in enumerate(probs):
        cum = np.float32(cum + p)
        if r < cum:
            return i
    return len(probs) - 1
