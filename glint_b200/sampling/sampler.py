"""Sampling options, the per-request generator and the device sampler.

Options and their meaning are the reference's ``SamplerConfig`` (src/sampling/sampler.rs:79-116):
temperature 0 is greedy (the argmax of the raw logits, before any penalty, :181-183); top_k 0,
top_p 1.0, min_p 0.0 and repeat_penalty 1.0 switch their stage off; seed ``None`` seeds from the
clock (:134-146).  The generator is xorshift64 with a uniform from its upper 24 bits (:35-70); its
state is the request's own, kept with the request so that batching never changes what it draws.
"""
from __future__ import annotations

import time
from collections import Counter
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from .. import ops

_MASK64 = (1 << 64) - 1


@dataclass
class SamplingParams:
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    min_p: float = 0.0
    repeat_penalty: float = 1.0
    seed: Optional[int] = None

    def validate(self):
        if self.temperature < 0:
            raise ValueError("temperature must be >= 0")
        if self.top_k < 0:
            raise ValueError("top_k must be >= 0")
        if not 0.0 < self.top_p <= 1.0:
            raise ValueError("top_p must be in (0, 1]")
        if not 0.0 <= self.min_p <= 1.0:
            raise ValueError("min_p must be in [0, 1]")
        if not self.repeat_penalty > 0:
            raise ValueError("repeat_penalty must be > 0")

    @property
    def greedy(self):
        return self.temperature == 0.0


class Xorshift64:
    """s ^= s << 13; s ^= s >> 7; s ^= s << 17 on 64 bits; a zero seed becomes 1."""

    def __init__(self, seed=None):
        if seed is None:
            seed = time.time_ns()
        self.state = (int(seed) & _MASK64) or 1

    def next_u64(self):
        s = self.state
        s ^= (s << 13) & _MASK64
        s ^= s >> 7
        s ^= (s << 17) & _MASK64
        self.state = s
        return s

    def next_f32(self):
        return np.float32(self.next_u64() >> 40) / np.float32(1 << 24)


class DeviceSampler:
    """Chooses one token per logits row with the CUDA kernels of ``csrc/sampling.cu``."""

    def __init__(self, rt, vocab_size):
        self.rt = rt
        self.vocab_size = vocab_size
        self._work = None

    def _scratch(self, rows):
        if self._work is None or self._work.shape[0] < rows:
            self._work = torch.empty((max(rows, 8), self.vocab_size), dtype=torch.float32, device=self.rt.device)
        return self._work[:rows]

    def sample_device(self, logits, params, rngs):
        """Like ``sample`` for rows without a repeat penalty, but the chosen tokens stay on the
        device (int32 [rows]); nothing waits for the GPU.  Uniform draws are taken from the rows'
        generators now, so the stream of draws is the same as with ``sample``."""
        rows = logits.shape[0]
        dev = logits.device
        chosen = torch.empty(rows, dtype=torch.int32, device=dev)
        if all(p.greedy for p in params):
            ops.argmax(logits, chosen)
            return chosen
        ops.argmax(logits, chosen)
        temp = [p.temperature if not p.greedy else 1.0 for p in params]
        uniform = [float(r.next_f32()) if not p.greedy else 0.0 for p, r in zip(params, rngs)]
        pack = torch.tensor([temp, uniform, [p.top_p for p in params], [p.min_p for p in params],
                             [float(p.top_k) for p in params], [0.0 if p.greedy else 1.0 for p in params]],
                            dtype=torch.float32).pin_memory().to(dev, non_blocking=True)
        drawn = torch.empty(rows, dtype=torch.int32, device=dev)
        ops.sample(logits, self._scratch(rows), pack[0].contiguous(), pack[4].to(torch.int32), pack[2].contiguous(),
                   pack[3].contiguous(), pack[1].contiguous(), drawn)
        return torch.where(pack[5] > 0, drawn, chosen)

    def sample(self, logits, params, rngs, histories):
        """``logits`` float32 [rows, vocab] on the device; per row its ``SamplingParams``, its
        ``Xorshift64`` and the tokens so far (for the repeat penalty).  Returns a list of ints."""
        rows = logits.shape[0]
        dev = logits.device
        greedy_out = torch.empty(rows, dtype=torch.int32, device=dev)
        ops.argmax(logits, greedy_out)
        if all(p.greedy for p in params):
            return [int(t) for t in greedy_out.tolist()]
        temp = [p.temperature if not p.greedy else 1.0 for p in params]
        uniform = [float(r.next_f32()) if not p.greedy else 0.0 for p, r in zip(params, rngs)]
        work = self._scratch(rows)
        src = logits
        if any(p.repeat_penalty != 1.0 and not p.greedy for p in params):
            offsets, toks, counts = [0], [], []
            for p, h in zip(params, histories):
                if p.repeat_penalty != 1.0 and not p.greedy:
                    for tok, c in Counter(h).items():
                        toks.append(tok)
                        counts.append(c)
                offsets.append(len(toks))
            i32 = lambda v: torch.tensor(v or [0], dtype=torch.int32, device=dev)
            pen = torch.tensor([p.repeat_penalty for p in params], dtype=torch.float32, device=dev)
            ops.apply_penalty(logits, work, i32(offsets), i32(toks), i32(counts), pen)
            src = work
        f32 = lambda v: torch.tensor(v, dtype=torch.float32, device=dev)
        out = torch.empty(rows, dtype=torch.int32, device=dev)
        ops.sample(src, work, f32(temp), torch.tensor([p.top_k for p in params], dtype=torch.int32, device=dev),
                   f32([p.top_p for p in params]), f32([p.min_p for p in params]), f32(uniform), out)
        drawn, greedy = out.tolist(), greedy_out.tolist()
        return [int(g if p.greedy else d) for p, g, d in zip(params, greedy, drawn)]
