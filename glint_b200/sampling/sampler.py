"""Sampling options, the per-request generator and the device sampler.

Options and their meaning are the reference's ``SamplerConfig`` (src/sampling/sampler.rs:79-116):
temperature 0 is greedy (the argmax of the raw logits, before any penalty, :181-183); top_k 0,
top_p 1.0, min_p 0.0 and repeat_penalty 1.0 switch their stage off; seed ``None`` seeds from the
clock (:134-146).  The generator is xorshift64 with a uniform from its upper 24 bits (:35-70); its
state is the request's own, kept in the request's slot on the device and advanced there, so that
batching never changes what it draws.
"""
from __future__ import annotations

import time
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


class TokenCounts:
    """How often each token occurs in a request's prompt and output, kept up to date as the output
    grows: the repeat penalty wants every past token with its count at every step, and counting
    thousands of tokens anew each time costs more than the step."""

    def __init__(self):
        self._reset()

    def _reset(self):
        self.index = {}                                  # token -> its place in the arrays
        self.tokens = np.empty(256, dtype=np.int32)
        self.counts = np.empty(256, dtype=np.int32)
        self.n = 0
        self.n_prompt = self.n_output = 0

    def _add(self, tok):
        at = self.index.get(tok)
        if at is not None:
            self.counts[at] += 1
            return
        if self.n == self.tokens.shape[0]:
            self.tokens = np.concatenate([self.tokens, np.empty_like(self.tokens)])
            self.counts = np.concatenate([self.counts, np.empty_like(self.counts)])
        self.index[tok] = self.n
        self.tokens[self.n] = tok
        self.counts[self.n] = 1
        self.n += 1

    def update(self, prompt, output):
        """Bring the counts up to ``prompt + output``; anything but a longer output starts over."""
        if len(prompt) != self.n_prompt or len(output) < self.n_output:
            self._reset()
            if len(prompt):
                toks, cnts = np.unique(np.asarray(prompt, dtype=np.int64), return_counts=True)
                self.tokens, self.counts = toks.astype(np.int32), cnts.astype(np.int32)
                self.n = len(toks)
                self.index = {int(t): i for i, t in enumerate(toks.tolist())}
            self.n_prompt = len(prompt)
        for tok in output[self.n_output:]:
            self._add(int(tok))
        self.n_output = len(output)
        return self

    def arrays(self):
        return self.tokens[:self.n], self.counts[:self.n]


def _counts_of(history):
    """(tokens, counts) int32 arrays of a row's history: a ``TokenCounts`` or a sequence of tokens."""
    if isinstance(history, TokenCounts):
        return history.arrays()
    if len(history) == 0:
        return np.empty(0, np.int32), np.empty(0, np.int32)
    toks, cnts = np.unique(np.asarray(history, dtype=np.int64), return_counts=True)
    return toks.astype(np.int32), cnts.astype(np.int32)


class DeviceSampler:
    """Chooses one token per logits row with the CUDA kernels of ``csrc/sampling.cu``.

    What a request needs for that lives in its slot, on the device: one record per request slot with
    its options, the state of its generator, its position and how many tokens were chosen for it
    (``attach`` declares the record to the cache manager, which zeroes it when a slot is taken;
    ``admit`` writes options and generator state once, when the request takes the slot).  Before the
    rows of a step are sampled one small kernel copies each row's options out of its slot's record,
    advances the generators of the rows that draw and hands the draws over; nothing about a row goes
    up from the host at every step except the repeat penalty's token counts.  The reference keeps
    position and generator state with the session (src/session/mod.rs:86,
    src/sampling/sampler.rs:35-37) and stores both in its snapshots (src/session/snapshot.rs:17-18).
    """

    HOST_WORDS = 8       # words of the record that the host writes at admission; the rest is the device's

    def __init__(self, rt, vocab_size, cache=None):
        self.rt = rt
        self.vocab_size = vocab_size
        self._work = None
        self._row_opts = None
        self._pen_stage = [None] * 4      # pinned buffers for the repeat penalty's lists
        self._pen_next = 0
        self.records = None
        self._host_records = None
        if cache is not None:
            self.attach(cache)

    # ---- the per-request record ---------------------------------------------------------------------

    def attach(self, cache):
        """Declare the per-request record to the cache manager, which owns the slots."""
        from ..cache import SlotStateNeed
        words = ops.sampler_record_words()
        self.records = cache.add_state("sampler", SlotStateNeed((words,), torch.int32))
        # one pinned row per slot: a slot's row is written again only after its last request has finished
        self._host_records = torch.zeros((cache.num_slots, words), dtype=torch.int32).pin_memory()
        self._copied = [None] * cache.num_slots       # per slot: the event behind the last copy of its row
        return self.records

    def admit(self, slot, params, rng_state, position=0, generated=0):
        """The request in ``slot`` samples with ``params`` and draws from a generator in ``rng_state``."""
        if self._copied[slot] is not None:
            self._copied[slot].synchronize()            # the row's previous copy has left the pinned buffer
        row = self._host_records[slot].numpy()
        row[:4].view(np.float32)[:] = (params.temperature, params.top_p, params.min_p, params.repeat_penalty)
        row[4] = params.top_k
        row[5] = 0 if params.greedy else 1
        state = int(rng_state) & _MASK64
        row[6:8].view(np.uint32)[:] = (state & 0xFFFFFFFF, state >> 32)
        row[8] = position
        row[9] = generated
        self.records[slot].copy_(self._host_records[slot], non_blocking=True)
        ev = self._copied[slot] or torch.cuda.Event()
        ev.record()
        self._copied[slot] = ev

    def slot_record(self, slot):
        """The record of ``slot`` read back from the device (waits for the GPU): a dictionary with the
        generator's state, the position and the count."""
        row = self.records[slot].cpu().numpy()
        lo, hi = row[6:8].view(np.uint32)
        return {"rng_state": int(lo) | (int(hi) << 32), "position": int(row[8]), "generated": int(row[9])}

    def generator_state(self, slot):
        return self.slot_record(slot)["rng_state"]

    # ---- scratch ------------------------------------------------------------------------------------

    def _scratch(self, rows):
        if self._work is None or self._work.shape[0] < rows:
            self._work = torch.empty((max(rows, 8), self.vocab_size), dtype=torch.float32, device=self.rt.device)
        return self._work[:rows]

    def _options(self, ctx, rows):
        """Per-row options and draws [7, rows] for the rows of the step ``ctx``, made on the device from
        the slots' records."""
        if self.records is None:
            raise RuntimeError("the sampler has no per-request records: call attach(cache) first")
        if self._row_opts is None or self._row_opts.shape[1] < rows:
            self._row_opts = torch.empty((7, max(rows, 64)), dtype=torch.float32, device=self.rt.device)
        # the first ``rows`` wanted rows of the step (rows that only fill a step up to a graph's size follow them)
        ops.sample_prepare(self.records, ctx.logit_slots[:rows], ctx.positions, ctx.logit_rows[:rows], self._row_opts)
        d = self._row_opts[:, :rows]
        return d, d[6].view(torch.int32)

    def _penalties(self, params, histories, penalty_row, dev):
        """The rows' (token, count) lists as one upload from a pinned buffer: offsets [rows + 1], tokens,
        counts.  None when no row has a penalty."""
        if histories is None or not any(p.repeat_penalty != 1.0 and not p.greedy for p in params):
            return None
        rows = len(params)
        offsets, toks, counts = [0], [], []
        for p, h in zip(params, histories):
            if p.repeat_penalty != 1.0 and not p.greedy:
                t, c = _counts_of(h)
                toks.append(t)
                counts.append(c)
                offsets.append(offsets[-1] + len(t))
            else:
                offsets.append(offsets[-1])
        n = offsets[-1]
        m = max(n, 1)
        size = rows + 1 + 2 * m
        k = self._pen_next
        self._pen_next = (k + 1) % len(self._pen_stage)
        host = self._pen_stage[k]
        if host is None or host.numel() < size:
            host = torch.empty(max(2 * size, 4096), dtype=torch.int32).pin_memory()
            self._pen_stage[k] = host
        pack = host.numpy()
        pack[:rows + 1] = offsets
        pack[rows + 1:rows + 1 + 2 * m] = 0
        if n:
            pack[rows + 1:rows + 1 + n] = np.concatenate(toks)
            pack[rows + 1 + m:rows + 1 + m + n] = np.concatenate(counts)
        d = host[:size].to(dev, non_blocking=True)
        return d[:rows + 1], d[rows + 1:rows + 1 + m], d[rows + 1 + m:rows + 1 + 2 * m], penalty_row

    def sample_device(self, logits, ctx, params, histories=None):
        """One token per row of ``logits`` (float32 [rows, vocab] on the device), left on the device
        (int32 [rows]); nothing waits for the GPU.  ``ctx`` is the context of the step that made the
        logits (which slot and position each row belongs to); ``params`` are the rows' ``SamplingParams``
        as admitted (the host only reads from them which kernels to launch); for the repeat penalty,
        ``histories`` holds the tokens so far (a sequence, or a ``TokenCounts`` that the caller keeps up
        to date)."""
        rows = logits.shape[0]
        dev = logits.device
        opt, top_k = self._options(ctx, rows)
        some_greedy = any(p.greedy for p in params)
        if some_greedy:
            chosen = torch.empty(rows, dtype=torch.int32, device=dev)
            ops.argmax(logits, chosen)
            if all(p.greedy for p in params):
                return chosen
        penalties = self._penalties(params, histories, opt[4], dev)
        drawn = torch.empty(rows, dtype=torch.int32, device=dev)
        ops.sample_rows(logits, self._scratch(rows), opt[0], top_k, opt[2], opt[3], opt[1], drawn, penalties)
        return torch.where(opt[5] > 0, drawn, chosen) if some_greedy else drawn

    def sample(self, logits, ctx, params, histories=None):
        """The same with the tokens brought to the host: a list of ints."""
        return [int(t) for t in self.sample_device(logits, ctx, params, histories).tolist()]
