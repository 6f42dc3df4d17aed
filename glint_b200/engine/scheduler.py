"""Continuous batching above the step function.

The reference's engine loop (src/server/engine.rs:449-671) admits requests first-come while
fewer than ``max_active`` run (:489-511), prefills each prompt whole and alone (:740-844),
then decodes one token per live sequence per step in one batch (:650-669); it samples from the
previous step's logits at the top of the loop (:543-566); a sequence finishes on its token
budget, on EOS (the EOS token is delivered) or at the context length (:548-578); when pages
run out in mid-decode that sequence ends with ``length`` and keeps what it produced
(:637-643, test :1123-1151).

This scheduler keeps those rules and adds what the reference leaves open: prompts are cut
into portions under a token budget per step and share steps with decoding requests, and
admission waits (instead of rejecting) while slots or pages are short.  Order within a step:
decoding requests first, then running prompts in admission order, then new admissions.

When pages run out: a request that cannot get pages for its next tokens waits while others
free pages; if nobody can run, the request admitted last is preempted — its pages and slot
are given back and it returns to the head of the queue with its produced tokens appended to
its prompt, to be recomputed; a request that cannot run even alone on an empty cache ends
with ``length`` and keeps what it produced.
"""
from __future__ import annotations

import time
from collections import deque
from dataclasses import dataclass, field
from typing import Optional

from ..errors import RequestError
from ..sampling import SamplingParams, TokenCounts, Xorshift64
from .step import StepEntry

FINISH_STOP = "stop"        # sampled the EOS token
FINISH_LENGTH = "length"    # token budget, context length, or the cache cannot hold it
FINISH_ABORTED = "aborted"


@dataclass
class Request:
    rid: object
    prompt: list
    max_tokens: int
    params: SamplingParams = field(default_factory=SamplingParams)
    eos_token_id: Optional[int] = None
    output: list = field(default_factory=list)
    finish_reason: Optional[str] = None
    slot: Optional[int] = None
    computed: int = 0            # tokens of prompt + output that are in the cache
    preemptions: int = 0
    rng_state: Optional[int] = None   # state of its xorshift64 generator when it takes a slot (the device advances it)
    order: int = 0
    unresolved: int = 0          # 1 while the newest token is still only on the device
    pending_index: int = 0       # its place among the tokens sampled by that step
    counts: Optional[TokenCounts] = None   # token counts for the repeat penalty, made at first use
    draining: bool = False       # reached its budget by count; finishes when its last token arrives
    t_submit: float = 0.0        # time.perf_counter() when it was queued, when its first token reached the host,
    t_first: float = 0.0         # and when it finished (time to first token, time per output token)
    t_finish: float = 0.0

    @property
    def tokens(self):
        return self.prompt + self.output

    def token_counts(self):
        """Counts of the tokens so far for the repeat penalty, brought up to date."""
        if self.counts is None:
            self.counts = TokenCounts()
        return self.counts.update(self.prompt, self.output)

    @property
    def num_tokens(self):
        return len(self.prompt) + len(self.output) + self.unresolved

    @property
    def generated(self):
        return len(self.output) + self.unresolved

    def token_slice(self, lo, hi):
        """tokens[lo:hi] without building the whole list."""
        n = len(self.prompt)
        if hi <= n:
            return self.prompt[lo:hi]
        if lo >= n:
            return self.output[lo - n:hi - n]
        return self.prompt[lo:] + self.output[:hi - n]

    @property
    def finished(self):
        return self.finish_reason is not None


class Scheduler:
    """``engine`` offers ``open()``, ``close(slot)``, ``step(entries) -> logits``, ``cache`` and
    ``last_ctx`` (the context of the step that ran last); ``sampler.sample(logits, ctx, params,
    histories) -> tokens``.  A sampler that keeps per-request state in the slots also offers
    ``admit(slot, params, rng_state, position, generated)`` and ``generator_state(slot)``."""

    def __init__(self, engine, sampler, max_step_tokens=2048, max_active=None, context_length=None,
                 lookahead=False):
        self.engine = engine
        self.sampler = sampler
        # With ``lookahead`` the next step is launched with the sampled tokens still on the device,
        # and the host reads them one step late (EOS is then seen one step late: the extra row is
        # discarded).  Needs a sampler with ``sample_device(logits, ctx, params, histories)``.
        self.lookahead = bool(lookahead) and hasattr(sampler, "sample_device")
        self._pending = None
        self._host_tokens = [None, None]
        self._host_flip = 0
        self.max_step_tokens = int(max_step_tokens)
        self.max_active = int(max_active or getattr(engine, "num_slots", engine.cache.num_slots))
        self.context_length = int(context_length or engine.cache.max_positions)
        self.waiting = deque()
        self.running = []
        self.finished = []
        self._order = 0
        self.counters = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "preemptions": 0}
        self.step_log = deque(maxlen=4096)   # per step: wall seconds, rows, bytes copied each way

    # ---- submission -------------------------------------------------------------------------------

    def add(self, request):
        """Queue a request.  An empty prompt or one longer than the context is refused at once
        (the reference drops them with ``Incomplete``, src/server/engine.rs:752-754)."""
        if len(request.prompt) == 0:
            raise RequestError("empty prompt")
        if len(request.prompt) > self.context_length:
            raise RequestError(f"prompt of {len(request.prompt)} tokens exceeds the context length "
                               f"{self.context_length}")
        request.params.validate()
        if request.max_tokens <= 0:
            request.finish_reason = FINISH_LENGTH
            self.finished.append(request)
            return
        if request.rng_state is None:
            request.rng_state = Xorshift64(request.params.seed).state
        request.order = self._order
        request.t_submit = time.perf_counter()
        self._order += 1
        self.waiting.append(request)

    @property
    def idle(self):
        return not self.waiting and not self.running and self._pending is None

    # ---- planning ---------------------------------------------------------------------------------

    def plan(self):
        """Decide the next step: a list of (request, number of tokens).  The decision itself (decoding
        requests first, running prompts under the budget, admissions while slots and pages allow) is the
        cache core's (``CacheManager.plan``, C++); this admits the requests it names (taking slots) but takes
        no pages: ``engine.step`` reserves them all-or-nothing, and the plan only holds rows that the cache can
        serve together."""
        cache = self.engine.cache
        running = [(r.slot, r.num_tokens - r.computed, r.computed == r.num_tokens - 1 and r.generated > 0)
                   for r in self.running]
        waiting = [r.num_tokens - r.computed for r in self.waiting]
        run_counts, admit_counts = cache.plan(self.max_step_tokens, self.max_active, running, waiting)
        decoders = [(r, n) for r, n, row in zip(self.running, run_counts, running) if n and row[2]]
        portions = [(r, n) for r, n, row in zip(self.running, run_counts, running) if n and not row[2]]
        rows = decoders + portions
        for n in admit_counts:
            r = self.waiting.popleft()
            r.slot = self.engine.open()
            self.running.append(r)
            if hasattr(self.sampler, "admit"):       # options and generator state go into the slot, once
                self.sampler.admit(r.slot, r.params, r.rng_state, r.computed, len(r.output))
            rows.append((r, n))
        return rows

    def _preempt_or_finish(self):
        """Nobody can run.  Free the request admitted last; if it is alone on an empty cache it
        can never run: end it with ``length``."""
        self._resolve()
        if not self.running:
            if not self.waiting:
                return
            r = self.waiting.popleft()   # cannot even be admitted alone
            self._finish(r, FINISH_LENGTH)
            return
        victim = max(self.running, key=lambda r: r.order)
        alone = len(self.running) == 1
        self.running.remove(victim)
        if hasattr(self.sampler, "generator_state"):   # its generator goes on from where it stands
            victim.rng_state = self.sampler.generator_state(victim.slot)
        self.engine.close(victim.slot)
        victim.slot = None
        victim.computed = 0
        if alone:
            self._finish(victim, FINISH_LENGTH)
        else:
            victim.preemptions += 1
            self.counters["preemptions"] += 1
            self.waiting.appendleft(victim)

    def _finish(self, r, reason):
        r.finish_reason = reason
        r.t_finish = time.perf_counter()
        if r.slot is not None:
            self.engine.close(r.slot)
            r.slot = None
        if r in self.running:
            self.running.remove(r)
        self.finished.append(r)

    # ---- one step ---------------------------------------------------------------------------------

    def step(self):
        """Plan, run and sample one step.  Returns the requests that finished in it."""
        if self.lookahead:
            return self._step_lookahead()
        self._resolve()
        done_before = len(self.finished)
        rows = self.plan()
        while not rows and not self.idle:
            self._preempt_or_finish()
            rows = self.plan()
        if not rows:
            return self.finished[done_before:]
        t_start = time.perf_counter()
        entries, sampled = [], []
        n_decode = n_prefill = 0
        for r, n in rows:
            toks = r.token_slice(r.computed, r.computed + n)
            last = r.computed + n == r.num_tokens
            entries.append(StepEntry(r.slot, toks, [n - 1] if last else []))
            if last:
                sampled.append(r)
            if r.output and n == 1 and last:
                n_decode += 1
            else:
                n_prefill += n
        logits = self.engine.step(entries)
        self.counters["steps"] += 1
        self.counters["decode_tokens"] += n_decode
        self.counters["prefill_tokens"] += n_prefill
        for r, n in rows:
            r.computed += n
        if sampled:
            histories = [r.token_counts() if (r.params.repeat_penalty != 1.0 and not r.params.greedy) else ()
                         for r in sampled]
            tokens = self.sampler.sample(logits, getattr(self.engine, "last_ctx", None), [r.params for r in sampled],
                                         histories)
            for r, tok in zip(sampled, tokens):
                r.output.append(int(tok))
                if r.t_first == 0.0:
                    r.t_first = time.perf_counter()
                # the reference's order of checks (src/server/engine.rs:548-578)
                if r.eos_token_id is not None and tok == r.eos_token_id:
                    self._finish(r, FINISH_STOP)
                elif len(r.output) >= r.max_tokens:
                    self._finish(r, FINISH_LENGTH)
                elif r.num_tokens >= self.context_length:
                    self._finish(r, FINISH_LENGTH)
        t_end = time.perf_counter()
        self.step_log.append({"seconds": t_end - t_start, "t_end": t_end, "decode_rows": n_decode,
                              "prefill_tokens": n_prefill,
                              "h2d_bytes": getattr(self.engine, "last_h2d_bytes", 0),
                              "d2h_bytes": 4 * len(sampled)})
        return self.finished[done_before:]

    # ---- one step with the sampled tokens left on the device ------------------------------------------

    def _resolve(self):
        """Read the tokens of the pending step (waits for it) and draw the consequences: append,
        EOS, budget.  A request that met EOS keeps nothing of the step launched meanwhile."""
        pend = self._pending
        if pend is None:
            return
        self._pending = None
        dev, host, event, sampled = pend
        event.synchronize()
        tokens = host[:len(sampled)].tolist()
        for r, tok in zip(sampled, tokens):
            if r.finished:
                continue                       # met EOS a step ago; this token is the discarded one
            r.output.append(int(tok))
            r.unresolved = 0
            if r.t_first == 0.0:
                r.t_first = time.perf_counter()
            if r.eos_token_id is not None and tok == r.eos_token_id:
                self._finish(r, FINISH_STOP)
            elif r.draining:
                self._finish(r, FINISH_LENGTH)

    def _step_lookahead(self):
        import torch
        done_before = len(self.finished)
        rows = self.plan()
        while not rows and not self.idle:
            if self._pending is not None:
                self._resolve()                # frees what finished; the plan may now have rows
            else:
                self._preempt_or_finish()
            rows = self.plan()
        if not rows:
            return self.finished[done_before:]
        t_start = time.perf_counter()
        entries, sampled, src_idx, dst_rows = [], [], [], []
        n_decode = n_prefill = offset = 0
        for r, n in rows:
            last = r.computed + n == r.num_tokens
            if r.unresolved:                   # its newest token is the pending step's, on the device
                toks = [0]
                src_idx.append(r.pending_index)
                dst_rows.append(offset)
            else:
                toks = r.token_slice(r.computed, r.computed + n)
            entries.append(StepEntry(r.slot, toks, [n - 1] if last else []))
            if last:
                sampled.append(r)
            if r.generated and n == 1 and last:
                n_decode += 1
            else:
                n_prefill += n
            offset += n
        prev = self._pending
        placed = (prev[0], src_idx, dst_rows) if src_idx else None
        logits = self.engine.step(entries, device_tokens=placed)
        self.counters["steps"] += 1
        self.counters["decode_tokens"] += n_decode
        self.counters["prefill_tokens"] += n_prefill
        for r, n in rows:
            r.computed += n
        # The previous step's tokens: they were this step's input, so they have long arrived, and the
        # repeat penalty of this step's rows counts them.
        self._resolve()
        new_pending = None
        if sampled:
            histories = [r.token_counts() if (r.params.repeat_penalty != 1.0 and not r.params.greedy) else ()
                         for r in sampled]
            dev = self.sampler.sample_device(logits, self.engine.last_ctx, [r.params for r in sampled], histories)
            k = self._host_flip
            self._host_flip ^= 1
            host = self._host_tokens[k]
            if host is None or host.numel() < len(sampled):
                host = torch.empty(max(len(sampled), self.max_active), dtype=torch.int32).pin_memory()
                self._host_tokens[k] = host
            host[:len(sampled)].copy_(dev, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
            new_pending = (dev, host, event, list(sampled))
        for i, r in enumerate(sampled):
            if r.finished:
                continue                       # EOS came to light just now: this step's row is void
            r.unresolved = 1
            r.pending_index = i
            if r.generated >= r.max_tokens or r.num_tokens >= self.context_length:
                r.draining = True              # no further rows; it finishes when this token arrives
                self.running.remove(r)
        self._pending = new_pending
        t_end = time.perf_counter()
        self.step_log.append({"seconds": t_end - t_start, "t_end": t_end, "decode_rows": n_decode,
                              "prefill_tokens": n_prefill,
                              "h2d_bytes": getattr(self.engine, "last_h2d_bytes", 0),
                              "d2h_bytes": 4 * len(sampled)})
        return self.finished[done_before:]

    def run(self):
        """Step until every queued request has finished; returns them in finishing order."""
        start = len(self.finished)
        while not self.idle:
            self.step()
        return self.finished[start:]

    def abort(self, request):
        if request in self.waiting:
            self.waiting.remove(request)
        self._finish(request, FINISH_ABORTED)
