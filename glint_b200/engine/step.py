"""The step function: one batch of (request, its next tokens) through the model, from the cache.

The reference has three calls: a whole prompt (or its tail from ``pos_offset``) of one
sequence, one token of one sequence, one token each of many sequences
(src/transformer/forward.rs:694-703, :435-444, :1328-1337); prompts of different requests are
never batched.  Here one ``step`` takes any mix: portions of prompts beside single decoded
tokens, cut anywhere.  As in the reference, the keys and values of all tokens of the step are
written first and then every token attends its request's cache up to its own position
(:875-877, :927-972).  Logits are computed only for the rows that are asked for.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache import CacheManager
from ..errors import RequestError


@dataclass
class StepEntry:
    """The next ``tokens`` of the request in ``slot``; ``want`` lists the places among these
    tokens whose logits are returned, in order."""
    slot: int
    tokens: list
    want: list = field(default_factory=list)


def _align4(n):
    return (n + 3) & ~3


def padded_size(n):
    """The batch size whose graph a step of ``n`` single tokens replays: itself up to 8, then the next
    multiple of 4 up to 32, of 8 up to 64, of 16 beyond.  A serving run whose batch shrinks request by request
    then captures a dozen graphs instead of one per size (each capture holds the GPU idle for milliseconds)."""
    if n <= 8:
        return n
    if n <= 32:
        return (n + 3) & ~3
    if n <= 64:
        return (n + 7) & ~7
    return (n + 15) & ~15


def _uneven(contexts):
    """How far the contexts of a step's single tokens fall short of the longest of them: 0 when they add
    up to more than 0.7 of (their number x the longest), 1 down to 0.35, 2 down to 0.175, else 3.  The
    split attention kernel shares a long context among more blocks when most others are short."""
    if not contexts:
        return 0
    share, level, bound = sum(contexts) / (len(contexts) * max(contexts)), 0, 0.7
    while level < 3 and share <= bound:
        level, bound = level + 1, bound / 2
    return level


class StepContext:
    """Everything about one step that parts may read.  Device tensors are int32.

    ``token_ids``, ``positions``, ``token_seq`` are per token; ``token_seq`` is the index of the
    token's request within this step, which is also its row in every block table.
    ``seq_slot``, ``seq_start`` (tokens cached before the step), ``cu_seqlens`` (token offsets,
    one more than requests) are per request; ``logit_rows`` are the token rows whose logits are
    wanted and ``logit_slots`` the request slots of those rows.  ``leading_single`` counts the requests at the front of the step that bring a single
    token (a scheduler puts its decoding requests first), ``leading_single_context`` is the longest
    context among them and ``uneven`` says how far the others fall short of it.  The ``h_`` fields are host copies for
    planning launches.  ``memo`` is empty at the start of
    a step: parts keep there what several layers of the step share (a table of rotation angles, say),
    under a key of their own parameters.
    """

    def __init__(self, cache, entries, meta_dev, staging, extra=()):
        n = len(entries)
        self.memo = {}
        lens = [len(e.tokens) for e in entries]
        T = sum(lens)
        self.num_tokens, self.num_seqs = T, n
        self.h_seq_lens = lens
        self.h_seq_slot = [e.slot for e in entries]
        self.h_seq_start = [cache.length(e.slot) for e in entries]
        self.h_cu_seqlens = [0]
        for l in lens:
            self.h_cu_seqlens.append(self.h_cu_seqlens[-1] + l)
        self.max_seq_len = max(lens)
        self.leading_single = next((i for i, l in enumerate(lens) if l != 1), n)   # requests in front that bring one token
        self.max_context = max(s + l for s, l in zip(self.h_seq_start, lens))
        self.leading_single_context = max([s + 1 for s in self.h_seq_start[:self.leading_single]] or [0])
        self.uneven = _uneven([s + 1 for s in self.h_seq_start[:self.leading_single]])
        rows, row_slots = [], []
        for i, e in enumerate(entries):
            for w in e.want:
                if not 0 <= w < lens[i]:
                    raise RequestError(f"wanted place {w} lies outside the {lens[i]} tokens given")
                rows.append(self.h_cu_seqlens[i] + w)
                row_slots.append(e.slot)
        self.num_logit_rows = len(rows)
        self.is_decode = self.max_seq_len == 1
        self._groups = cache.groups
        tables = cache.block_tables(self.h_seq_slot)
        max_pages = [t.shape[1] for t in tables]

        # one packed int32 buffer -> one copy to the device
        sizes = [T, T, T, n, n, n + 1, len(rows), len(rows)] + [n * mp for mp in max_pages] + [len(x) for x in extra]
        offs, total = [], 0
        for s in sizes:
            offs.append(total)
            total += _align4(max(s, 1))
        pack = staging(total)
        ids = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries])
        pack[offs[0]:offs[0] + T] = ids
        pos = np.concatenate([np.arange(s, s + l, dtype=np.int64) for s, l in zip(self.h_seq_start, lens)])
        pack[offs[1]:offs[1] + T] = pos
        pack[offs[2]:offs[2] + T] = np.repeat(np.arange(n, dtype=np.int64), lens)
        pack[offs[3]:offs[3] + n] = self.h_seq_slot
        pack[offs[4]:offs[4] + n] = self.h_seq_start
        pack[offs[5]:offs[5] + n + 1] = self.h_cu_seqlens
        if rows:
            pack[offs[6]:offs[6] + len(rows)] = rows
            pack[offs[7]:offs[7] + len(rows)] = row_slots
        for g, t in enumerate(tables):
            pack[offs[8 + g]:offs[8 + g] + t.size] = t.reshape(-1)
        first_extra = 8 + len(tables)
        for k, x in enumerate(extra):
            if len(x):
                pack[offs[first_extra + k]:offs[first_extra + k] + len(x)] = x
        dev = meta_dev(pack, total)
        self.h2d_bytes = total * 4
        cut = lambda k, size: dev[offs[k]:offs[k] + size]
        self.token_ids = cut(0, T)
        self.positions = cut(1, T)
        self.token_seq = cut(2, T)
        self.seq_slot = cut(3, n)
        self.seq_start = cut(4, n)
        self.cu_seqlens = cut(5, n + 1)
        self.logit_rows = cut(6, len(rows))
        self.logit_slots = cut(7, len(rows))
        self.block_tables = [cut(8 + g, n * mp).view(n, mp) for g, mp in enumerate(max_pages)]
        self.extra = [cut(first_extra + k, len(x)) for k, x in enumerate(extra)]

    @property
    def groups(self):
        """The cache manager's paged groups, in the order of ``block_tables``."""
        return self._groups

    def block_table(self, group):
        """Device block table [requests of this step, max pages] of a cache group."""
        for g, t in zip(self._groups, self.block_tables):
            if g is group:
                return t
        raise KeyError(group.name)


class Engine:
    """A model, its cache and the step function.  Requests are known here only by slot."""

    def __init__(self, model, num_pages, num_slots=64, page_size=16, use_graphs=True):
        self.model = model
        self.use_graphs = use_graphs
        self._graphs = {}
        self._graph_pool = None
        self.rt = model.rt
        needs, cache_of = model.cache_needs()
        # With graphs, steps of single tokens are padded to a few batch sizes (see padded_size): the rows
        # that fill a step up belong to a slot and a page of their own, beyond what the caller asked for.
        spare = 1 if use_graphs else 0
        self.cache = CacheManager(needs, cache_of, num_slots + spare, num_pages + spare, page_size,
                                  model.spec.max_positions, self.rt.dtype, self.rt.device)
        self.num_slots = num_slots
        from .. import ops
        self._fallbacks_before = ops.fallbacks()
        self._pad_entry = None
        if use_graphs:
            slot = self.cache.alloc_slot()
            self.cache.reserve([(slot, 1)])             # one page in every group, position 0, never advanced
            for g in self.cache.groups:
                g.pool.hidden = 1
            self._pad_entry = StepEntry(slot, [0], [0])
        self.vocab_size = model.spec.vocab_size
        self._meta_dev = None
        self._staging = []
        self._staging_events = []
        self._staging_next = 0
        self.steps = 0
        self.graph_counts = {"eager": 0, "first_sight": 0, "captured": 0, "replayed": 0}
        self.tokens_run = 0
        self.last_h2d_bytes = 0
        self.last_ctx = None          # the context of the step that ran last (its device arrays stay valid until the next step)

    # ---- request slots ----------------------------------------------------------------------------

    def open(self):
        """Admit a request: returns its slot."""
        return self.cache.alloc_slot()

    def close(self, slot):
        """The request is finished: its pages and its slot are given back."""
        self.cache.free_slot(slot)

    # ---- metadata staging -------------------------------------------------------------------------

    def _stage(self, total):
        """A pinned int32 host buffer of at least ``total`` elements that no copy in flight reads."""
        k = self._staging_next
        if len(self._staging) < 4:
            self._staging.append(None)
            self._staging_events.append(None)
            k = len(self._staging) - 1
        self._staging_next = (k + 1) % 4
        if self._staging_events[k] is not None:
            self._staging_events[k].synchronize()
        buf = self._staging[k]
        if buf is None or buf.numel() < total:
            buf = torch.empty(max(total, 4096), dtype=torch.int32).pin_memory()
            self._staging[k] = buf
        self._staging_current = k
        return buf.numpy()

    def _upload(self, pack, total):
        if self._meta_dev is None or self._meta_dev.numel() < total:
            groups = len(self.cache.groups)
            roomy = 3 * 16384 + self.cache.num_slots * (8 + groups * max([g.max_pages for g in self.cache.groups] or [0]))
            self._meta_dev = torch.empty(max(total * 2, roomy), dtype=torch.int32, device=self.rt.device)
            self._graphs.clear()      # captured launches point into the old buffer
        k = self._staging_current
        self._meta_dev[:total].copy_(self._staging[k][:total], non_blocking=True)
        ev = self._staging_events[k] or torch.cuda.Event()
        ev.record()
        self._staging_events[k] = ev
        return self._meta_dev

    # ---- the step ---------------------------------------------------------------------------------

    def validate(self, entries):
        if not entries:
            raise RequestError("a step needs at least one entry")
        seen = set()
        for e in entries:
            if e.slot in seen:
                raise RequestError(f"slot {e.slot} appears twice in one step")
            seen.add(e.slot)
            if len(e.tokens) == 0:
                raise RequestError("an entry without tokens")
            if len(e.tokens) == 1:
                lo = hi = e.tokens[0]
            else:
                lo, hi = min(e.tokens), max(e.tokens)
            if lo < 0 or hi >= self.vocab_size:
                raise RequestError(f"token id {lo if lo < 0 else hi} lies outside the vocabulary of "
                                   f"{self.vocab_size}")

    def step(self, entries, device_tokens=None):
        """Run the entries as one batch.  Returns float32 logits [wanted rows, vocab] on the
        device, in the order of the entries and of each ``want`` (``None`` if nothing is wanted).
        The tensor is valid until the next step.  ``device_tokens`` (int32 on the device, one
        per token of the step) replaces the entries' token ids, for callers whose tokens never
        leave the device (the entries then carry placeholders of the right count).  A tuple
        ``(source, source_indices, token_rows)`` replaces only the listed token rows, each with
        ``source[source_indices[i]]``.

        Raises ``PagePoolExhausted`` before anything ran when the cache cannot hold the new
        tokens; the cache is then unchanged apart from pages that a window had already passed.
        """
        self.validate(entries)
        rows = [(e.slot, len(e.tokens)) for e in entries]
        self.cache.reserve(rows)
        n_real = len(entries)
        real_tokens = sum(n for _, n in rows)
        if self._graphable(entries):
            # a step of single tokens replays a graph captured for its padded size: the rows behind the
            # caller's are one token at position 0 of the spare slot, and their logits are dropped
            entries = list(entries) + [self._pad_entry] * (padded_size(n_real) - n_real)
        with torch.cuda.device(self.rt.device):
            placed = isinstance(device_tokens, tuple)      # (source tensor, source indices, token rows)
            extra = (device_tokens[1], device_tokens[2]) if placed else ()
            ctx = StepContext(self.cache, entries, self._upload, self._stage, extra)
            if placed:
                from .. import ops
                if len(device_tokens[1]):
                    ops.place_tokens(ctx.token_ids, ctx.extra[1], device_tokens[0], ctx.extra[0])
            elif device_tokens is not None:
                ctx.token_ids[:real_tokens].copy_(device_tokens, non_blocking=True)
            if self.model.program(self.cache, ctx.num_tokens, ctx.num_logit_rows)[2]:
                self._graphs.clear()      # the values moved: captured launches point into the old ones
            key = self._graph_key(entries, ctx)
            if key is None:
                self.graph_counts["eager"] += 1
                logits = self.model.forward(ctx, self.cache)
            else:
                logits = self._run_graphed(key, ctx)
                if len(entries) > n_real:
                    logits = logits[:n_real]
        self.cache.advance(rows)
        self.steps += 1
        if self.steps == 1 and self.rt.tensor_cores:
            self._note_fallbacks()
        self.tokens_run += real_tokens
        self.last_h2d_bytes = ctx.h2d_bytes
        self.last_ctx = ctx
        return logits

    def _note_fallbacks(self):
        """Say once, after the first step, if sizes of this model kept operations off the tensor cores."""
        import sys
        from .. import ops
        n = ops.fallbacks() - self._fallbacks_before
        if n > 0:
            print(f"[glint_b200] note: {n} operations of the first step ran on CUDA-core kernels although the engine "
                  f"is bfloat16: no tensor-core kernel takes their sizes (products want K in steps of 8, attention "
                  f"head sizes in steps of 16 up to 256); results are right, speed is not", file=sys.stderr, flush=True)

    # ---- CUDA graphs for decode steps -------------------------------------------------------------

    def _graphable(self, entries):
        return self.use_graphs and all(len(e.tokens) == 1 and len(e.want) == 1 for e in entries)

    def _graph_key(self, entries, ctx):
        """Steps of single tokens with logits wanted for each are launch-bound: they replay a
        captured graph.  The key holds everything a captured launch depends on beyond the
        step's device metadata: the number of requests, the context bucket that sizes the
        split of the attention kernels, and how uneven the contexts are (which changes that split)."""
        if not self.use_graphs or not ctx.is_decode:
            return None
        if any(list(e.want) != [0] for e in entries):
            return None
        bucket = 256
        while bucket < ctx.max_context:
            bucket *= 2
        return (ctx.num_seqs, bucket, ctx.uneven)

    def _run_graphed(self, key, ctx):
        ctx.max_context = key[1]          # launches are planned for the bucket, not the exact length
        entry = self._graphs.get(key)
        if entry is None:                 # first sight: run eagerly (also warms lazy set-up)
            self._graphs[key] = "seen"
            self.graph_counts["first_sight"] += 1
            return self.model.forward(ctx, self.cache)
        if entry == "seen":
            from .. import ops
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            before = ops.launches()
            with torch.cuda.graph(graph, pool=self._graph_pool):
                logits = self.model.forward(ctx, self.cache)
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            entry = (graph, logits, ops.launches() - before, self._meta_dev.data_ptr())
            self._graphs[key] = entry
            self.graph_counts["captured"] += 1
        graph, logits, launches, meta_ptr = entry
        assert meta_ptr == self._meta_dev.data_ptr()
        graph.replay()
        self.graph_counts["replayed"] += 1
        from .. import ops
        ops.launch_count += launches
        return logits
