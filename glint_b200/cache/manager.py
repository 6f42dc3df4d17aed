"""Cache manager: paged keys and values, block tables, and fixed-size per-request state.

The reference keeps 16-position pages of one layer each, per-layer page tables of equal
length, a capacity-bounded pool with a free list and ``live/peak/pooled`` statistics, an
all-or-nothing ``reserve`` before every forward pass, and gives pages back when the sequence
is dropped (src/cache/paged.rs:55-75, :100-242, :256-257, :316-324, :369-403).  Its layers
all keep every position; the sliding window only narrows reads
(src/transformer/forward.rs:574-582).

Here a page id is valid in every layer of its *group*: layers whose mixers declare the same
cache need (kv heads, head size, window) share one pool and one block table per request.  A
group with a window gives a page back as soon as no later query can reach it.  Beside the
pages, every run-order entry whose mixer declares a fixed-size state gets one row per request
slot.  The slot also carries the request's length; the sampler's generator state lives with
the request in the scheduler.

All bookkeeping is host-side and exact: a page is either free or owned by one slot of one
group; taking is all-or-nothing; giving back a page that is not owned raises.  The bookkeeping
itself (pools, block tables, slots, lengths) is C++ (``csrc/host/cache_core.cpp``); the classes
here own the device storage, turn the core's codes into exceptions, and show its tables as
numpy arrays.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import ctypes

import numpy as np
import torch

from ..errors import GlintError, PagePoolExhausted, SlotsExhausted
from . import core


class PagedNeed:
    """What a mixer that keeps something per token declares.  The cache manager asks only this of
    a declaration, so a mixer that caches something else than keys and values of one shape (one
    latent vector per token, keys and values of different widths) brings a class of its own:

    * ``paged`` is True; ``window`` is ``None`` (every position is kept) or the number of last
      positions a later token can still reach (pages behind it are given back);
    * ``group_key()``: hashable; layers with equal keys share one pool of pages and one block
      table per request;
    * ``allocate(layers, num_pages, page_size, dtype, device)``: the device storage of a group
      with that many member layers, in whatever form ``view`` understands;
    * ``view(storage, layer)``: what the mixer of member ``layer`` gets as its ``view`` (the
      manager adds ``group``, ``page_size``, ``num_pages`` and ``writes`` to it);
    * ``bytes_per_token(element_size)``: bytes one token takes in one layer;
    * ``readable_by(other)``: whether a layer declaring ``other`` may read this layer's cache.
    """
    paged = True
    window = None

    def group_key(self):
        raise NotImplementedError

    def group_name(self):
        return str(self.group_key())

    def allocate(self, layers, num_pages, page_size, dtype, device):
        raise NotImplementedError

    def view(self, storage, layer):
        raise NotImplementedError

    def bytes_per_token(self, element_size):
        raise NotImplementedError

    def readable_by(self, other):
        return self.group_key() == other.group_key()


class LayerView:
    """One member layer's part of a group's storage; the need's ``view`` fills in its tensors."""


@dataclass(frozen=True)
class PagedKVNeed(PagedNeed):
    """Keys and values of every position (``window`` None) or of the last ``window`` positions,
    ``num_kv_heads`` x ``head_dim`` each, as ``[layers][pages][kv heads][page][head_dim]``."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None

    def group_key(self):
        return (self.num_kv_heads, self.head_dim, self.window)

    def group_name(self):
        w = "all" if self.window is None else f"window{self.window}"
        return f"kv{self.num_kv_heads}x{self.head_dim}/{w}"

    def allocate(self, layers, num_pages, page_size, dtype, device):
        shape = (layers, num_pages, self.num_kv_heads, page_size, self.head_dim)
        return (torch.zeros(shape, dtype=dtype, device=device), torch.zeros(shape, dtype=dtype, device=device))

    def view(self, storage, layer):
        v = LayerView()
        v.k, v.v = storage[0][layer], storage[1][layer]
        return v

    def bytes_per_token(self, element_size):
        return 2 * self.num_kv_heads * self.head_dim * element_size

    def readable_by(self, other):
        return (getattr(other, "num_kv_heads", None), getattr(other, "head_dim", None)) == (self.num_kv_heads, self.head_dim)


@dataclass(frozen=True)
class SlotStateNeed:
    """A mixer's declaration of a state of fixed size: one tensor of ``shape`` and ``dtype`` per
    request, zero at admission.  ``allocate(num_slots, device)`` makes the rows of all slots."""
    shape: tuple
    dtype: torch.dtype = torch.float32
    paged = False

    def allocate(self, num_slots, device):
        return torch.zeros((num_slots,) + tuple(self.shape), dtype=self.dtype, device=device)


def is_paged(need):
    return need is not None and bool(getattr(need, "paged", False))


def cache_bytes_per_token(needs, cache_of, element_size):
    """Bytes one token takes in all layers that keep pages of their own."""
    return sum(n.bytes_per_token(element_size) for n, of in zip(needs, cache_of) if is_paged(n) and of is None)


class PagePool:
    """Free list of page ids 0..capacity-1 of one group (last in, first out, so pages are reused soon).
    The list itself is kept by the C++ core; this class is its face."""

    def __init__(self, name, capacity, handle=None):
        self.name = name
        self.capacity = int(capacity)
        self._lib = core.lib()
        self._own = handle is None
        self._h = self._lib.glint_pool_create(self.capacity) if handle is None else handle
        self.hidden = 0          # pages held for the engine's own use: not counted in the statistics

    def __del__(self):
        try:
            if self._own and self._h:
                self._lib.glint_pool_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def _stats(self):
        out = (ctypes.c_longlong * 5)()
        self._lib.glint_pool_stats(self._h, out)
        return list(out)

    @property
    def available(self):
        return self._stats()[3]

    @property
    def live(self):
        return self._stats()[1]

    @property
    def peak_live(self):
        return self._stats()[2]

    @property
    def reuses(self):
        return self._stats()[4]

    @property
    def _free(self):
        out = (ctypes.c_int * max(self.capacity, 1))()
        n = self._lib.glint_pool_free_list(self._h, out, self.capacity)
        return list(out[:n])

    def take(self, n):
        out = (ctypes.c_int * max(n, 1))()
        rc = self._lib.glint_pool_take(self._h, n, out)
        if rc == core.EXHAUSTED:
            raise PagePoolExhausted(self.name, n, self.available, self.capacity)
        if rc != core.OK:
            raise GlintError(f"page pool '{self.name}': bad request for {n} pages")
        return list(out[:n])

    def give(self, pages):
        arr, n = core.int_array([int(p) for p in pages])
        bad = ctypes.c_int(-1)
        if self._lib.glint_pool_give(self._h, arr, n, ctypes.byref(bad)) != core.OK:
            raise GlintError(f"page {bad.value} of group '{self.name}' given back but not owned")

    def stats(self):
        _, live, peak, free, reuses = self._stats()
        return {"capacity": self.capacity - self.hidden, "live": live - self.hidden,
                "peak_live": peak - self.hidden, "pooled": free, "reuses": reuses}


class PagedGroup:
    """One pool, its device storage for all member layers, and the block tables of all slots.  Pool and
    tables live in the C++ core (``index`` is the group's place there); ``table``, ``first_live`` and
    ``end_live`` are views of its memory."""

    def __init__(self, need, members, handle, index, num_pages, num_slots, page_size, max_positions, dtype, device):
        lib = core.lib()
        self.need = need
        self.name = need.group_name()
        self.members = list(members)          # run-order indices that own a layer of storage here
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_pages = (max_positions + page_size - 1) // page_size
        self.pool = PagePool(self.name, num_pages, handle=lib.glint_cache_pool(handle, index))
        self.element_size = torch.empty((), dtype=dtype).element_size()
        self.storage = need.allocate(len(self.members), num_pages, page_size, dtype, device)
        self.table = core.as_array(lib.glint_cache_table(handle, index), (num_slots, self.max_pages))
        self.first_live = core.as_array(lib.glint_cache_first_live(handle, index), (num_slots,))   # first page index still held
        self.end_live = core.as_array(lib.glint_cache_end_live(handle, index), (num_slots,))       # one past the last page held

    def bytes_per_token(self):
        return len(self.members) * self.need.bytes_per_token(self.element_size)

    def owned_pages(self, slot):
        return [int(p) for p in self.table[slot] if p >= 0]


def CacheView(group, layer_in_group, writes):
    """What one run-order entry's mixer sees of a paged group: its own layer of the storage, as the
    group's declaration lays it out, with the group, the page geometry and whether it writes."""
    view = group.need.view(group.storage, layer_in_group)
    view.group = group
    view.layer_in_group = layer_in_group
    view.page_size = group.page_size
    view.num_pages = group.num_pages
    view.writes = writes           # False when the entry reads another entry's cache
    return view


class CacheManager:
    """Owns every group, the request slots and the per-request state tensors.

    ``needs[i]`` is the declaration of run-order entry ``i`` (``PagedKVNeed``, ``SlotStateNeed``
    or ``None``); ``cache_of[i]`` names the earlier entry whose cache entry ``i`` reads, if any.
    ``num_pages`` is the capacity of every group's pool.
    """

    def __init__(self, needs, cache_of, num_slots, num_pages, page_size, max_positions, dtype, device):
        if page_size <= 0 or num_pages <= 0 or num_slots <= 0:
            raise GlintError("page size, page count and slot count must be positive")
        self.num_slots = num_slots
        self.page_size = page_size
        self.max_positions = max_positions
        self.device = device
        self.dtype = dtype
        self.groups = []
        self.views = [None] * len(needs)
        self.states = [None] * len(needs)
        by_key = {}
        for i, need in enumerate(needs):
            if is_paged(need) and cache_of[i] is None:
                by_key.setdefault(need.group_key(), (need, []))[1].append(i)
        # pools, block tables, slots and lengths are kept by the C++ core, one group per distinct need
        self._lib = core.lib()
        windows, n_groups = core.int_array([-1 if need.window is None else int(need.window) for need, _ in by_key.values()])
        self._h = self._lib.glint_cache_create(n_groups, windows, num_slots, num_pages, page_size, max_positions)
        if not self._h:
            raise GlintError("the cache core refused these sizes")
        placed = {}
        for index, (need, members) in enumerate(by_key.values()):
            g = PagedGroup(need, members, self._h, index, num_pages, num_slots, page_size, max_positions, dtype, device)
            self.groups.append(g)
            for j, i in enumerate(members):
                placed[i] = (g, j)
                self.views[i] = CacheView(g, j, writes=True)
        for i, need in enumerate(needs):
            if is_paged(need) and cache_of[i] is not None:
                src = cache_of[i]
                if src not in placed:
                    raise GlintError(f"run-order entry {i} reads the cache of entry {src}, which owns none")
                g, j = placed[src]
                if not g.need.readable_by(need):
                    raise GlintError(f"run-order entry {i} cannot read the cache of entry {src}: shapes differ")
                self.views[i] = CacheView(g, j, writes=False)
            elif need is not None and not is_paged(need):
                self.states[i] = need.allocate(num_slots, device)
        self.named_states = {}
        self.lengths = core.as_array(self._lib.glint_cache_lengths(self._h), (num_slots,))

    def __del__(self):
        try:
            if self._h:
                self.groups.clear()                     # their views point into the core's memory
                self._lib.glint_cache_destroy(self._h)
                self._h = None
        except Exception:
            pass

    def add_state(self, name, need):
        """A fixed-size record per request slot for something beside the mixers (the sampler keeps the
        request's options, generator state, position and count there): ``need`` is a ``SlotStateNeed``;
        the rows are zero now and again whenever a request takes its slot.  Returns the tensor [slots, *shape]."""
        if name in self.named_states:
            return self.named_states[name]
        st = self.named_states[name] = need.allocate(self.num_slots, self.device)
        return st

    # ---- slots ----------------------------------------------------------------------------------

    @property
    def free_slots(self):
        return self._lib.glint_cache_free_slots(self._h)

    def slot_live(self, slot):
        return bool(self._lib.glint_cache_slot_live(self._h, int(slot)))

    def alloc_slot(self):
        slot = ctypes.c_int(-1)
        if self._lib.glint_cache_alloc_slot(self._h, ctypes.byref(slot)) != core.OK:
            raise SlotsExhausted(f"all {self.num_slots} request slots are in use")
        for st in list(self.states) + list(self.named_states.values()):
            if st is not None:
                st[slot.value].zero_()
        return slot.value

    def free_slot(self, slot):
        bad = ctypes.c_int(-1)
        rc = self._lib.glint_cache_free_slot(self._h, int(slot), ctypes.byref(bad))
        if rc == core.SLOT_NOT_LIVE:
            raise GlintError(f"slot {slot} freed but not in use")
        if rc != core.OK:
            raise GlintError(f"page {bad.value} of slot {slot} given back but not owned")

    def length(self, slot):
        return int(self.lengths[slot])

    # ---- pages ----------------------------------------------------------------------------------

    @staticmethod
    def _rows(rows):
        slots, n = core.int_array([int(s) for s, _ in rows])
        counts, _ = core.int_array([int(k) for _, k in rows])
        return slots, counts, n

    def pages_short(self, rows):
        """For ``rows`` = [(slot, n_new_tokens)], the first group that cannot serve them all as
        (group name, needed, available), or ``None``.  Counts pages a window frees first."""
        slots, counts, n = self._rows(rows)
        group, need, have = ctypes.c_int(0), ctypes.c_longlong(0), ctypes.c_longlong(0)
        if self._lib.glint_cache_pages_short(self._h, slots, counts, n, ctypes.byref(group), ctypes.byref(need),
                                             ctypes.byref(have)):
            return (self.groups[group.value].name, need.value, have.value)
        return None

    def plan(self, budget, max_active, running, waiting):
        """One step's plan for a continuous-batching scheduler, decided by the C++ core: ``running`` holds
        (slot, tokens still to compute, is it decoding) per running request in admission order, ``waiting``
        the tokens to compute per queued request in queue order.  Decoding requests first with one token each,
        then running prompts with what the budget leaves, then admissions while slots are free; a row joins
        only if the cache can serve it together with the rows before it.  Returns (tokens per running request,
        tokens per admitted request); takes no page and no slot."""
        slots, n_run = core.int_array([int(r[0]) for r in running])
        remaining, _ = core.int_array([int(r[1]) for r in running])
        decoding, _ = core.int_array([1 if r[2] else 0 for r in running])
        wait, n_wait = core.int_array([int(w) for w in waiting])
        out_run = (ctypes.c_int * max(n_run, 1))()
        out_wait = (ctypes.c_int * max(n_wait, 1))()
        admitted = self._lib.glint_cache_plan(self._h, int(budget), int(max_active), n_run, slots, remaining, decoding,
                                              n_wait, wait, out_run, out_wait)
        return list(out_run[:n_run]), list(out_wait[:admitted])

    def reserve(self, rows):
        """Make room for ``n`` more tokens of each (slot, n) in ``rows``; all or nothing.

        Pages behind a window are given back first (they are dead whatever happens next); then
        either every group serves every row, or ``PagePoolExhausted`` is raised and no page
        was taken.  Also raises when a row would pass the model's context length.
        """
        slots, counts, n = self._rows(rows)
        slot, group, need, have = ctypes.c_int(-1), ctypes.c_int(0), ctypes.c_longlong(0), ctypes.c_longlong(0)
        rc = self._lib.glint_cache_reserve(self._h, slots, counts, n, ctypes.byref(slot), ctypes.byref(group),
                                           ctypes.byref(need), ctypes.byref(have))
        if rc == core.OK:
            return
        if rc == core.EXHAUSTED:
            g = self.groups[group.value]
            raise PagePoolExhausted(g.name, need.value, have.value, g.pool.capacity)
        if rc == core.SLOT_NOT_LIVE:
            raise GlintError(f"slot {slot.value} is not in use")
        if rc == core.CONTEXT:
            asked = dict((int(s), int(k)) for s, k in rows)[slot.value]
            raise GlintError(f"slot {slot.value}: {self.length(slot.value) + asked} positions exceed the "
                             f"context length {self.max_positions}")
        if rc == core.TABLE_FULL:
            raise GlintError(f"slot {slot.value}: positions exceed the block table of {self.groups[0].max_pages} pages")
        raise GlintError(f"the cache core failed with code {rc}")

    def advance(self, rows):
        """After the step ran: the slots now hold ``n`` more tokens each."""
        slots, counts, n = self._rows(rows)
        self._lib.glint_cache_advance(self._h, slots, counts, n)

    def block_tables(self, slots):
        """Per group, the block-table rows of ``slots`` as one int32 array [len(slots), max_pages]."""
        idx = np.asarray(slots, dtype=np.int64)
        return [g.table[idx] for g in self.groups]

    def group_index(self, group):
        return self.groups.index(group)

    def stats(self):
        return {g.name: g.pool.stats() for g in self.groups}

    def bytes_per_token(self):
        return sum(g.bytes_per_token() for g in self.groups)

    def check_consistency(self):
        """Every page is free or owned by exactly one slot of its group (used by tests)."""
        for g in self.groups:
            seen = {}
            for slot in range(self.num_slots):
                for p in g.owned_pages(slot):
                    if p in seen:
                        raise AssertionError(f"page {p} of {g.name} held by slots {seen[p]} and {slot}")
                    seen[p] = slot
                    if not self.slot_live(slot):
                        raise AssertionError(f"page {p} of {g.name} held by free slot {slot}")
            free = set(g.pool._free)
            if len(free) != len(g.pool._free):
                raise AssertionError(f"{g.name}: a page is on the free list twice")
            if free & set(seen):
                raise AssertionError(f"{g.name}: pages both free and held: {sorted(free & set(seen))}")
            if len(free) + len(seen) != g.pool.capacity:
                raise AssertionError(f"{g.name}: {g.pool.capacity - len(free) - len(seen)} pages lost")
