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
group; taking is all-or-nothing; giving back a page that is not owned raises.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

from ..errors import GlintError, PagePoolExhausted, SlotsExhausted


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
    """Free list of page ids 0..capacity-1 of one group (LIFO, so pages are reused soon)."""

    def __init__(self, name, capacity):
        self.name = name
        self.capacity = int(capacity)
        self._free = list(range(self.capacity - 1, -1, -1))
        self._owned = [False] * self.capacity
        self.peak_live = 0
        self.reuses = 0
        self.hidden = 0          # pages held for the engine's own use: not counted in the statistics
        self._ever_used = [False] * self.capacity

    @property
    def available(self):
        return len(self._free)

    @property
    def live(self):
        return self.capacity - len(self._free)

    def take(self, n):
        if n > len(self._free):
            raise PagePoolExhausted(self.name, n, len(self._free), self.capacity)
        pages = [self._free.pop() for _ in range(n)]
        for p in pages:
            assert not self._owned[p], f"page {p} of {self.name} handed out twice"
            self._owned[p] = True
            if self._ever_used[p]:
                self.reuses += 1
            self._ever_used[p] = True
        self.peak_live = max(self.peak_live, self.live)
        return pages

    def give(self, pages):
        for p in pages:
            if not (0 <= p < self.capacity) or not self._owned[p]:
                raise GlintError(f"page {p} of group '{self.name}' given back but not owned")
            self._owned[p] = False
            self._free.append(p)

    def stats(self):
        return {"capacity": self.capacity - self.hidden, "live": self.live - self.hidden,
                "peak_live": self.peak_live - self.hidden, "pooled": self.available, "reuses": self.reuses}


class PagedGroup:
    """One pool, its device storage for all member layers, and the block tables of all slots."""

    def __init__(self, need, members, num_pages, num_slots, page_size, max_positions, dtype, device):
        self.need = need
        self.name = need.group_name()
        self.members = list(members)          # run-order indices that own a layer of storage here
        self.page_size = page_size
        self.num_pages = num_pages
        self.max_pages = (max_positions + page_size - 1) // page_size
        self.pool = PagePool(self.name, num_pages)
        self.element_size = torch.empty((), dtype=dtype).element_size()
        self.storage = need.allocate(len(self.members), num_pages, page_size, dtype, device)
        self.table = np.full((num_slots, self.max_pages), -1, dtype=np.int32)
        self.first_live = np.zeros(num_slots, dtype=np.int64)   # first page index still held
        self.end_live = np.zeros(num_slots, dtype=np.int64)     # one past the last page held

    def bytes_per_token(self):
        return len(self.members) * self.need.bytes_per_token(self.element_size)

    # pages that queries at positions >= start can still reach begin at this page index
    def _first_needed_page(self, start):
        if self.need.window is None:
            return 0
        return max(0, start - self.need.window + 1) // self.page_size

    def release_behind(self, slot, start):
        """Give back pages that no query at position >= ``start`` can reach."""
        first = min(self._first_needed_page(start), int(self.end_live[slot]))
        lo = int(self.first_live[slot])
        if first > lo:
            pages = [int(p) for p in self.table[slot, lo:first] if p >= 0]
            self.pool.give(pages)
            self.table[slot, lo:first] = -1
            self.first_live[slot] = first
        return max(0, first - lo)

    def pages_needed(self, slot, start, n):
        """How many new pages the tokens [start, start+n) need beyond those already held."""
        end_page = (start + n + self.page_size - 1) // self.page_size
        begin = max(int(self.end_live[slot]), self._first_needed_page(start))
        return max(0, end_page - begin)

    def extend(self, slot, start, n):
        end_page = (start + n + self.page_size - 1) // self.page_size
        begin = max(int(self.end_live[slot]), self._first_needed_page(start))
        if end_page > self.max_pages:
            raise GlintError(f"positions up to {start + n} exceed the block table of {self.max_pages} pages")
        if end_page > begin:
            pages = self.pool.take(end_page - begin)
            self.table[slot, begin:end_page] = pages
            if int(self.end_live[slot]) == int(self.first_live[slot]):
                self.first_live[slot] = begin     # nothing was held: the held range starts here
            self.end_live[slot] = end_page

    def release_all(self, slot):
        lo, hi = int(self.first_live[slot]), int(self.end_live[slot])
        pages = [int(p) for p in self.table[slot, lo:hi] if p >= 0]
        self.pool.give(pages)
        self.table[slot, :] = -1
        self.first_live[slot] = 0
        self.end_live[slot] = 0

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
        placed = {}
        for need, members in by_key.values():
            g = PagedGroup(need, members, num_pages, num_slots, page_size, max_positions, dtype, device)
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
        self._free_slots = list(range(num_slots - 1, -1, -1))
        self._slot_live = [False] * num_slots
        self.lengths = np.zeros(num_slots, dtype=np.int64)

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
        return len(self._free_slots)

    def alloc_slot(self):
        if not self._free_slots:
            raise SlotsExhausted(f"all {self.num_slots} request slots are in use")
        slot = self._free_slots.pop()
        self._slot_live[slot] = True
        self.lengths[slot] = 0
        for st in list(self.states) + list(self.named_states.values()):
            if st is not None:
                st[slot].zero_()
        return slot

    def free_slot(self, slot):
        if not (0 <= slot < self.num_slots) or not self._slot_live[slot]:
            raise GlintError(f"slot {slot} freed but not in use")
        for g in self.groups:
            g.release_all(slot)
        self._slot_live[slot] = False
        self.lengths[slot] = 0
        self._free_slots.append(slot)

    def length(self, slot):
        return int(self.lengths[slot])

    # ---- pages ----------------------------------------------------------------------------------

    def pages_short(self, rows):
        """For ``rows`` = [(slot, n_new_tokens)], the first group that cannot serve them all as
        (group name, needed, available), or ``None``.  Counts pages a window frees first."""
        for g in self.groups:
            need = 0
            freed = 0
            for slot, n in rows:
                start = int(self.lengths[slot])
                first = min(g._first_needed_page(start), int(g.end_live[slot]))
                freed += max(0, first - int(g.first_live[slot]))
                need += g.pages_needed(slot, start, n)
            if need > g.pool.available + freed:
                return (g.name, need, g.pool.available + freed)
        return None

    def reserve(self, rows):
        """Make room for ``n`` more tokens of each (slot, n) in ``rows``; all or nothing.

        Pages behind a window are given back first (they are dead whatever happens next); then
        either every group serves every row, or ``PagePoolExhausted`` is raised and no page
        was taken.  Also raises when a row would pass the model's context length.
        """
        for slot, n in rows:
            if not self._slot_live[slot]:
                raise GlintError(f"slot {slot} is not in use")
            if int(self.lengths[slot]) + n > self.max_positions:
                raise GlintError(f"slot {slot}: {int(self.lengths[slot]) + n} positions exceed the "
                                 f"context length {self.max_positions}")
        for g in self.groups:
            for slot, n in rows:
                g.release_behind(slot, int(self.lengths[slot]))
        for g in self.groups:
            need = sum(g.pages_needed(slot, int(self.lengths[slot]), n) for slot, n in rows)
            if need > g.pool.available:
                raise PagePoolExhausted(g.name, need, g.pool.available, g.pool.capacity)
        for g in self.groups:
            for slot, n in rows:
                g.extend(slot, int(self.lengths[slot]), n)

    def advance(self, rows):
        """After the step ran: the slots now hold ``n`` more tokens each."""
        for slot, n in rows:
            self.lengths[slot] += n

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
                    if not self._slot_live[slot]:
                        raise AssertionError(f"page {p} of {g.name} held by free slot {slot}")
            free = set(g.pool._free)
            if len(free) != len(g.pool._free):
                raise AssertionError(f"{g.name}: a page is on the free list twice")
            if free & set(seen):
                raise AssertionError(f"{g.name}: pages both free and held: {sorted(free & set(seen))}")
            if len(free) + len(seen) != g.pool.capacity:
                raise AssertionError(f"{g.name}: {g.pool.capacity - len(free) - len(seen)} pages lost")
