#include "cache_core.h"

#include <algorithm>
#include <vector>

struct GlintPool {
  int capacity = 0;
  std::vector<int> free_list;       // the back is taken next
  std::vector<char> owned, ever_used;
  long long peak_live = 0, reuses = 0;
  int live() const { return capacity - (int)free_list.size(); }
};

extern "C" GlintPool* glint_pool_create(int capacity) {
  if (capacity < 0) return nullptr;
  GlintPool* p = new GlintPool();
  p->capacity = capacity;
  p->free_list.resize(capacity);
  for (int i = 0; i < capacity; ++i) p->free_list[i] = capacity - 1 - i;      // page 0 is taken first
  p->owned.assign(capacity, 0);
  p->ever_used.assign(capacity, 0);
  return p;
}

extern "C" void glint_pool_destroy(GlintPool* p) { delete p; }

extern "C" int glint_pool_take(GlintPool* p, int n, int* out) {
  if (n < 0) return GLINT_CACHE_BAD_ARG;
  if (n > (int)p->free_list.size()) return GLINT_CACHE_EXHAUSTED;
  for (int i = 0; i < n; ++i) {
    const int page = p->free_list.back();
    p->free_list.pop_back();
    p->owned[page] = 1;
    if (p->ever_used[page]) ++p->reuses;
    p->ever_used[page] = 1;
    out[i] = page;
  }
  p->peak_live = std::max<long long>(p->peak_live, p->live());
  return GLINT_CACHE_OK;
}

extern "C" int glint_pool_give(GlintPool* p, const int* pages, int n, int* bad) {
  for (int i = 0; i < n; ++i) {
    const int page = pages[i];
    if (page < 0 || page >= p->capacity || !p->owned[page]) {
      if (bad) *bad = page;
      return GLINT_CACHE_NOT_OWNED;
    }
    p->owned[page] = 0;
    p->free_list.push_back(page);
  }
  return GLINT_CACHE_OK;
}

extern "C" void glint_pool_stats(const GlintPool* p, long long out[5]) {
  out[0] = p->capacity;
  out[1] = p->live();
  out[2] = p->peak_live;
  out[3] = (long long)p->free_list.size();
  out[4] = p->reuses;
}

extern "C" int glint_pool_free_list(const GlintPool* p, int* out, int cap) {
  const int n = (int)p->free_list.size();
  for (int i = 0; i < n && i < cap; ++i) out[i] = p->free_list[i];
  return n;
}

// ---------------------------------------------------------------------------------------------------------

struct Group {
  long long window = -1;            // < 0: every position is kept
  GlintPool* pool = nullptr;
  std::vector<int32_t> table;       // [num_slots][max_pages]
  std::vector<int64_t> first_live, end_live;
};

struct GlintCache {
  int num_slots = 0, num_pages = 0, page_size = 0, max_positions = 0, max_pages = 0;
  std::vector<Group> groups;
  std::vector<int64_t> lengths;
  std::vector<char> slot_live;
  std::vector<int> free_slots;      // the back is taken next

  // pages that queries at positions >= start can still reach begin at this page index
  long long first_needed_page(const Group& g, long long start) const {
    if (g.window < 0) return 0;
    return std::max<long long>(0, start - g.window + 1) / page_size;
  }
  // new pages the tokens [start, start + n) need beyond those already held
  long long pages_needed(const Group& g, int slot, long long start, long long n) const {
    const long long end_page = (start + n + page_size - 1) / page_size;
    const long long begin = std::max<long long>(g.end_live[slot], first_needed_page(g, start));
    return std::max<long long>(0, end_page - begin);
  }
  // pages a release behind `start` would give back
  long long freed_behind(const Group& g, int slot, long long start) const {
    const long long first = std::min<long long>(first_needed_page(g, start), g.end_live[slot]);
    return std::max<long long>(0, first - g.first_live[slot]);
  }
};

extern "C" GlintCache* glint_cache_create(int num_groups, const int* windows, int num_slots, int num_pages,
                                          int page_size, int max_positions) {
  if (num_groups < 0 || num_slots <= 0 || num_pages <= 0 || page_size <= 0 || max_positions <= 0) return nullptr;
  GlintCache* c = new GlintCache();
  c->num_slots = num_slots; c->num_pages = num_pages; c->page_size = page_size; c->max_positions = max_positions;
  c->max_pages = (max_positions + page_size - 1) / page_size;
  c->groups.resize(num_groups);
  for (int g = 0; g < num_groups; ++g) {
    Group& grp = c->groups[g];
    grp.window = windows[g];
    grp.pool = glint_pool_create(num_pages);
    grp.table.assign((size_t)num_slots * c->max_pages, -1);
    grp.first_live.assign(num_slots, 0);
    grp.end_live.assign(num_slots, 0);
  }
  c->lengths.assign(num_slots, 0);
  c->slot_live.assign(num_slots, 0);
  for (int s = num_slots - 1; s >= 0; --s) c->free_slots.push_back(s);        // slot 0 is taken first
  return c;
}

extern "C" void glint_cache_destroy(GlintCache* c) {
  if (!c) return;
  for (Group& g : c->groups) glint_pool_destroy(g.pool);
  delete c;
}

extern "C" GlintPool* glint_cache_pool(GlintCache* c, int group) { return c->groups[group].pool; }
extern "C" int32_t* glint_cache_table(GlintCache* c, int group) { return c->groups[group].table.data(); }
extern "C" int64_t* glint_cache_first_live(GlintCache* c, int group) { return c->groups[group].first_live.data(); }
extern "C" int64_t* glint_cache_end_live(GlintCache* c, int group) { return c->groups[group].end_live.data(); }
extern "C" int64_t* glint_cache_lengths(GlintCache* c) { return c->lengths.data(); }
extern "C" int glint_cache_max_pages(const GlintCache* c) { return c->max_pages; }
extern "C" int glint_cache_free_slots(const GlintCache* c) { return (int)c->free_slots.size(); }
extern "C" int glint_cache_slot_live(const GlintCache* c, int slot) {
  return slot >= 0 && slot < c->num_slots && c->slot_live[slot];
}

extern "C" int glint_cache_alloc_slot(GlintCache* c, int* slot) {
  if (c->free_slots.empty()) return GLINT_CACHE_NO_SLOT;
  *slot = c->free_slots.back();
  c->free_slots.pop_back();
  c->slot_live[*slot] = 1;
  c->lengths[*slot] = 0;
  return GLINT_CACHE_OK;
}

static int release_range(GlintCache* c, Group& g, int slot, long long lo, long long hi, int* bad) {
  int32_t* row = g.table.data() + (size_t)slot * c->max_pages;
  for (long long i = lo; i < hi; ++i) {
    if (row[i] >= 0) {
      const int page = row[i];
      const int rc = glint_pool_give(g.pool, &page, 1, bad);
      if (rc != GLINT_CACHE_OK) return rc;
    }
    row[i] = -1;
  }
  return GLINT_CACHE_OK;
}

extern "C" int glint_cache_free_slot(GlintCache* c, int slot, int* bad_page) {
  if (!glint_cache_slot_live(c, slot)) return GLINT_CACHE_SLOT_NOT_LIVE;
  for (Group& g : c->groups) {
    const int rc = release_range(c, g, slot, g.first_live[slot], g.end_live[slot], bad_page);
    if (rc != GLINT_CACHE_OK) return rc;
    g.first_live[slot] = 0;
    g.end_live[slot] = 0;
  }
  c->slot_live[slot] = 0;
  c->lengths[slot] = 0;
  c->free_slots.push_back(slot);
  return GLINT_CACHE_OK;
}

extern "C" int glint_cache_release_behind(GlintCache* c, int group, int slot, long long start) {
  Group& g = c->groups[group];
  const long long first = std::min<long long>(c->first_needed_page(g, start), g.end_live[slot]);
  const long long lo = g.first_live[slot];
  if (first > lo) {
    int bad = -1;
    if (release_range(c, g, slot, lo, first, &bad) != GLINT_CACHE_OK) return -1;
    g.first_live[slot] = first;
    return (int)(first - lo);
  }
  return 0;
}

// Rows of live slots, and `fresh` rows of requests that would start in a slot of their own (nothing cached,
// nothing held): the first group that cannot serve them all, or none.
static int short_for(const GlintCache* c, const int* slots, const int* counts, int n, const int* fresh, int n_fresh,
                     int* group, long long* need, long long* available) {
  for (int gi = 0; gi < (int)c->groups.size(); ++gi) {
    const Group& g = c->groups[gi];
    long long want = 0, freed = 0;
    for (int i = 0; i < n; ++i) {
      const long long start = c->lengths[slots[i]];
      freed += c->freed_behind(g, slots[i], start);
      want += c->pages_needed(g, slots[i], start, counts[i]);
    }
    for (int i = 0; i < n_fresh; ++i) want += ((long long)fresh[i] + c->page_size - 1) / c->page_size;
    const long long have = (long long)g.pool->free_list.size() + freed;
    if (want > have) {
      if (group) *group = gi;
      if (need) *need = want;
      if (available) *available = have;
      return 1;
    }
  }
  return 0;
}

extern "C" int glint_cache_pages_short(const GlintCache* c, const int* slots, const int* counts, int n, int* group,
                                       long long* need, long long* available) {
  return short_for(c, slots, counts, n, nullptr, 0, group, need, available);
}

// One step's plan (the reference's engine loop admits first-come while fewer than max_active run and
// decodes one token per live sequence per step, src/server/engine.rs:489-511, :650-669; the token budget and
// the portions are this engine's).  Running requests come in admission order with their slot, the tokens
// they still have to compute, and whether they are decoding (one token behind their newest); waiting ones
// in queue order with their tokens.  Decoding requests go first with one token each, then running prompts
// with as much as the budget leaves, then new admissions while a slot is free; a row joins only if the cache
// can serve it together with the rows before it.  out_running[i] and out_waiting[i] get the tokens of that
// request in this step (0: not in it); admissions stop at the first waiting request that does not fit.
// Returns the number of admissions.  Takes no page and no slot.
extern "C" int glint_cache_plan(const GlintCache* c, int budget, int max_active, int n_running, const int* slots,
                                const int* remaining, const int* decoding, int n_waiting, const int* waiting,
                                int* out_running, int* out_waiting) {
  std::vector<int> row_slots, row_counts, fresh;
  row_slots.reserve(n_running);
  row_counts.reserve(n_running);
  for (int i = 0; i < n_running; ++i) out_running[i] = 0;
  for (int i = 0; i < n_waiting; ++i) out_waiting[i] = 0;
  auto fits = [&](int slot, int n) {
    row_slots.push_back(slot);
    row_counts.push_back(n);
    const bool ok = !short_for(c, row_slots.data(), row_counts.data(), (int)row_slots.size(), nullptr, 0, nullptr,
                               nullptr, nullptr);
    if (!ok) {
      row_slots.pop_back();
      row_counts.pop_back();
    }
    return ok;
  };
  // the usual case: every decoding request fits, one check
  int n_decoding = 0;
  for (int i = 0; i < n_running; ++i)
    if (decoding[i]) {
      row_slots.push_back(slots[i]);
      row_counts.push_back(1);
      ++n_decoding;
    }
  if (n_decoding > 0 && n_decoding <= budget &&
      !short_for(c, row_slots.data(), row_counts.data(), n_decoding, nullptr, 0, nullptr, nullptr, nullptr)) {
    for (int i = 0; i < n_running; ++i)
      if (decoding[i]) out_running[i] = 1;
    budget -= n_decoding;
  } else {
    row_slots.clear();
    row_counts.clear();
    for (int i = 0; i < n_running; ++i)
      if (decoding[i] && budget >= 1 && fits(slots[i], 1)) {
        out_running[i] = 1;
        --budget;
      }
  }
  for (int i = 0; i < n_running; ++i) {
    if (decoding[i]) continue;
    const int n = std::min(remaining[i], budget);
    if (n > 0 && fits(slots[i], n)) {        // a portion that does not fit waits for pages
      out_running[i] = n;
      budget -= n;
    }
  }
  int admitted = 0;
  int free_slots = (int)c->free_slots.size();
  while (admitted < n_waiting && budget > 0 && n_running + admitted < max_active && free_slots > 0) {
    const int n = std::min(waiting[admitted], budget);
    fresh.push_back(n);
    if (short_for(c, row_slots.data(), row_counts.data(), (int)row_slots.size(), fresh.data(), (int)fresh.size(),
                  nullptr, nullptr, nullptr)) {
      fresh.pop_back();
      break;
    }
    out_waiting[admitted] = n;
    budget -= n;
    --free_slots;
    ++admitted;
  }
  return admitted;
}

extern "C" int glint_cache_reserve(GlintCache* c, const int* slots, const int* counts, int n, int* info_slot,
                                   int* group, long long* need, long long* available) {
  for (int i = 0; i < n; ++i) {
    if (!glint_cache_slot_live(c, slots[i])) { *info_slot = slots[i]; return GLINT_CACHE_SLOT_NOT_LIVE; }
    if (c->lengths[slots[i]] + counts[i] > c->max_positions) { *info_slot = slots[i]; return GLINT_CACHE_CONTEXT; }
  }
  // pages behind a window are dead whatever happens next: they go back first
  for (int gi = 0; gi < (int)c->groups.size(); ++gi)
    for (int i = 0; i < n; ++i)
      if (glint_cache_release_behind(c, gi, slots[i], c->lengths[slots[i]]) < 0) return GLINT_CACHE_NOT_OWNED;
  for (int gi = 0; gi < (int)c->groups.size(); ++gi) {
    const Group& g = c->groups[gi];
    long long want = 0;
    for (int i = 0; i < n; ++i) want += c->pages_needed(g, slots[i], c->lengths[slots[i]], counts[i]);
    if (want > (long long)g.pool->free_list.size()) {
      *group = gi; *need = want; *available = (long long)g.pool->free_list.size();
      return GLINT_CACHE_EXHAUSTED;
    }
  }
  for (Group& g : c->groups) {
    for (int i = 0; i < n; ++i) {
      const int slot = slots[i];
      const long long start = c->lengths[slot];
      const long long end_page = (start + counts[i] + c->page_size - 1) / c->page_size;
      const long long begin = std::max<long long>(g.end_live[slot], c->first_needed_page(g, start));
      if (end_page > c->max_pages) { *info_slot = slot; return GLINT_CACHE_TABLE_FULL; }
      if (end_page > begin) {
        int32_t* row = g.table.data() + (size_t)slot * c->max_pages;
        const int rc = glint_pool_take(g.pool, (int)(end_page - begin), row + begin);
        if (rc != GLINT_CACHE_OK) return rc;          // cannot happen: the groups were checked above
        if (g.end_live[slot] == g.first_live[slot]) g.first_live[slot] = begin;     // nothing was held: the held range starts here
        g.end_live[slot] = end_page;
      }
    }
  }
  return GLINT_CACHE_OK;
}

extern "C" void glint_cache_advance(GlintCache* c, const int* slots, const int* counts, int n) {
  for (int i = 0; i < n; ++i) c->lengths[slots[i]] += counts[i];
}
