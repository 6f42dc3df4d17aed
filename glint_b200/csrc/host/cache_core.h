// Bookkeeping of the paged cache on the host: page pools, block tables, request slots.
//
// The reference keeps 16-position pages in a capacity-bounded pool with a free list and
// live/peak/pooled statistics, per-sequence page tables, and an all-or-nothing reserve before
// every forward pass (src/cache/paged.rs:55-75, :100-242, :369-403).  Here a pool belongs to a
// group of layers with the same cache need; a group with a window gives a page back as soon as no
// later query can reach it; a request slot carries its length.  Device memory is not touched here:
// the Python side owns the storage and uploads the block tables.
#pragma once
#include <stdint.h>

extern "C" {

enum {
  GLINT_CACHE_OK = 0,
  GLINT_CACHE_EXHAUSTED = 1,       // a pool cannot serve the request; nothing was taken
  GLINT_CACHE_CONTEXT = 2,         // a slot would pass the context length
  GLINT_CACHE_SLOT_NOT_LIVE = 3,
  GLINT_CACHE_NOT_OWNED = 4,       // a page was given back that its giver does not own
  GLINT_CACHE_NO_SLOT = 5,
  GLINT_CACHE_TABLE_FULL = 6,      // positions beyond the block table
  GLINT_CACHE_BAD_ARG = 7
};

// ---- one pool of pages (ids 0 .. capacity - 1; last in, first out, so pages are reused soon) -------------
struct GlintPool;
GlintPool* glint_pool_create(int capacity);
void glint_pool_destroy(GlintPool* p);
// Takes n pages into out, all or nothing: GLINT_CACHE_EXHAUSTED leaves the pool as it was.
int glint_pool_take(GlintPool* p, int n, int* out);
// Gives pages back; a page that is not owned stops the call with GLINT_CACHE_NOT_OWNED and its id in *bad.
int glint_pool_give(GlintPool* p, const int* pages, int n, int* bad);
// capacity, live, peak live, available, reuses
void glint_pool_stats(const GlintPool* p, long long out[5]);
int glint_pool_free_list(const GlintPool* p, int* out, int cap);

// ---- all groups, their block tables, and the request slots ---------------------------------------------
struct GlintCache;
// windows[g] < 0: the group keeps every position
GlintCache* glint_cache_create(int num_groups, const int* windows, int num_slots, int num_pages, int page_size,
                               int max_positions);
void glint_cache_destroy(GlintCache* c);
GlintPool* glint_cache_pool(GlintCache* c, int group);
int32_t* glint_cache_table(GlintCache* c, int group);         // [num_slots][max_pages], -1 where no page is held
int64_t* glint_cache_first_live(GlintCache* c, int group);    // [num_slots] first page index still held
int64_t* glint_cache_end_live(GlintCache* c, int group);      // [num_slots] one past the last page held
int64_t* glint_cache_lengths(GlintCache* c);                  // [num_slots] tokens cached
int glint_cache_max_pages(const GlintCache* c);
int glint_cache_free_slots(const GlintCache* c);
int glint_cache_alloc_slot(GlintCache* c, int* slot);
int glint_cache_free_slot(GlintCache* c, int slot, int* bad_page);
int glint_cache_slot_live(const GlintCache* c, int slot);
// Could the rows (slot, new tokens) all be served?  0: yes; 1: no, with the first group that cannot and what it
// needs and has (pages that a window frees first are counted as available).
int glint_cache_pages_short(const GlintCache* c, const int* slots, const int* counts, int n, int* group,
                            long long* need, long long* available);
// One step's plan for a continuous-batching scheduler: which running requests run how many tokens and how many
// waiting requests are admitted with how many tokens (see cache_core.cpp); takes no page and no slot.
int glint_cache_plan(const GlintCache* c, int budget, int max_active, int n_running, const int* slots,
                     const int* remaining, const int* decoding, int n_waiting, const int* waiting, int* out_running,
                     int* out_waiting);
// Room for counts[i] more tokens of slots[i]; all or nothing.  Pages behind a window are given back first.
int glint_cache_reserve(GlintCache* c, const int* slots, const int* counts, int n, int* info_slot, int* group,
                        long long* need, long long* available);
void glint_cache_advance(GlintCache* c, const int* slots, const int* counts, int n);
// Gives back the pages of `slot` in `group` that no query at position >= start can reach; returns how many.
int glint_cache_release_behind(GlintCache* c, int group, int slot, long long start);

}  // extern "C"
