// Host-side bookkeeping of the paged cache, in C++ behind a C interface (loaded with ctypes by
// cache/native.py): page pools (a LIFO free list with reference counts) and, per group of layers, a
// block table per request slot. Nothing here touches a device; the Python cache manager owns the
// device tensors and the mapping from request ids to slots. The reference's counterparts are
// `BlockPool` and the scheduler's block tables (crates/specrt/src/sched.rs:18-96, 1106-1130).
//
// A group with a window gives a page back as soon as every position in it has fallen out of the
// window of the request's next token. All calls are meant for one thread.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

thread_local std::string g_error;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_error = buf;
  return code;
}

struct Pool {
  int num_pages;
  std::vector<int> free_list;   // back() is handed out next
  std::vector<int> refs;
  explicit Pool(int n) : num_pages(n), refs(n, 0) {
    free_list.reserve(n);
    for (int p = n - 1; p >= 0; p--) free_list.push_back(p);   // page 0 first
  }
  int allocate() {
    if (free_list.empty()) return -1;
    const int p = free_list.back();
    free_list.pop_back();
    refs[p] = 1;
    return p;
  }
  int held(int page, const char* verb) const {
    if (page < 0 || page >= num_pages) return fail(1, "page %d is outside the pool of %d pages", page, num_pages);
    if (refs[page] <= 0) return fail(2, "page %d is %s but nobody holds it", page, verb);
    return 0;
  }
  int share(int page) {
    if (int e = held(page, "shared")) return e;
    refs[page]++;
    return 0;
  }
  int release(int page) {
    if (int e = held(page, "freed")) return e;
    if (--refs[page] == 0) free_list.push_back(page);
    return 0;
  }
  int check() const {
    std::vector<char> on_list(num_pages, 0);
    for (int p : free_list) {
      if (p < 0 || p >= num_pages) return fail(1, "the free list holds page %d, outside the pool", p);
      if (on_list[p]) return fail(1, "page %d is on the free list twice", p);
      on_list[p] = 1;
    }
    for (int p = 0; p < num_pages; p++)
      if ((on_list[p] != 0) == (refs[p] > 0))
        return fail(1, "page %d has reference count %d but is %s the free list", p, refs[p], on_list[p] ? "on" : "not on");
    return 0;
  }
};

struct Cache {
  int page_size, max_requests, max_tokens, table_width;
  std::vector<int> windows;            // per group, 0 = none
  std::vector<Pool> pools;             // per group
  std::vector<int> tables;             // [groups][max_requests][table_width], -1 = no page
  std::vector<int> length;             // per slot: positions whose state is in the cache
  std::vector<char> live;              // per slot
  std::vector<int> free_slots;         // back() is handed out next

  int* row(int g, int slot) { return tables.data() + ((size_t)g * max_requests + slot) * table_width; }
  int first_live_page(int g, int len) const {   // pages below hold only positions that no token at position >= len can see
    if (windows[g] <= 0) return 0;
    const int lo = len - windows[g] + 1;
    return lo > 0 ? lo / page_size : 0;
  }
  int pages_for(int len) const { return (len + page_size - 1) / page_size; }
  bool is_live(int slot) const { return slot >= 0 && slot < max_requests && live[slot]; }
};

}  // namespace

extern "C" {

const char* ibh_last_error() { return g_error.c_str(); }

// ---------------------------------------------------------------- a pool alone
void* ibh_pool_new(int num_pages) { return num_pages > 0 ? new Pool(num_pages) : nullptr; }
void ibh_pool_free(void* p) { delete (Pool*)p; }
int ibh_pool_num_pages(void* p) { return ((Pool*)p)->num_pages; }
int ibh_pool_free_pages(void* p) { return (int)((Pool*)p)->free_list.size(); }
int ibh_pool_allocate(void* p) { return ((Pool*)p)->allocate(); }
int ibh_pool_share(void* p, int page) { return ((Pool*)p)->share(page); }
int ibh_pool_release(void* p, int page) { return ((Pool*)p)->release(page); }
int ibh_pool_refcount(void* p, int page) {
  Pool* pool = (Pool*)p;
  return page >= 0 && page < pool->num_pages ? pool->refs[page] : -1;
}
int ibh_pool_check(void* p) { return ((Pool*)p)->check(); }

// ---------------------------------------------------------------- the cache: pools, tables, slots
void* ibh_cache_new(int n_groups, const int* windows, int page_size, int num_pages, int max_requests, int max_tokens) {
  if (n_groups < 0 || page_size <= 0 || num_pages <= 0 || max_requests <= 0 || max_tokens <= 0) {
    fail(1, "cache: sizes must be positive");
    return nullptr;
  }
  Cache* c = new Cache();
  c->page_size = page_size;
  c->max_requests = max_requests;
  c->max_tokens = max_tokens;
  c->table_width = (max_tokens + page_size - 1) / page_size;
  c->windows.assign(windows, windows + n_groups);
  for (int g = 0; g < n_groups; g++) c->pools.emplace_back(num_pages);
  c->tables.assign((size_t)n_groups * max_requests * c->table_width, -1);
  c->length.assign(max_requests, 0);
  c->live.assign(max_requests, 0);
  for (int s = max_requests - 1; s >= 0; s--) c->free_slots.push_back(s);
  return c;
}
void ibh_cache_free(void* c) { delete (Cache*)c; }
void* ibh_cache_pool(void* c, int g) { return &((Cache*)c)->pools[g]; }
int* ibh_cache_tables(void* c) { return ((Cache*)c)->tables.data(); }
int ibh_cache_table_width(void* c) { return ((Cache*)c)->table_width; }
int ibh_cache_free_slots(void* c) { return (int)((Cache*)c)->free_slots.size(); }

// A slot with empty tables, or -1 when every slot is taken.
int ibh_cache_admit(void* cp) {
  Cache* c = (Cache*)cp;
  if (c->free_slots.empty()) return -1;
  const int slot = c->free_slots.back();
  c->free_slots.pop_back();
  c->live[slot] = 1;
  c->length[slot] = 0;
  return slot;
}

int ibh_cache_length(void* cp, int slot) {
  Cache* c = (Cache*)cp;
  return c->is_live(slot) ? c->length[slot] : -1;
}

// Per group, the pages to allocate before the slot (or, with slot < 0, a request not yet admitted that
// starts from `length`) holds new_length positions.
void ibh_cache_pages_missing(void* cp, int slot, int new_length, int length, int* out) {
  Cache* c = (Cache*)cp;
  const bool known = c->is_live(slot);
  const int cur = known ? c->length[slot] : length;
  const int last = c->pages_for(new_length);
  for (int g = 0; g < (int)c->pools.size(); g++) {
    const int first = c->first_live_page(g, cur);
    int n = 0;
    if (!known) {
      n = last > first ? last - first : 0;
    } else {
      const int* row = c->row(g, slot);
      for (int p = first; p < last && p < c->table_width; p++) n += row[p] < 0;
    }
    out[g] = n;
  }
}

// Allocate, in every group, the pages for positions up to new_length - 1. All or nothing.
// 0: done; 1: a group has no page left (nothing changed); 2: beyond the per-request limit; 3: unknown slot.
int ibh_cache_extend(void* cp, int slot, int new_length) {
  Cache* c = (Cache*)cp;
  if (!c->is_live(slot)) return fail(3, "slot %d holds no request", slot);
  if (new_length > c->max_tokens) return fail(2, "%d tokens, more than the limit of %d", new_length, c->max_tokens);
  std::vector<std::pair<int, int>> taken;
  const int last = c->pages_for(new_length);
  for (int g = 0; g < (int)c->pools.size(); g++) {
    int* row = c->row(g, slot);
    for (int p = c->first_live_page(g, c->length[slot]); p < last; p++) {
      if (row[p] >= 0) continue;
      const int page = c->pools[g].allocate();
      if (page < 0) {
        for (auto& t : taken) {
          int* r = c->row(t.first, slot);
          c->pools[t.first].release(r[t.second]);
          r[t.second] = -1;
        }
        return fail(1, "needs a page for positions %d.. but group %d has none free (%d pages, all in use)", p * c->page_size, g,
                    c->pools[g].num_pages);
      }
      row[p] = page;
      taken.emplace_back(g, p);
    }
  }
  return 0;
}

// Undo an extend that no commit followed: free the pages beyond the committed length.
int ibh_cache_shrink_to_committed(void* cp, int slot) {
  Cache* c = (Cache*)cp;
  if (!c->is_live(slot)) return fail(3, "slot %d holds no request", slot);
  const int keep = c->pages_for(c->length[slot]);
  for (int g = 0; g < (int)c->pools.size(); g++) {
    int* row = c->row(g, slot);
    for (int p = keep; p < c->table_width; p++)
      if (row[p] >= 0) {
        c->pools[g].release(row[p]);
        row[p] = -1;
      }
  }
  return 0;
}

// The slot now holds new_length positions; windowed groups give back the pages that passed.
int ibh_cache_commit(void* cp, int slot, int new_length) {
  Cache* c = (Cache*)cp;
  if (!c->is_live(slot)) return fail(3, "slot %d holds no request", slot);
  c->length[slot] = new_length;
  for (int g = 0; g < (int)c->pools.size(); g++) {
    if (c->windows[g] <= 0) continue;
    const int first = c->first_live_page(g, new_length);
    int* row = c->row(g, slot);
    for (int p = 0; p < first && p < c->table_width; p++)
      if (row[p] >= 0) {
        c->pools[g].release(row[p]);
        row[p] = -1;
      }
  }
  return 0;
}

// The request ends: all its pages and its slot are given back.
int ibh_cache_release(void* cp, int slot) {
  Cache* c = (Cache*)cp;
  if (!c->is_live(slot)) return fail(3, "slot %d holds no request", slot);
  for (int g = 0; g < (int)c->pools.size(); g++) {
    int* row = c->row(g, slot);
    for (int p = 0; p < c->table_width; p++)
      if (row[p] >= 0) {
        c->pools[g].release(row[p]);
        row[p] = -1;
      }
  }
  c->live[slot] = 0;
  c->length[slot] = 0;
  c->free_slots.push_back(slot);
  return 0;
}

// What a step of single decoded tokens needs for its n rows, written where the caller's (pinned) input block
// has it: positions (the rows' committed lengths), and per group the rows' block tables, tables_out[g] being
// int32 [rows][table_width] of which the first n rows are written.
int ibh_cache_fill_rows(void* cp, const int* slots, int n, int* positions, int** tables_out) {
  Cache* c = (Cache*)cp;
  for (int i = 0; i < n; i++) {
    if (!c->is_live(slots[i])) return fail(3, "slot %d holds no request", slots[i]);
    positions[i] = c->length[slots[i]];
  }
  for (int g = 0; g < (int)c->pools.size(); g++)
    for (int i = 0; i < n; i++) memcpy(tables_out[g] + (size_t)i * c->table_width, c->row(g, slots[i]), sizeof(int) * c->table_width);
  return 0;
}

// No page lost, held twice or freed twice: every pool is consistent, a page's reference count equals the
// number of table entries that name it, and every slot is either held or free, once.
int ibh_cache_check(void* cp) {
  Cache* c = (Cache*)cp;
  for (int g = 0; g < (int)c->pools.size(); g++) {
    if (int e = c->pools[g].check()) return e;
    std::vector<int> counts(c->pools[g].num_pages, 0);
    for (int s = 0; s < c->max_requests; s++) {
      const int* row = c->row(g, s);
      for (int p = 0; p < c->table_width; p++) {
        if (row[p] < 0) continue;
        if (!c->live[s]) return fail(1, "group %d: free slot %d still names page %d", g, s, row[p]);
        if (row[p] >= c->pools[g].num_pages) return fail(1, "group %d: slot %d names page %d, outside the pool", g, s, row[p]);
        counts[row[p]]++;
      }
    }
    for (int p = 0; p < c->pools[g].num_pages; p++)
      if (counts[p] != c->pools[g].refs[p])
        return fail(1, "group %d: page %d is named by %d table entries but has reference count %d", g, p, counts[p], c->pools[g].refs[p]);
  }
  std::vector<char> seen(c->max_requests, 0);
  int held = 0;
  for (int s = 0; s < c->max_requests; s++) held += c->live[s] != 0;
  for (int s : c->free_slots) {
    if (s < 0 || s >= c->max_requests || seen[s] || c->live[s])
      return fail(1, "state slots are inconsistent: a slot is lost, held twice or both held and free");
    seen[s] = 1;
  }
  if (held + (int)c->free_slots.size() != c->max_requests) return fail(1, "state slots are inconsistent: a slot is lost, held twice or both held and free");
  return 0;
}

}  // extern "C"
