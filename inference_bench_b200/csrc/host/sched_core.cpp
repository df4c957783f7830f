// The scheduler's decisions, in C++ behind a C interface (loaded with ctypes by engine/scheduler.py):
// which requests are admitted, which are preempted when pages run out, what every running request
// computes in the next step, and when a request is finished. It works on the cache core directly
// (slots, pages); token values, sampling parameters and request ids stay with the Python caller,
// which is told what was admitted, preempted and finished so that it can keep its own maps.
//
// Policy, after the reference's scheduler (crates/specrt/src/sched.rs; docs/specrt-scheduler.md):
//   * every step, each decoding request gets one row (sched.rs:1403-1418); if one of them needs a new
//     page and none is free, the most recently admitted request is preempted: its pages and slot are
//     given back and it returns to the front of the waiting queue, to be recomputed (sched.rs:1090-1130);
//   * the rest of the token budget goes to prompts: waiting requests are admitted first come first
//     served while a slot is free and all pages for their tokens plus one are free beyond a small
//     reserve (sched.rs:1132-1230, 959-961), then running prompts get portions, shortest remaining
//     first, each at most prefill_chunk tokens (sched.rs:1457-1530);
//   * the last portion of a prompt samples (sched.rs:1496-1497);
//   * a request finishes on a stop token, at max_tokens, or at the context limit (sched.rs:1577-1589).
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <deque>
#include <string>
#include <vector>

extern "C" {
// the cache core (cache_core.cpp)
int ibh_cache_admit(void*);
int ibh_cache_extend(void*, int, int);
int ibh_cache_release(void*, int);
int ibh_cache_free_slots(void*);
void ibh_cache_pages_missing(void*, int, int, int, int*);
void* ibh_cache_pool(void*, int);
int ibh_pool_num_pages(void*);
int ibh_pool_free_pages(void*);
}

namespace {

thread_local std::string g_sched_error;

struct Seq {
  int prompt_len = 0, n_tokens = 0, generated = 0, computed = 0, max_tokens = 0, preemptions = 0, slot = -1;
  long long order = 0;
  int state = 0;   // 0 gone, 1 waiting, 2 running
  bool decoding() const { return generated > 0 && computed == n_tokens - 1; }
  int remaining() const { return n_tokens - computed; }
};

struct Sched {
  void* cache;
  int n_groups, max_num_seqs, max_batched_tokens, prefill_chunk, limit;   // limit: min(max_ctx, the cache's tokens per request)
  std::vector<Seq> seqs;
  std::deque<int> waiting;
  std::vector<int> running;
  long long next_order = 0, total_preemptions = 0;

  int min_pool_pages() const {
    int m = -1;
    for (int g = 0; g < n_groups; g++) {
      const int n = ibh_pool_num_pages(ibh_cache_pool(cache, g));
      m = m < 0 ? n : std::min(m, n);
    }
    return m < 0 ? 0 : m;
  }
  bool can_extend_new(int new_length, int reserve) const {   // a request not yet admitted
    if (new_length > limit) return false;   // the cache's own limit is part of `limit`
    std::vector<int> missing(std::max(1, n_groups));
    ibh_cache_pages_missing(cache, -1, new_length, 0, missing.data());
    for (int g = 0; g < n_groups; g++)
      if (missing[g] + reserve > ibh_pool_free_pages(ibh_cache_pool(cache, g))) return false;
    return true;
  }
  void drop_running(int h) { running.erase(std::remove(running.begin(), running.end(), h), running.end()); }
  void release(int h) {
    Seq& s = seqs[h];
    if (s.state == 2) drop_running(h);
    if (s.slot >= 0) ibh_cache_release(cache, s.slot);
    s.slot = -1;
  }
};

}  // namespace

extern "C" {

const char* ibh_sched_last_error() { return g_sched_error.c_str(); }

void* ibh_sched_new(void* cache, int n_groups, int max_num_seqs, int max_batched_tokens, int prefill_chunk, int limit) {
  Sched* s = new Sched();
  s->cache = cache;
  s->n_groups = n_groups;
  s->max_num_seqs = max_num_seqs;
  s->max_batched_tokens = max_batched_tokens;
  s->prefill_chunk = prefill_chunk;
  s->limit = limit;
  return s;
}
void ibh_sched_free(void* s) { delete (Sched*)s; }

// A new request at the back of the waiting queue; returns its handle. What can never run is refused by the caller.
int ibh_sched_submit(void* sp, int prompt_len, int max_tokens) {
  Sched* s = (Sched*)sp;
  Seq q;
  q.prompt_len = q.n_tokens = prompt_len;
  q.max_tokens = max_tokens;
  q.state = 1;
  s->seqs.push_back(q);
  const int h = (int)s->seqs.size() - 1;
  s->waiting.push_back(h);
  return h;
}

// 0: unknown or gone; 1: it was waiting; 2: it was running (its pages and slot are given back).
int ibh_sched_cancel(void* sp, int h) {
  Sched* s = (Sched*)sp;
  if (h < 0 || h >= (int)s->seqs.size() || s->seqs[h].state == 0) return 0;
  Seq& q = s->seqs[h];
  const int was = q.state;
  if (was == 1) s->waiting.erase(std::remove(s->waiting.begin(), s->waiting.end(), h), s->waiting.end());
  else s->release(h);
  q.state = 0;
  return was;
}

int ibh_sched_n_waiting(void* sp) { return (int)((Sched*)sp)->waiting.size(); }
int ibh_sched_n_running(void* sp) { return (int)((Sched*)sp)->running.size(); }
void ibh_sched_waiting(void* sp, int* out) { std::copy(((Sched*)sp)->waiting.begin(), ((Sched*)sp)->waiting.end(), out); }
void ibh_sched_running(void* sp, int* out) { std::copy(((Sched*)sp)->running.begin(), ((Sched*)sp)->running.end(), out); }
long long ibh_sched_total_preemptions(void* sp) { return ((Sched*)sp)->total_preemptions; }

// 1 when something runs, nothing waits and every running request decodes: the state in which steps can be kept one ahead.
int ibh_sched_steady(void* sp) {
  Sched* s = (Sched*)sp;
  if (s->running.empty() || !s->waiting.empty()) return 0;
  for (int h : s->running)
    if (!s->seqs[h].decoding()) return 0;
  return 1;
}

// out[0..6] = n_tokens, generated, computed, order, preemptions, slot, state
void ibh_sched_get(void* sp, int h, long long* out) {
  const Seq& q = ((Sched*)sp)->seqs[h];
  out[0] = q.n_tokens, out[1] = q.generated, out[2] = q.computed, out[3] = q.order, out[4] = q.preemptions, out[5] = q.slot, out[6] = q.state;
}

// Decide the next step. Every decoder gets room for one more position (the newest request is preempted
// until it has), waiting requests are admitted, then the step's rows are listed: decoders first, one
// token each, then prompt portions, shortest remaining first. Output, each array sized by the caller
// for every live request: preempted handles; admitted (handle, slot) pairs; entries (handle, first
// position, tokens, 1 if the entry samples). counts[0..4] = preempted, admitted, entries, decode rows, prompt tokens.
void ibh_sched_plan(void* sp, int* preempted, int* admitted, int* entries, int* counts) {
  Sched* s = (Sched*)sp;
  int n_pre = 0, n_adm = 0, n_ent = 0;
  // ---- room for every decoder's next position
  std::vector<int> decoders;
  for (int h : s->running)
    if (s->seqs[h].decoding()) decoders.push_back(h);
  std::sort(decoders.begin(), decoders.end(), [&](int a, int b) { return s->seqs[a].order < s->seqs[b].order; });
  for (int h : decoders) {
    while (s->seqs[h].state == 2) {
      if (ibh_cache_extend(s->cache, s->seqs[h].slot, s->seqs[h].computed + 1) == 0) break;
      int victim = s->running[0];
      for (int r : s->running)
        if (s->seqs[r].order > s->seqs[victim].order) victim = r;
      Seq& v = s->seqs[victim];   // recompute later: everything it holds is freed; what it has emitted stays emitted
      s->release(victim);
      v.computed = 0;
      v.preemptions++;
      v.state = 1;
      s->total_preemptions++;
      s->waiting.push_front(victim);
      preempted[n_pre++] = victim;
    }
  }
  // ---- admission
  int n_dec = 0;
  for (int h : s->running) n_dec += s->seqs[h].decoding();
  const int budget = std::max(0, s->max_batched_tokens - n_dec);
  int planned = 0;
  for (int h : s->running)
    if (!s->seqs[h].decoding()) planned += std::min(s->seqs[h].remaining(), s->prefill_chunk);
  while (!s->waiting.empty() && planned < budget) {
    const int h = s->waiting.front();
    Seq& q = s->seqs[h];
    if ((int)s->running.size() >= s->max_num_seqs || ibh_cache_free_slots(s->cache) == 0) break;
    const int pool = s->min_pool_pages();
    const int reserve = s->running.empty() ? 0 : std::max(1, pool / 100);   // sched.rs:959-961
    if (!s->can_extend_new(q.n_tokens + 1, reserve)) break;
    s->waiting.pop_front();
    q.slot = ibh_cache_admit(s->cache);
    ibh_cache_extend(s->cache, q.slot, q.n_tokens + 1);
    q.order = s->next_order++;
    q.state = 2;
    s->running.push_back(h);
    admitted[2 * n_adm] = h;
    admitted[2 * n_adm + 1] = q.slot;
    n_adm++;
    planned += std::min(q.remaining(), s->prefill_chunk);
  }
  // ---- the step's rows
  int rows = 0, prompt_tokens = 0;
  for (int h : s->running) {
    const Seq& q = s->seqs[h];
    if (!q.decoding()) continue;
    entries[4 * n_ent] = h, entries[4 * n_ent + 1] = q.computed, entries[4 * n_ent + 2] = 1, entries[4 * n_ent + 3] = 1;
    n_ent++, rows++;
  }
  std::vector<int> prompts;
  for (int h : s->running)
    if (!s->seqs[h].decoding()) prompts.push_back(h);
  std::stable_sort(prompts.begin(), prompts.end(), [&](int a, int b) {
    const Seq &x = s->seqs[a], &y = s->seqs[b];
    return x.remaining() != y.remaining() ? x.remaining() < y.remaining() : x.order < y.order;
  });
  int left = s->max_batched_tokens - rows;
  for (int h : prompts) {
    if (left <= 0) break;
    const Seq& q = s->seqs[h];
    const int n = std::min({q.remaining(), s->prefill_chunk, left});
    entries[4 * n_ent] = h, entries[4 * n_ent + 1] = q.computed, entries[4 * n_ent + 2] = n, entries[4 * n_ent + 3] = n == q.remaining();
    n_ent++;
    left -= n;
    prompt_tokens += n;
  }
  counts[0] = n_pre, counts[1] = n_adm, counts[2] = n_ent, counts[3] = rows, counts[4] = prompt_tokens;
}

// The step ran: n more positions of the request are in the cache.
void ibh_sched_computed(void* sp, int h, int n) { ((Sched*)sp)->seqs[h].computed += n; }

// A sampled token arrives. 0: the request goes on; 1: it was a stop token (not counted); 2: it was the last
// one (max_tokens or the context limit). A finished request's pages and slot are given back at once.
int ibh_sched_accept(void* sp, int h, int is_stop) {
  Sched* s = (Sched*)sp;
  Seq& q = s->seqs[h];
  if (is_stop) {
    s->release(h);
    q.state = 0;
    return 1;
  }
  q.n_tokens++;
  q.generated++;
  if (q.generated >= q.max_tokens || q.n_tokens >= s->limit) {
    s->release(h);
    q.state = 0;
    return 2;
  }
  return 0;
}

}  // extern "C"
