// The host side of the engine in native code: page pools, the cache manager and the scheduler.
//
// These are the decisions that run between two steps of the GPU: which pages a request holds,
// which requests run next and with how many tokens, who is preempted when pages run out.  The
// policies follow the reference's BlockManager and Scheduler (src/block_manager.cpp,
// src/scheduler.cpp) with the changes described at each class.  Python reaches them through the C
// functions at the end of the file (csrc/host.py); a plain Python restatement of the same classes
// lives with the tests and is compared with this code decision by decision.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <deque>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#define NVH_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_last_error;

enum { OK = 0, ERR_NO_PAGES = -1, ERR_NO_SLOT = -2, ERR_STATE = -3, ERR_NO_PROGRESS = -4, ERR_POOL_TOO_SMALL = -5 };

int fail(int code, const std::string& msg) {
  g_last_error = msg;
  return code;
}

uint64_t splitmix64(uint64_t x) {
  x += 0x9E3779B97F4A7C15ULL;
  x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ULL;
  x = (x ^ (x >> 27)) * 0x94D049BB133111EBULL;
  return x ^ (x >> 31);
}

// Hash of one full page given the hash of the page before it (src/block_manager.cpp:28-35).
uint64_t chain_hash(const int* tokens, int n, bool has_prefix, uint64_t prefix) {
  uint64_t h = has_prefix ? prefix : 0x243F6A8885A308D3ULL;
  h ^= 0x1C6E4A8DC4B3F8A1ULL + (uint64_t)n * 0x9E3779B97F4A7C15ULL;
  for (int i = 0; i < n; ++i) h = splitmix64(h ^ (uint64_t)(uint32_t)tokens[i]);
  return h;
}

// ------------------------------------------------------------------------------------------ BlockPool
// Pages of one layer group: a free list, reference counts and (optionally) hashes of full pages.
// Fresh pages come from the front of the free list, a released page goes to its back and keeps its
// hash until it is handed out again, so that a later request with the same prefix can revive it
// (src/block_manager.cpp:37-54, 85-93).  The free list is a doubly linked list over page ids, so
// reviving a page from its middle costs O(1).
class BlockPool {
 public:
  int num_pages, page_size;
  std::vector<int> ref_count;
  std::vector<uint8_t> has_hash, in_free;
  std::vector<uint64_t> page_hash;
  std::vector<std::vector<int>> page_tokens;
  std::unordered_map<uint64_t, int> hash_to_page;
  std::vector<int> prev, next;
  int head = -1, tail = -1, n_free = 0;

  BlockPool(int n, int ps)
      : num_pages(n), page_size(ps), ref_count(n, 0), has_hash(n, 0), in_free(n, 0), page_hash(n, 0), page_tokens(n),
        prev(n, -1), next(n, -1) {
    for (int i = 0; i < n; ++i) push_back(i);
  }
  void push_back(int p) {
    prev[p] = tail;
    next[p] = -1;
    if (tail >= 0) next[tail] = p; else head = p;
    tail = p;
    in_free[p] = 1;
    ++n_free;
  }
  void unlink(int p) {
    if (prev[p] >= 0) next[prev[p]] = next[p]; else head = next[p];
    if (next[p] >= 0) prev[next[p]] = prev[p]; else tail = prev[p];
    in_free[p] = 0;
    --n_free;
  }
  void forget(int p) {
    if (has_hash[p]) {
      auto it = hash_to_page.find(page_hash[p]);
      if (it != hash_to_page.end() && it->second == p) hash_to_page.erase(it);
    }
    has_hash[p] = 0;
    page_tokens[p].clear();
  }
  int allocate() {                       // a fresh page with one reference, or -1
    if (head < 0) return -1;
    int p = head;
    unlink(p);
    forget(p);
    ref_count[p] = 1;
    return p;
  }
  int share(int p) {                     // one more reference to a page found by its hash; a free page is revived
    if (ref_count[p] == 0) {
      if (!in_free[p]) return fail(ERR_STATE, "page " + std::to_string(p) + " is neither used nor free");
      unlink(p);
    }
    ++ref_count[p];
    return OK;
  }
  int release(int p) {
    if (ref_count[p] <= 0) return fail(ERR_STATE, "page " + std::to_string(p) + " released more often than taken");
    if (--ref_count[p] == 0) push_back(p);
    return OK;
  }
  int lookup(uint64_t h, const int* tokens, int n) const {
    auto it = hash_to_page.find(h);
    if (it == hash_to_page.end()) return -1;
    const auto& pt = page_tokens[it->second];
    if ((int)pt.size() != n || !std::equal(pt.begin(), pt.end(), tokens)) return -1;
    return it->second;
  }
  void set_hash(int p, uint64_t h, const int* tokens, int n) {
    forget(p);
    has_hash[p] = 1;
    page_hash[p] = h;
    page_tokens[p].assign(tokens, tokens + n);
    hash_to_page[h] = p;
  }
  // Every page is either free (no reference, once in the free list) or used; with `held` (page -> number
  // of block-table entries that name it) the counts must agree.
  int check(const std::vector<int>* held) const {
    std::vector<int> seen(num_pages, 0);
    int walked = 0;
    for (int p = head; p >= 0; p = next[p]) {
      if (++seen[p] > 1 || ++walked > num_pages) return fail(ERR_STATE, "the free list holds page " + std::to_string(p) + " twice");
    }
    if (walked != n_free) return fail(ERR_STATE, "the free list's length is wrong");
    for (int p = 0; p < num_pages; ++p) {
      const bool free_ = seen[p] == 1;
      if (free_ != (bool)in_free[p]) return fail(ERR_STATE, "page " + std::to_string(p) + ": free flag and free list disagree");
      if (free_ && ref_count[p] != 0)
        return fail(ERR_STATE, "page " + std::to_string(p) + " is free but has " + std::to_string(ref_count[p]) + " references");
      if (!free_ && ref_count[p] <= 0) return fail(ERR_STATE, "page " + std::to_string(p) + " is lost: not free, no reference");
      if (held && ref_count[p] != (*held)[p])
        return fail(ERR_STATE, "page " + std::to_string(p) + ": " + std::to_string(ref_count[p]) + " references, " +
                                   std::to_string((*held)[p]) + " table entries");
    }
    return OK;
  }
};

// ------------------------------------------------------------------------------------------ CacheManager
// Which pages and which state slot every live request holds.  Layers with the same needs form a group
// with pages and block tables of its own (one group for layers that read every earlier key, one per
// window size); a group with a window gives a page back as soon as every position in it lies before
// the window of the next row to run.  A request also holds one state slot from open to close.  Hashing
// of full pages, so that requests with a common prefix share them (src/block_manager.cpp:56-98,
// 121-134), is offered only for a single group without a window.
struct RequestCache {
  int64_t rid = 0;
  int slot = 0;
  std::vector<std::vector<int>> tables;   // per group: page ids, -1 where given back
  std::vector<uint8_t> dirty;             // per group: the table has changed since it last went to the device
  int num_tokens = 0;                     // tokens whose keys/values (or state) are in the cache
  int hashed_pages = 0;                   // leading full pages that carry a hash
  bool has_last = false;
  uint64_t last_hash = 0;
};

class CacheManager {
 public:
  std::vector<int> windows;
  int page_size, max_requests;
  std::vector<BlockPool> pools;
  std::vector<int> free_slots;            // a stack: slot 0 is handed out first
  std::unordered_map<int64_t, RequestCache> requests;
  bool prefix_caching;

  // `has_state`: some layer keeps a fixed-size state per request instead of (or beside) pages.  Such a state has
  // seen every token of its request, so a request must never skip tokens that another request's pages hold:
  // prefix sharing is refused then, as it is for more than one group or a window.  `groups` may be 0 (a model
  // without paged layers): requests then hold a state slot and nothing else.
  CacheManager(const int* w, const int* n_pages, int groups, int ps, int max_req, bool prefix, bool has_state)
      : windows(w, w + groups), page_size(ps), max_requests(max_req) {
    for (int g = 0; g < groups; ++g) pools.emplace_back(n_pages[g], ps);
    for (int s = max_req - 1; s >= 0; --s) free_slots.push_back(s);
    prefix_caching = prefix && !has_state && groups == 1 && windows[0] == 0;
  }
  RequestCache* find(int64_t rid) {
    auto it = requests.find(rid);
    return it == requests.end() ? nullptr : &it->second;
  }
  int open(int64_t rid) {
    if (requests.count(rid)) return fail(ERR_STATE, "request is already open");
    if (free_slots.empty()) return fail(ERR_NO_SLOT, "no free state slot");
    RequestCache rc;
    rc.rid = rid;
    rc.slot = free_slots.back();
    free_slots.pop_back();
    rc.tables.resize(pools.size());
    rc.dirty.assign(pools.size(), 1);
    const int slot = rc.slot;
    requests.emplace(rid, std::move(rc));
    return slot;
  }
  int close(int64_t rid) {
    auto it = requests.find(rid);
    if (it == requests.end()) return fail(ERR_STATE, "request is not open");
    for (size_t g = 0; g < pools.size(); ++g) {
      auto& table = it->second.tables[g];
      for (auto p = table.rbegin(); p != table.rend(); ++p)      // reverse order, as src/block_manager.cpp:100-108
        if (*p >= 0) {
          int rc = pools[g].release(*p);
          if (rc) return rc;
        }
    }
    free_slots.push_back(it->second.slot);
    requests.erase(it);
    return OK;
  }
  int first_needed_page(int g, int start) const {    // lowest page that rows from position `start` on still read
    const int w = windows[g];
    if (w <= 0) return 0;
    return std::max(0, start + 1 - w) / page_size;
  }
  void pages_needed(const RequestCache& rc, int start, int end, int* out) const {
    for (size_t g = 0; g < pools.size(); ++g) {
      const auto& table = rc.tables[g];
      const int total = (end + page_size - 1) / page_size;
      const int fresh = std::max(0, total - (int)table.size());
      const int first = std::min(first_needed_page((int)g, start), (int)table.size());
      int back = 0;
      for (int i = 0; i < first; ++i)
        if (table[i] >= 0 && pools[g].ref_count[table[i]] == 1) ++back;
      out[g] = fresh - back;
    }
  }
  bool can_extend(const RequestCache& rc, int start, int end) const {
    std::vector<int> need(pools.size());
    pages_needed(rc, start, end, need.data());
    for (size_t g = 0; g < pools.size(); ++g)
      if (need[g] > pools[g].n_free) return false;
    return true;
  }
  // Makes the cache ready for rows at positions [start, end): gives back pages that have left the window,
  // then takes pages up to `end`.  ERR_NO_PAGES (nothing but the give-back changed) if a group runs out.
  int extend(int64_t rid, int start, int end) {
    RequestCache* rc = find(rid);
    if (!rc) return fail(ERR_STATE, "request is not open");
    if (start != rc->num_tokens)
      return fail(ERR_STATE, "rows start at " + std::to_string(start) + " but " + std::to_string(rc->num_tokens) +
                                 " tokens are cached");
    for (size_t g = 0; g < pools.size(); ++g) {
      auto& table = rc->tables[g];
      const int first = std::min(first_needed_page((int)g, start), (int)table.size());
      for (int i = 0; i < first; ++i)
        if (table[i] >= 0) {
          int r = pools[g].release(table[i]);
          if (r) return r;
          table[i] = -1;
          rc->dirty[g] = 1;
        }
    }
    if (!can_extend(*rc, start, end)) return fail(ERR_NO_PAGES, "no free blocks");
    for (size_t g = 0; g < pools.size(); ++g) {
      auto& table = rc->tables[g];
      const int total = (end + page_size - 1) / page_size;
      while ((int)table.size() < total) {
        table.push_back(pools[g].allocate());
        rc->dirty[g] = 1;
      }
    }
    return OK;
  }
  // Rows up to `end` have run.  With prefix caching, `tokens` (the request's ids so far) lets newly
  // completed pages be hashed (src/block_manager.cpp:121-134).
  int commit(int64_t rid, int end, const int* tokens, int n_tokens) {
    RequestCache* rc = find(rid);
    if (!rc) return fail(ERR_STATE, "request is not open");
    rc->num_tokens = end;
    if (prefix_caching && tokens) {
      BlockPool& pool = pools[0];
      const int full = std::min(end, n_tokens) / page_size;
      for (int i = rc->hashed_pages; i < full; ++i) {
        const int* toks = tokens + (size_t)i * page_size;
        const uint64_t h = chain_hash(toks, page_size, rc->has_last, rc->last_hash);
        rc->has_last = true;
        rc->last_hash = h;
        if (pool.lookup(h, toks, page_size) < 0) pool.set_hash(rc->tables[0][i], h, toks, page_size);
      }
      rc->hashed_pages = std::max(rc->hashed_pages, full);
    }
    return OK;
  }
  // Pages holding the longest cached prefix of `tokens`; never the page that holds the last token, so that
  // at least one row is left to run (src/block_manager.cpp:56-73).
  int match_prefix(const int* tokens, int n, int* pages, uint64_t* hashes, int cap) const {
    if (!prefix_caching) return 0;
    const BlockPool& pool = pools[0];
    const int n_pages = (n + page_size - 1) / page_size;
    bool has = false;
    uint64_t h = 0;
    int count = 0;
    for (int i = 0; i + 1 < n_pages && count < cap; ++i) {
      const int* toks = tokens + (size_t)i * page_size;
      h = chain_hash(toks, page_size, has, h);
      has = true;
      const int p = pool.lookup(h, toks, page_size);
      if (p < 0) break;
      pages[count] = p;
      hashes[count] = h;
      ++count;
    }
    return count;
  }
  int adopt_prefix(int64_t rid, const int* pages, const uint64_t* hashes, int n) {
    RequestCache* rc = find(rid);
    if (!rc) return fail(ERR_STATE, "request is not open");
    if (n == 0) return rc->num_tokens;
    if (!prefix_caching) return fail(ERR_STATE, "adopt_prefix: this manager shares no pages");
    if (rc->num_tokens || !rc->tables[0].empty()) return fail(ERR_STATE, "adopt_prefix on a request that already holds pages");
    for (int i = 0; i < n; ++i) {
      int r = pools[0].share(pages[i]);
      if (r) return r;
      rc->tables[0].push_back(pages[i]);
      rc->dirty[0] = 1;
      rc->has_last = true;
      rc->last_hash = hashes[i];
    }
    rc->hashed_pages = n;
    rc->num_tokens = n * page_size;
    return rc->num_tokens;
  }
  // Fresh pages a request of `tokens_len` tokens would take after adopting the matched pages (a matched page
  // that is currently free must be revived, which costs a free page too).
  int new_pages_for(int tokens_len, const int* pages, int n) const {
    const int total = (tokens_len + page_size - 1) / page_size;
    int revived = 0;
    for (int i = 0; i < n; ++i)
      if (pools[0].ref_count[pages[i]] == 0) ++revived;
    return total - n + revived;
  }
  // The device's copies of the block tables can no longer be trusted (a step was prepared but never ran): every
  // request's tables travel again with its next step.
  void touch_all() {
    for (auto& kv : requests) std::fill(kv.second.dirty.begin(), kv.second.dirty.end(), 1);
  }
  int check() const {
    std::vector<uint8_t> used(max_requests, 0);
    for (const auto& kv : requests) {
      const int s = kv.second.slot;
      if (s < 0 || s >= max_requests || used[s]) return fail(ERR_STATE, "a state slot is held twice");
      used[s] = 1;
    }
    for (int s : free_slots)
      if (s < 0 || s >= max_requests || used[s]) return fail(ERR_STATE, "a state slot is held twice");
      else used[s] = 1;
    if (requests.size() + free_slots.size() != (size_t)max_requests) return fail(ERR_STATE, "a state slot is lost");
    for (size_t g = 0; g < pools.size(); ++g) {
      std::vector<int> held(pools[g].num_pages, 0);
      for (const auto& kv : requests)
        for (int p : kv.second.tables[g])
          if (p >= 0) ++held[p];
      int r = pools[g].check(&held);
      if (r) return r;
    }
    return OK;
  }
};

// ------------------------------------------------------------------------------------------ Scheduler
// Admits requests, cuts prompts into portions under a token budget, decodes, finishes and frees.
// Unlike the reference's scheduler (src/scheduler.cpp:23-89), which runs either prompt portions or
// decode tokens in a step, every step takes one decode token of each running request first and fills
// the rest of the token budget with prompt portions.  Kept from it: FIFO admission (27-35), a sequence
// moves to `running` when its whole prompt is cached (45-50), recompute-preemption of the most recently
// admitted running sequence when pages run out (16-21, 61-71), finishing on the stop token or
// max_tokens (101-108).
struct Seq {
  int64_t id;
  std::vector<int> tokens;
  int num_prompt;
  int max_tokens;
  bool ignore_eos;
  int status = 0;          // 0 waiting, 1 running, 2 finished
  int num_preemptions = 0;
};

struct Scheduled {
  Seq* seq;
  int start, count, samples;
};

class Scheduler {
 public:
  CacheManager* m;
  int max_num_seqs, max_batched, max_model_len, eos, prefill_chunk;
  std::deque<Seq*> waiting, running;
  std::unordered_map<int64_t, std::unique_ptr<Seq>> seqs;
  int num_preemptions = 0;

  Scheduler(CacheManager* mgr, int max_seqs, int max_tok, int max_len, int eos_, int chunk)
      : m(mgr), max_num_seqs(max_seqs), max_batched(max_tok), max_model_len(max_len), eos(eos_), prefill_chunk(chunk) {}

  int cached(const Seq* s) const {
    auto it = m->requests.find(s->id);
    return it == m->requests.end() ? 0 : it->second.num_tokens;
  }
  bool finished() const { return waiting.empty() && running.empty(); }

  // Gives back what the sequence holds and queues it at the front (src/scheduler.cpp:16-21).
  void preempt(Seq* s) {
    s->status = 0;
    ++s->num_preemptions;
    ++num_preemptions;
    if (m->find(s->id)) m->close(s->id);
    waiting.push_front(s);
  }

  int schedule(std::vector<Scheduled>& out) {
    out.clear();
    int budget = max_batched;
    const int preempted_before = num_preemptions;

    // 1. one token for every running sequence, oldest first
    std::deque<Seq*> kept;
    while (!running.empty() && (int)out.size() < max_num_seqs && budget > 0) {
      Seq* s = running.front();
      running.pop_front();
      const int n = cached(s);
      bool ok = true;
      for (;;) {
        const int rc = m->extend(s->id, n, n + 1);           // takes the page now (src/scheduler.cpp:75)
        if (rc == OK) break;
        if (rc != ERR_NO_PAGES) return rc;
        if (!running.empty()) {
          Seq* victim = running.back();
          running.pop_back();
          preempt(victim);
        } else if (!kept.empty() && kept.back() != s) {
          Seq* victim = kept.back();
          kept.pop_back();
          out.erase(std::remove_if(out.begin(), out.end(), [&](const Scheduled& x) { return x.seq == victim; }), out.end());
          ++budget;
          preempt(victim);
        } else {
          preempt(s);
          ok = false;
          break;
        }
      }
      if (!ok) break;
      out.push_back({s, n, 1, 1});
      kept.push_back(s);
      --budget;
    }
    for (Seq* s : running) kept.push_back(s);
    running.swap(kept);

    // 2. prompt portions from the waiting queue, in order; no admission in a step that had to preempt
    while (!waiting.empty() && (int)out.size() < max_num_seqs && budget > 0 && num_preemptions == preempted_before) {
      Seq* s = waiting.front();
      bool opened_here = false;
      const int n_tok = (int)s->tokens.size();
      if (!m->find(s->id)) {
        if (m->free_slots.empty()) break;
        std::vector<int> pages(n_tok / m->page_size + 1);
        std::vector<uint64_t> hashes(pages.size());
        const int matched = m->match_prefix(s->tokens.data(), n_tok, pages.data(), hashes.data(), (int)pages.size());
        const int cap = prefill_chunk ? prefill_chunk : budget;
        const int first = std::min(std::min(n_tok - matched * m->page_size, budget), cap);
        const int end = matched * m->page_size + first;
        bool fits = m->pools.empty() || m->new_pages_for(end, pages.data(), matched) <= m->pools[0].n_free;
        for (size_t g = 1; g < m->pools.size() && fits; ++g)
          if ((end + m->page_size - 1) / m->page_size > m->pools[g].n_free) fits = false;
        if (!fits) break;
        m->open(s->id);
        m->adopt_prefix(s->id, pages.data(), hashes.data(), matched);
        opened_here = true;
      }
      const int start = cached(s);
      const int cap = prefill_chunk ? prefill_chunk : budget;
      const int count = std::min(std::min(n_tok - start, budget), cap);
      const int rc = m->extend(s->id, start, start + count);
      if (rc == ERR_NO_PAGES) {
        if (opened_here) m->close(s->id);
        break;
      }
      if (rc != OK) return rc;
      const bool completes = start + count == n_tok;
      out.push_back({s, start, count, completes ? 1 : 0});
      budget -= count;
      if (!completes) break;     // the head of the queue is part way through its prompt; it goes on next step
      waiting.pop_front();
      s->status = 1;
      running.push_back(s);
    }

    if (!out.empty() || finished()) return OK;
    // 3. nothing can run: free pages held by waiting sequences, newest first, and try again
    for (auto it = waiting.rbegin(); it != waiting.rend() && (it + 1) != waiting.rend(); ++it) {
      Seq* v = *it;
      if (m->find(v->id)) {
        m->close(v->id);
        ++v->num_preemptions;
        ++num_preemptions;
        return schedule(out);
      }
    }
    Seq* head = waiting.empty() ? nullptr : waiting.front();
    if (head && m->find(head->id) && cached(head) > 0)
      return fail(ERR_POOL_TOO_SMALL, "scheduler could not make progress: the cache pool is smaller than one request");
    return fail(ERR_NO_PROGRESS, "scheduler could not make progress");
  }

  // `sampled[i]` is the token drawn for out[i] where out[i].samples; finished sequences' ids go to `done`.
  int postprocess(const std::vector<Scheduled>& out, const int* sampled, std::vector<int64_t>& done) {
    done.clear();
    for (size_t i = 0; i < out.size(); ++i) {
      Seq* s = out[i].seq;
      if (!m->find(s->id)) continue;                          // preempted after it was scheduled
      int rc = m->commit(s->id, out[i].start + out[i].count, s->tokens.data(), (int)s->tokens.size());
      if (rc) return rc;
      if (!out[i].samples) continue;
      const int token = sampled[i];
      s->tokens.push_back(token);
      const int completion = (int)s->tokens.size() - s->num_prompt;
      if ((!s->ignore_eos && eos >= 0 && token == eos) || completion >= s->max_tokens || (int)s->tokens.size() >= max_model_len) {
        s->status = 2;
        m->close(s->id);
        auto it = std::find(running.begin(), running.end(), s);
        if (it != running.end()) running.erase(it);
        done.push_back(s->id);
      }
    }
    return OK;
  }
};

struct SchedHandle {
  Scheduler s;
  std::vector<Scheduled> last;
  std::vector<int64_t> done;
  SchedHandle(CacheManager* m, int a, int b, int c, int d, int e) : s(m, a, b, c, d, e) {}
};

}  // namespace

// =============================================================================================== C interface
NVH_API const char* nvh_last_error() { return g_last_error.c_str(); }
NVH_API uint64_t nvh_chain_hash(const int* tokens, int n, int has_prefix, uint64_t prefix) {
  return chain_hash(tokens, n, has_prefix != 0, prefix);
}

// ---- a pool on its own (the manager's pools are reached with nvh_manager_pool)
NVH_API void* nvh_pool_create(int num_pages, int page_size) { return num_pages < 0 ? nullptr : new BlockPool(num_pages, page_size); }
NVH_API void nvh_pool_destroy(void* p) { delete (BlockPool*)p; }
NVH_API int nvh_pool_num_pages(void* p) { return ((BlockPool*)p)->num_pages; }
NVH_API int nvh_pool_num_free(void* p) { return ((BlockPool*)p)->n_free; }
NVH_API int nvh_pool_ref_count(void* p, int page) { return ((BlockPool*)p)->ref_count[page]; }
NVH_API int nvh_pool_allocate(void* p) {
  int r = ((BlockPool*)p)->allocate();
  return r >= 0 ? r : fail(ERR_NO_PAGES, "no free blocks");
}
NVH_API int nvh_pool_share(void* p, int page) { return ((BlockPool*)p)->share(page); }
NVH_API int nvh_pool_release(void* p, int page) { return ((BlockPool*)p)->release(page); }
NVH_API int nvh_pool_lookup(void* p, uint64_t h, const int* tokens, int n) { return ((BlockPool*)p)->lookup(h, tokens, n); }
NVH_API void nvh_pool_set_hash(void* p, int page, uint64_t h, const int* tokens, int n) {
  ((BlockPool*)p)->set_hash(page, h, tokens, n);
}
NVH_API int nvh_pool_check(void* p, const int* held) {
  BlockPool* bp = (BlockPool*)p;
  if (!held) return bp->check(nullptr);
  std::vector<int> h(held, held + bp->num_pages);
  return bp->check(&h);
}

// ---- the cache manager
NVH_API void* nvh_manager_create(const int* windows, const int* num_pages, int groups, int page_size, int max_requests,
                                 int prefix_caching, int has_state) {
  return new CacheManager(windows, num_pages, groups, page_size, max_requests, prefix_caching != 0, has_state != 0);
}
NVH_API void nvh_manager_destroy(void* m) { delete (CacheManager*)m; }
NVH_API void* nvh_manager_pool(void* m, int g) { return &((CacheManager*)m)->pools[g]; }
NVH_API int nvh_manager_groups(void* m) { return (int)((CacheManager*)m)->pools.size(); }
NVH_API int nvh_manager_prefix_caching(void* m) { return ((CacheManager*)m)->prefix_caching ? 1 : 0; }
NVH_API int nvh_manager_free_slots(void* m) { return (int)((CacheManager*)m)->free_slots.size(); }
NVH_API int nvh_manager_num_requests(void* m) { return (int)((CacheManager*)m)->requests.size(); }
NVH_API int nvh_has(void* m, int64_t rid) { return ((CacheManager*)m)->find(rid) ? 1 : 0; }
NVH_API int nvh_open(void* m, int64_t rid) { return ((CacheManager*)m)->open(rid); }
NVH_API int nvh_close(void* m, int64_t rid) { return ((CacheManager*)m)->close(rid); }
NVH_API int nvh_extend(void* m, int64_t rid, int start, int end) { return ((CacheManager*)m)->extend(rid, start, end); }
NVH_API int nvh_can_extend(void* m, int64_t rid, int start, int end) {
  RequestCache* rc = ((CacheManager*)m)->find(rid);
  return rc && ((CacheManager*)m)->can_extend(*rc, start, end) ? 1 : 0;
}
NVH_API int nvh_pages_needed(void* m, int64_t rid, int start, int end, int* out) {
  RequestCache* rc = ((CacheManager*)m)->find(rid);
  if (!rc) return fail(ERR_STATE, "request is not open");
  ((CacheManager*)m)->pages_needed(*rc, start, end, out);
  return OK;
}
NVH_API int nvh_commit(void* m, int64_t rid, int end, const int* tokens, int n) {
  return ((CacheManager*)m)->commit(rid, end, tokens, n);
}
// info: 0 slot, 1 num_tokens, 2 hashed_pages
NVH_API int nvh_request_info(void* m, int64_t rid, int what) {
  RequestCache* rc = ((CacheManager*)m)->find(rid);
  if (!rc) return fail(ERR_STATE, "request is not open");
  return what == 0 ? rc->slot : (what == 1 ? rc->num_tokens : rc->hashed_pages);
}
// Copies the block table of a request in group g into out (at most cap entries); returns its length.
NVH_API int nvh_table(void* m, int64_t rid, int g, int* out, int cap) {
  RequestCache* rc = ((CacheManager*)m)->find(rid);
  if (!rc) return fail(ERR_STATE, "request is not open");
  const auto& t = rc->tables[g];
  const int n = (int)t.size();
  if (out) std::memcpy(out, t.data(), sizeof(int) * (size_t)std::min(n, cap));
  return n;
}
NVH_API int nvh_match_prefix(void* m, const int* tokens, int n, int* pages, uint64_t* hashes, int cap) {
  return ((CacheManager*)m)->match_prefix(tokens, n, pages, hashes, cap);
}
NVH_API int nvh_adopt_prefix(void* m, int64_t rid, const int* pages, const uint64_t* hashes, int n) {
  return ((CacheManager*)m)->adopt_prefix(rid, pages, hashes, n);
}
NVH_API int nvh_new_pages_for(void* m, int tokens_len, const int* pages, int n) {
  return ((CacheManager*)m)->new_pages_for(tokens_len, pages, n);
}
NVH_API int nvh_manager_check(void* m) { return ((CacheManager*)m)->check(); }

// Rows up to ends[i] of request rids[i] have run (no hashing of pages: the caller that wants it commits one by one).
NVH_API int nvh_commit_many(void* m, int S, const int64_t* rids, const int* ends) {
  CacheManager* cm = (CacheManager*)m;
  for (int i = 0; i < S; ++i) {
    const int r = cm->commit(rids[i], ends[i], nullptr, 0);
    if (r) return r;
  }
  return OK;
}

// ---- the index arrays of one step
// Layout of the one int32 buffer that carries a step's index arrays to the device, every segment starting on a
// multiple of four ints: ids[T] pos[T] row_entry[T] cu[S+1] pos0[S] slot[S] want[W] single[S] (the batch rows of
// the entries that have one row, in entry order, then -1); per group table_src[S] (which uploaded row holds the
// entry's block table, -1: the device's copy is current) and table_len[S] (pages in the entry's table); with
// `sampling` temp[W] (float bits) and u[2W] (doubles); and last, per group, the uploaded rows
// [rows[g]][max_blocks] (rows == nullptr: S rows per group, the most a step can need).  offsets[] receives the
// 8 + 2 * groups (+ 2) + groups segment starts; the return value is the buffer's length in ints.
static inline int align4(int n) { return (n + 3) & ~3; }
NVH_API int nvh_step_layout(int S, int T, int W, int groups, int max_blocks, int sampling, const int* rows,
                            int* offsets) {
  int off = 0, k = 0;
  auto seg = [&](long long len) {
    if (offsets) offsets[k] = off;
    ++k;
    off = align4(off + (int)len);
  };
  const int lens[8] = {T, T, T, S + 1, S, S, W, S};
  for (int i = 0; i < 8; ++i) seg(lens[i]);
  for (int g = 0; g < groups; ++g) {
    seg(S);
    seg(S);
  }
  if (sampling) {
    seg(W);
    seg(2 * W);
  }
  for (int g = 0; g < groups; ++g) seg((long long)(rows ? rows[g] : S) * max_blocks);
  return off < 4 ? 4 : off;
}

// Takes the pages that the entries' next rows need and writes the step's arrays into `buf` (cap ints).  Entry i is
// request rids[i] with lens[i] next tokens (tokens[] holds them back to back) whose wanted places are
// wants[wants_cu[i] .. wants_cu[i+1]).  info[2i], info[2i+1] receive the entry's state slot and first position.
// Requests must be open.  A request's block table travels only if it has changed since it last did (a page taken
// or given back, a new request): the device keeps the tables of all live requests by state slot.  `fixed_rows` = 0:
// the uploaded rows are packed (as many as there are); > 0: every group has room for that many (the layout of a
// captured step, which must not depend on the step).  offsets[] receives the segment starts (see
// nvh_step_layout), uploaded[g] the number of rows that travel for group g.  Returns the length used, or an error:
// then nothing was written and no table counts as sent (the entries before the failing one keep the pages they
// took: taking them again is harmless).
NVH_API int nvh_prepare_step(void* m, int S, const int64_t* rids, const int* lens, const int* tokens,
                             const int* wants_cu, const int* wants, int max_blocks, int max_model_len, int sampling,
                             int fixed_rows, int* buf, int cap, int* info, int* offsets, int* uploaded) {
  CacheManager* cm = (CacheManager*)m;
  const int G = (int)cm->pools.size();
  if (G > 64) return fail(ERR_STATE, "too many cache groups");
  int T = 0;
  for (int i = 0; i < S; ++i) {
    if (lens[i] < 1) return fail(ERR_STATE, "an entry needs at least one token");
    T += lens[i];
  }
  const int W = wants_cu[S];
  // first everything that can fail: the pages, the places, the widths
  std::vector<RequestCache*> rcs(S);
  int n_up[64] = {0};
  for (int i = 0; i < S; ++i) {
    RequestCache* rc = cm->find(rids[i]);
    if (!rc) return fail(ERR_STATE, "request is not open");
    for (int j = 0; j < i; ++j)
      if (rcs[j] == rc) return fail(ERR_STATE, "a request appears twice in one step");
    rcs[i] = rc;
    const int start = rc->num_tokens, n = lens[i], end = start + n;
    if (end > max_model_len)
      return fail(ERR_STATE, "request " + std::to_string(rids[i]) + ": " + std::to_string(end) +
                                 " tokens exceed the longest sequence " + std::to_string(max_model_len));
    for (int w = wants_cu[i]; w < wants_cu[i + 1]; ++w)
      if (wants[w] < 0 || wants[w] >= n)
        return fail(ERR_STATE, "wanted place " + std::to_string(wants[w]) + " is not among the entry's " +
                                   std::to_string(n) + " tokens");
    const int r = cm->extend(rids[i], start, end);
    if (r) return r;
    for (int g = 0; g < G; ++g)
      if ((int)rc->tables[g].size() > max_blocks)
        return fail(ERR_STATE, "a request holds more pages than the block table is wide");
  }
  for (int i = 0; i < S; ++i)
    for (int g = 0; g < G; ++g) n_up[g] += rcs[i]->dirty[g] ? 1 : 0;
  int rows[64];
  for (int g = 0; g < G; ++g) {
    if (fixed_rows > 0 && n_up[g] > fixed_rows) return fail(ERR_STATE, "more block tables to send than the step has room for");
    rows[g] = fixed_rows > 0 ? fixed_rows : n_up[g];
  }
  int off[8 + 3 * 64 + 2];
  const int total = nvh_step_layout(S, T, W, G, max_blocks, sampling, rows, off);
  const int rows_at = 8 + 2 * G + (sampling ? 2 : 0);        // index of the first group's uploaded rows in off[]
  int used = G == 0 ? total : off[rows_at];                   // what travels ends with the last row that does
  for (int g = 0; g < G; ++g)
    if (n_up[g] > 0) used = align4(off[rows_at + g] + n_up[g] * max_blocks);
  if (used < 4) used = 4;
  if (used > cap || total > cap) return fail(ERR_STATE, "the step's arrays do not fit the staging buffer");
  std::fill(buf, buf + used, -1);
  int* ids = buf + off[0];
  int* pos = buf + off[1];
  int* row_entry = buf + off[2];
  int* cu = buf + off[3];
  int* pos0 = buf + off[4];
  int* slot = buf + off[5];
  int* want = buf + off[6];
  int* single = buf + off[7];
  int row = 0, n_single = 0;
  int next_up[64] = {0};
  cu[0] = 0;
  for (int i = 0; i < S; ++i) {
    RequestCache* rc = rcs[i];
    const int start = rc->num_tokens, n = lens[i];
    for (int j = 0; j < n; ++j) {
      ids[row + j] = tokens[row + j];
      pos[row + j] = start + j;
      row_entry[row + j] = i;
    }
    for (int w = wants_cu[i]; w < wants_cu[i + 1]; ++w) want[w] = row + wants[w];
    if (n == 1) single[n_single++] = row;
    pos0[i] = start;
    slot[i] = rc->slot;
    info[2 * i] = rc->slot;
    info[2 * i + 1] = start;
    for (int g = 0; g < G; ++g) {
      const auto& t = rc->tables[g];
      buf[off[8 + 2 * g + 1] + i] = (int)t.size();
      if (!rc->dirty[g]) continue;              // table_src stays -1
      const int r = next_up[g]++;
      buf[off[8 + 2 * g] + i] = r;
      std::memcpy(buf + off[rows_at + g] + (size_t)r * max_blocks, t.data(), sizeof(int) * t.size());
      rc->dirty[g] = 0;
    }
    row += n;
    cu[i + 1] = row;
  }
  if (offsets) std::memcpy(offsets, off, sizeof(int) * (size_t)(rows_at + G));
  if (uploaded) std::memcpy(uploaded, n_up, sizeof(int) * (size_t)G);
  return used;
}
NVH_API void nvh_touch_tables(void* m) { ((CacheManager*)m)->touch_all(); }

// ---- the scheduler
NVH_API void* nvs_create(void* manager, int max_num_seqs, int max_batched_tokens, int max_model_len, int eos,
                         int prefill_chunk) {
  return new SchedHandle((CacheManager*)manager, max_num_seqs, max_batched_tokens, max_model_len, eos, prefill_chunk);
}
NVH_API void nvs_destroy(void* s) { delete (SchedHandle*)s; }
NVH_API int nvs_add(void* s, int64_t seq_id, const int* tokens, int n, int num_prompt, int max_tokens, int ignore_eos) {
  Scheduler& sc = ((SchedHandle*)s)->s;
  if (sc.seqs.count(seq_id)) return fail(ERR_STATE, "sequence id is already known");
  auto q = std::make_unique<Seq>();
  q->id = seq_id;
  q->tokens.assign(tokens, tokens + n);
  q->num_prompt = num_prompt;
  q->max_tokens = max_tokens;
  q->ignore_eos = ignore_eos != 0;
  Seq* raw = q.get();
  sc.seqs.emplace(seq_id, std::move(q));
  sc.waiting.push_back(raw);
  return OK;
}
NVH_API int nvs_is_finished(void* s) { return ((SchedHandle*)s)->s.finished() ? 1 : 0; }
NVH_API int nvs_num_preemptions(void* s) { return ((SchedHandle*)s)->s.num_preemptions; }
NVH_API int nvs_queue_sizes(void* s, int* waiting, int* running) {
  Scheduler& sc = ((SchedHandle*)s)->s;
  *waiting = (int)sc.waiting.size();
  *running = (int)sc.running.size();
  return OK;
}
// info: 0 status, 1 num_preemptions, 2 num_tokens
NVH_API int nvs_seq_info(void* s, int64_t seq_id, int what) {
  Scheduler& sc = ((SchedHandle*)s)->s;
  auto it = sc.seqs.find(seq_id);
  if (it == sc.seqs.end()) return fail(ERR_STATE, "unknown sequence");
  return what == 0 ? it->second->status : (what == 1 ? it->second->num_preemptions : (int)it->second->tokens.size());
}
NVH_API int nvs_forget(void* s, int64_t seq_id) {               // drops a finished sequence's record
  Scheduler& sc = ((SchedHandle*)s)->s;
  auto it = sc.seqs.find(seq_id);
  if (it == sc.seqs.end()) return OK;
  if (it->second->status != 2) return fail(ERR_STATE, "only finished sequences can be forgotten");
  sc.seqs.erase(it);
  return OK;
}
// One step's decisions.  Returns the number of scheduled entries (arrays filled up to cap) or an error.
NVH_API int nvs_schedule(void* s, int64_t* seq_ids, int* starts, int* counts, int* samples, int cap) {
  SchedHandle* h = (SchedHandle*)s;
  int rc = h->s.schedule(h->last);
  if (rc) return rc;
  const int n = (int)h->last.size();
  if (n > cap) return fail(ERR_STATE, "schedule: output arrays too short");
  for (int i = 0; i < n; ++i) {
    seq_ids[i] = h->last[i].seq->id;
    starts[i] = h->last[i].start;
    counts[i] = h->last[i].count;
    samples[i] = h->last[i].samples;
  }
  return n;
}
// After the step: `sampled[i]` for entry i of the last schedule (ignored where it did not sample).  Returns the
// number of finished sequences, their ids in `finished`.
NVH_API int nvs_postprocess(void* s, const int* sampled, int64_t* finished, int cap) {
  SchedHandle* h = (SchedHandle*)s;
  int rc = h->s.postprocess(h->last, sampled, h->done);
  if (rc) return rc;
  const int n = (int)h->done.size();
  for (int i = 0; i < n && i < cap; ++i) finished[i] = h->done[i];
  return n;
}

// A token that was recorded as a stand-in (a negative number, while the step that draws it was still running) gets
// its value.
NVH_API int nvs_patch_token(void* s, int64_t seq_id, int index, int token) {
  Scheduler& sc = ((SchedHandle*)s)->s;
  auto it = sc.seqs.find(seq_id);
  if (it == sc.seqs.end()) return fail(ERR_STATE, "unknown sequence");
  std::vector<int>& t = it->second->tokens;
  if (index < 0 || index >= (int)t.size()) return fail(ERR_STATE, "token index out of range");
  t[index] = token;
  return OK;
}
// A sequence turns out to have ended (its stop token was drawn in a step whose tokens were read late): it gives
// back what it holds and leaves its queue, wherever the decisions made meanwhile have put it.
NVH_API int nvs_finish_late(void* s, int64_t seq_id) {
  Scheduler& sc = ((SchedHandle*)s)->s;
  auto it = sc.seqs.find(seq_id);
  if (it == sc.seqs.end()) return fail(ERR_STATE, "unknown sequence");
  Seq* q = it->second.get();
  if (q->status == 2) return OK;
  q->status = 2;
  if (sc.m->find(q->id)) sc.m->close(q->id);
  auto r = std::find(sc.running.begin(), sc.running.end(), q);
  if (r != sc.running.end()) sc.running.erase(r);
  auto w = std::find(sc.waiting.begin(), sc.waiting.end(), q);
  if (w != sc.waiting.end()) sc.waiting.erase(w);
  return OK;
}
