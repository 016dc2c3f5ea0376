// Host side of the engine's runtime in C++: pools of pages, block tables, fixed-size state
// slots and the step transaction (reserve -> commit / roll back), the packing of a step's
// metadata, and the scheduler's decisions (admission, the next step's entries, finishing,
// preemption).  No device code; the Python classes in leone_b200/cache/pages.py,
// leone_b200/engine/batch.py and leone_b200/engine/scheduler.py are fronts over these functions.
//
// The reference keeps keys and values in growing segments per session and uses pages only as
// the unit of admission (crates/leone/src/kv.rs:14-31, 637-674; crates/leone/src/scheduler.rs:
// 652-667 rounds a reservation up to kv_page_tokens).  Here the pages are real: a request's
// tokens live in fixed-size pages scattered over a pool and found through its block table.
// What is kept from the reference is the transaction: space for a step is reserved before the
// step runs and a request's length advances only when the step is committed (prepare_append ->
// write_span -> commit_append, crates/leone/src/kv.rs:326-347, 791-927); a failed step rolls
// back.
//
// Layers with different needs form different groups.  A group has its own pool and its own
// block table per request.  Two kinds exist: "full" keeps every page until the request ends;
// "window" gives a page back as soon as every later query lies more than `window` tokens past
// its last token.  Requests are named by 64-bit ids (the Python front maps its hashable names).
//
// Every function returns a code (0 ok, 1 out of pages or slots, 2 a broken rule, -1 a bad
// handle or argument) and leaves a message for leone_host_last_error().
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <vector>

namespace {

enum Code { kOk = 0, kOutOfPages = 1, kRuleBroken = 2, kBadArgument = -1 };

thread_local std::string g_error;

int fail(Code code, const std::string& message) {
  g_error = message;
  return code;
}

// Free list over ids 0..n-1; LIFO, so what is given back is handed out again at once.
struct FreeList {
  int n = 0;
  std::vector<int> free_;
  std::vector<char> held;
  int high_water = 0;

  explicit FreeList(int count) : n(count), held(count, 0) {
    free_.reserve(count);
    for (int i = count - 1; i >= 0; --i) free_.push_back(i);
  }
  int num_free() const { return (int)free_.size(); }
  int num_held() const { return n - (int)free_.size(); }
  // All or nothing.
  int take(int count, std::vector<int>* out, const char* what) {
    if (count > (int)free_.size())
      return fail(kOutOfPages, std::string("asked for ") + std::to_string(count) + " " + what + ", " +
                                   std::to_string(free_.size()) + " free of " + std::to_string(n));
    for (int i = 0; i < count; ++i) {
      const int id = free_.back();
      free_.pop_back();
      if (held[id]) return fail(kRuleBroken, std::string(what) + " " + std::to_string(id) + " handed out twice");
      held[id] = 1;
      out->push_back(id);
    }
    high_water = std::max(high_water, num_held());
    return kOk;
  }
  int give_back(int id, const char* what) {
    if (id < 0 || id >= n || !held[id])
      return fail(kRuleBroken, std::string(what) + " " + std::to_string(id) + " freed but not held");
    held[id] = 0;
    free_.push_back(id);
    return kOk;
  }
};

struct Request {
  int slot = -1;
  long long committed = 0, reserved = 0;
  bool fresh = true;        // no step has been committed yet: a state slot must be cleared
  long long version = 0;    // changes whenever a block table changes other than by growing at its end
};

struct Group {
  int kind = 0;             // 0 full, 1 window
  long long window = 0;
  int page_tokens = 1;
  FreeList pool;
  std::unordered_map<long long, std::vector<int>> tables;   // request -> page per logical block; -1 where a window has passed

  Group(int kind_, long long window_, int page_tokens_, int pages)
      : kind(kind_), window(window_), page_tokens(page_tokens_), pool(pages) {}
  long long blocks_for(long long length) const { return (length + page_tokens - 1) / page_tokens; }
  // First logical block that a query at position >= committed can still read.
  long long first_live_block(long long committed) const {
    if (kind != 1) return 0;
    const long long oldest_key = committed - window + 1;
    return oldest_key <= 0 ? 0 : oldest_key / page_tokens;
  }
  long long pages_needed(const std::vector<int>& table, long long new_len) const {
    return std::max(0ll, blocks_for(new_len) - (long long)table.size());
  }
};

struct Manager {
  int page_tokens;
  std::vector<Group> groups;
  FreeList slots;
  std::unordered_map<long long, Request> requests;
  long long versions = 0;

  Manager(int page_tokens_, int num_slots) : page_tokens(page_tokens_), slots(num_slots) {}
  Request* find(long long rid) {
    auto it = requests.find(rid);
    return it == requests.end() ? nullptr : &it->second;
  }
};

int unknown(long long rid) { return fail(kRuleBroken, "request " + std::to_string(rid) + " is not open"); }

}  // namespace

extern "C" {

const char* leone_host_last_error() { return g_error.c_str(); }

// ---- a free list on its own (pages of one pool, or state slots) ---------------------------
void* leone_freelist_create(int count) { return count > 0 ? new FreeList(count) : nullptr; }
void leone_freelist_destroy(void* h) { delete static_cast<FreeList*>(h); }
int leone_freelist_num_free(void* h) { return static_cast<FreeList*>(h)->num_free(); }
int leone_freelist_high_water(void* h) { return static_cast<FreeList*>(h)->high_water; }
int leone_freelist_take(void* h, int count, int* out) {
  std::vector<int> got;
  const int r = static_cast<FreeList*>(h)->take(count, &got, "pages");
  if (r == kOk) std::copy(got.begin(), got.end(), out);
  return r;
}
int leone_freelist_give_back(void* h, const int* ids, int count) {
  for (int i = 0; i < count; ++i) {
    const int r = static_cast<FreeList*>(h)->give_back(ids[i], "page");
    if (r != kOk) return r;
  }
  return kOk;
}

// ---- the cache manager --------------------------------------------------------------------
void* leone_cache_create(int n_groups, const int* kinds, const long long* windows, int page_tokens,
                         int num_pages, int num_slots) {
  if (n_groups < 0 || page_tokens <= 0 || num_pages <= 0 || num_slots <= 0) return nullptr;
  for (int i = 0; i < n_groups; ++i)
    if ((kinds[i] != 0 && kinds[i] != 1) || (kinds[i] == 1 && windows[i] <= 0)) return nullptr;
  Manager* m = new Manager(page_tokens, num_slots);
  for (int i = 0; i < n_groups; ++i) m->groups.emplace_back(kinds[i], windows[i], page_tokens, num_pages);
  return m;
}
void leone_cache_destroy(void* h) { delete static_cast<Manager*>(h); }

int leone_cache_open(void* h, long long rid, int* slot) {
  Manager* m = static_cast<Manager*>(h);
  if (m->find(rid)) return fail(kRuleBroken, "request " + std::to_string(rid) + " is already open");
  std::vector<int> got;
  const int r = m->slots.take(1, &got, "state slots");
  if (r != kOk) return r;
  Request rc;
  rc.slot = got[0];
  rc.version = ++m->versions;
  m->requests[rid] = rc;
  for (Group& g : m->groups) g.tables[rid] = {};
  *slot = rc.slot;
  return kOk;
}

int leone_cache_close(void* h, long long rid) {
  Manager* m = static_cast<Manager*>(h);
  Request* rc = m->find(rid);
  if (!rc) return unknown(rid);
  for (Group& g : m->groups) {
    auto it = g.tables.find(rid);
    for (int p : it->second)
      if (p >= 0) {
        const int r = g.pool.give_back(p, "page");
        if (r != kOk) return r;
      }
    g.tables.erase(it);
  }
  const int r = m->slots.give_back(rc->slot, "state slot");
  m->requests.erase(rid);
  return r;
}

int leone_cache_is_open(void* h, long long rid) { return static_cast<Manager*>(h)->find(rid) ? 1 : 0; }
int leone_cache_num_open(void* h) { return (int)static_cast<Manager*>(h)->requests.size(); }

// what: 0 committed length, 1 reserved length, 2 slot, 3 fresh, 4 table version
int leone_cache_get(void* h, long long rid, int what, long long* value) {
  Request* rc = static_cast<Manager*>(h)->find(rid);
  if (!rc) return unknown(rid);
  switch (what) {
    case 0: *value = rc->committed; break;
    case 1: *value = rc->reserved; break;
    case 2: *value = rc->slot; break;
    case 3: *value = rc->fresh ? 1 : 0; break;
    case 4: *value = rc->version; break;
    default: return fail(kBadArgument, "unknown field");
  }
  return kOk;
}

// Would reserve succeed for these (request, new length) pairs together?  (1 yes, 0 no)
int leone_cache_can_reserve(void* h, int n, const long long* rids, const long long* new_lens) {
  Manager* m = static_cast<Manager*>(h);
  for (Group& g : m->groups) {
    long long need = 0;
    for (int i = 0; i < n; ++i) {
      auto it = g.tables.find(rids[i]);
      if (it == g.tables.end()) return 0;
      need += g.pages_needed(it->second, new_lens[i]);
    }
    if (need > g.pool.num_free()) return 0;
  }
  return 1;
}

// Take pages so each request can hold new_len tokens.  All or nothing.
int leone_cache_reserve(void* h, int n, const long long* rids, const long long* new_lens) {
  Manager* m = static_cast<Manager*>(h);
  for (int i = 0; i < n; ++i) {
    Request* rc = m->find(rids[i]);
    if (!rc) return unknown(rids[i]);
    if (new_lens[i] < rc->committed)
      return fail(kRuleBroken, "request " + std::to_string(rids[i]) + ": cannot reserve " +
                                   std::to_string(new_lens[i]) + " below its length");
  }
  if (!leone_cache_can_reserve(h, n, rids, new_lens)) return fail(kOutOfPages, "not enough free pages for this step");
  for (int i = 0; i < n; ++i) {
    Request* rc = m->find(rids[i]);
    for (Group& g : m->groups) {
      std::vector<int>& table = g.tables[rids[i]];
      const int r = g.pool.take((int)g.pages_needed(table, new_lens[i]), &table, "pages");
      if (r != kOk) return r;
    }
    rc->reserved = std::max(rc->reserved, new_lens[i]);
  }
  return kOk;
}

// The step that wrote tokens up to new_len succeeded.
int leone_cache_commit(void* h, long long rid, long long new_len) {
  Manager* m = static_cast<Manager*>(h);
  Request* rc = m->find(rid);
  if (!rc) return unknown(rid);
  if (new_len > rc->reserved || new_len < rc->committed)
    return fail(kRuleBroken, "request " + std::to_string(rid) + ": commit to " + std::to_string(new_len) +
                                 " outside what was reserved");
  rc->committed = new_len;
  rc->fresh = false;
  for (Group& g : m->groups) {
    if (g.kind != 1) continue;
    std::vector<int>& table = g.tables[rid];
    const long long live_from = std::min(g.first_live_block(new_len), (long long)table.size());
    bool any = false;
    for (long long b = 0; b < live_from; ++b)
      if (table[b] >= 0) {
        const int r = g.pool.give_back(table[b], "page");
        if (r != kOk) return r;
        table[b] = -1;
        any = true;
      }
    if (any) rc->version = ++m->versions;
  }
  return kOk;
}

// Several requests at once, for the decode loop (one call a step instead of one a request).
// reserve_steps: pages for `steps` more tokens of every request, all or nothing; then, for each
// request, its committed length, its table version, its slot, and per group the length of its
// block table after the reservation (table_lens[g * n + i]).
int leone_cache_reserve_steps(void* h, int n, const long long* rids, long long steps, long long* lengths,
                              long long* versions, int* slots, int* table_lens) {
  Manager* m = static_cast<Manager*>(h);
  if (steps < 0) return fail(kBadArgument, "a negative number of steps");
  std::vector<long long> want(n);
  for (int i = 0; i < n; ++i) {
    Request* rc = m->find(rids[i]);
    if (!rc) return unknown(rids[i]);
    lengths[i] = rc->committed;
    want[i] = rc->committed + steps;
  }
  const int r = leone_cache_reserve(h, n, rids, want.data());
  if (r != kOk) return r;
  for (int i = 0; i < n; ++i) {
    const Request* rc = m->find(rids[i]);
    versions[i] = rc->version;
    slots[i] = rc->slot;
    for (size_t g = 0; g < m->groups.size(); ++g)
      table_lens[g * n + i] = (int)m->groups[g].tables[rids[i]].size();
  }
  return kOk;
}
int leone_cache_commit_many(void* h, int n, const long long* rids, const long long* new_lens) {
  for (int i = 0; i < n; ++i) {
    const int r = leone_cache_commit(h, rids[i], new_lens[i]);
    if (r != kOk) return r;
  }
  return kOk;
}

// Drop everything past `length` tokens (crates/leone/src/kv.rs:929-950); length < 0: roll
// back to the committed length (the step failed).
int leone_cache_truncate(void* h, long long rid, long long length) {
  Manager* m = static_cast<Manager*>(h);
  Request* rc = m->find(rid);
  if (!rc) return unknown(rid);
  if (length < 0) length = rc->committed;
  if (length > rc->committed)
    return fail(kRuleBroken, "request " + std::to_string(rid) + ": cannot truncate to " + std::to_string(length) +
                                 " past its length");
  // A window group has given back the pages that queries past the committed length cannot
  // see.  A query at a shorter length sees further back: if those pages are gone the rewind
  // cannot be served from the cache (the tokens would have to be computed again), so it is
  // refused before anything changes.
  for (Group& g : m->groups) {
    if (g.kind != 1) continue;
    const std::vector<int>& table = g.tables[rid];
    const long long keep = std::min<long long>(g.blocks_for(length), (long long)table.size());
    for (long long b = g.first_live_block(length); b < keep; ++b)
      if (table[b] < 0)
        return fail(kRuleBroken, "request " + std::to_string(rid) + ": cannot truncate to " + std::to_string(length) +
                                     ": its window has released block " + std::to_string(b) +
                                     ", which a query at that length reads");
  }
  for (Group& g : m->groups) {
    std::vector<int>& table = g.tables[rid];
    const size_t keep = (size_t)g.blocks_for(length);
    if (table.size() > keep) {
      for (size_t b = keep; b < table.size(); ++b)
        if (table[b] >= 0) {
          const int r = g.pool.give_back(table[b], "page");
          if (r != kOk) return r;
        }
      table.resize(keep);
      rc->version = ++m->versions;
    }
  }
  rc->committed = length;
  rc->reserved = length;
  return kOk;
}

// ---- views for the step function -------------------------------------------------------------
int leone_cache_table_len(void* h, int gid, long long rid) {
  Manager* m = static_cast<Manager*>(h);
  if (gid < 0 || gid >= (int)m->groups.size()) return fail(kBadArgument, "no such group");
  auto it = m->groups[gid].tables.find(rid);
  return it == m->groups[gid].tables.end() ? -1 : (int)it->second.size();
}
// Entries [from, from + count) of a request's block table.
int leone_cache_table_copy(void* h, int gid, long long rid, int from, int count, int* out) {
  Manager* m = static_cast<Manager*>(h);
  if (gid < 0 || gid >= (int)m->groups.size()) return fail(kBadArgument, "no such group");
  auto it = m->groups[gid].tables.find(rid);
  if (it == m->groups[gid].tables.end()) return unknown(rid);
  if (from < 0 || count < 0 || (size_t)(from + count) > it->second.size()) return fail(kBadArgument, "table range");
  std::copy(it->second.begin() + from, it->second.begin() + from + count, out);
  return kOk;
}
// The block tables of n requests as rows of `width` entries, -1 where there is no page.
int leone_cache_block_table(void* h, int gid, int n, const long long* rids, int width, int* out) {
  Manager* m = static_cast<Manager*>(h);
  if (gid < 0 || gid >= (int)m->groups.size()) return fail(kBadArgument, "no such group");
  Group& g = m->groups[gid];
  for (int i = 0; i < n; ++i) {
    auto it = g.tables.find(rids[i]);
    if (it == g.tables.end()) return unknown(rids[i]);
    if ((int)it->second.size() > width)
      return fail(kRuleBroken, "block table needs " + std::to_string(it->second.size()) + " columns, only " +
                                   std::to_string(width) + " given");
    int* row = out + (size_t)i * width;
    std::copy(it->second.begin(), it->second.end(), row);
    std::fill(row + it->second.size(), row + width, -1);
  }
  return kOk;
}

// ---- accounting ------------------------------------------------------------------------------
// what: 0 pages in the pool, 1 free, 2 held, 3 most ever held
int leone_cache_pool(void* h, int gid, int what) {
  Manager* m = static_cast<Manager*>(h);
  if (gid < 0 || gid >= (int)m->groups.size()) return fail(kBadArgument, "no such group");
  const FreeList& p = m->groups[gid].pool;
  return what == 0 ? p.n : what == 1 ? p.num_free() : what == 2 ? p.num_held() : p.high_water;
}
int leone_cache_slots(void* h, int what) {
  const FreeList& s = static_cast<Manager*>(h)->slots;
  return what == 0 ? s.n : s.num_free();
}
long long leone_cache_first_live_block(void* h, int gid, long long committed) {
  return static_cast<Manager*>(h)->groups[gid].first_live_block(committed);
}

// Every page is either free or in exactly one table; counts add up.
int leone_cache_check_invariants(void* h) {
  Manager* m = static_cast<Manager*>(h);
  for (size_t gi = 0; gi < m->groups.size(); ++gi) {
    Group& g = m->groups[gi];
    std::unordered_map<int, long long> seen;
    for (auto& kv : g.tables)
      for (int p : kv.second) {
        if (p < 0) continue;
        auto ins = seen.emplace(p, kv.first);
        if (!ins.second)
          return fail(kRuleBroken, "group " + std::to_string(gi) + ": page " + std::to_string(p) + " held by " +
                                       std::to_string(ins.first->second) + " and " + std::to_string(kv.first));
      }
    std::unordered_set<int> free_set(g.pool.free_.begin(), g.pool.free_.end());
    if (free_set.size() != g.pool.free_.size())
      return fail(kRuleBroken, "group " + std::to_string(gi) + ": a page is on the free list twice");
    for (auto& kv : seen)
      if (free_set.count(kv.first))
        return fail(kRuleBroken, "group " + std::to_string(gi) + ": a held page is on the free list");
    if ((int)(free_set.size() + seen.size()) != g.pool.n)
      return fail(kRuleBroken, "group " + std::to_string(gi) + ": " +
                                   std::to_string(g.pool.n - (int)free_set.size() - (int)seen.size()) + " pages lost");
  }
  std::unordered_set<int> held;
  for (auto& kv : m->requests)
    if (!held.insert(kv.second.slot).second) return fail(kRuleBroken, "a state slot is held twice");
  if ((int)held.size() + m->slots.num_free() != m->slots.n) return fail(kRuleBroken, "a state slot was lost");
  return kOk;
}

// ---- a step's metadata -------------------------------------------------------------------------
// Lays a step out as one int32 array: token_ids[N] positions[N] seq_of_token[N] q_start[B+1]
// ctx_len[B] slot_ids[B] logit_rows[M], then the groups' block tables.  Sequence i brings
// counts[i] tokens (taken in order from `tokens`) starting at position starts[i] and wants the
// logits at the places wants[want_start[i] .. want_start[i+1]) among them.  `out` must hold
// leone_pack_step_size words.  Returns 0, or 2 with a message if a wanted place is outside
// its sequence's tokens.  (positions: crates/leone/src/cpu.rs:1759-1765, prefill position =
// start + t.)
long long leone_pack_step_size(int b, long long n_tokens, long long n_wanted, long long table_words) {
  return 3 * n_tokens + (b + 1) + 2 * (long long)b + n_wanted + table_words;
}
int leone_pack_step(int b, const long long* counts, const long long* tokens, const long long* starts,
                    const long long* slots, const long long* want_start, const long long* wants, int* out) {
  long long n = 0;
  for (int i = 0; i < b; ++i) n += counts[i];
  const long long m = want_start[b];
  int* token_ids = out;
  int* positions = out + n;
  int* seq_of_token = out + 2 * n;
  int* q_start = out + 3 * n;
  int* ctx_len = q_start + (b + 1);
  int* slot_ids = ctx_len + b;
  int* logit_rows = slot_ids + b;
  long long at = 0;
  for (int i = 0; i < b; ++i) {
    q_start[i] = (int)at;
    for (long long t = 0; t < counts[i]; ++t, ++at) {
      token_ids[at] = (int)tokens[at];
      positions[at] = (int)(starts[i] + t);
      seq_of_token[at] = i;
    }
    ctx_len[i] = (int)(starts[i] + counts[i]);
    slot_ids[i] = (int)slots[i];
    for (long long w = want_start[i]; w < want_start[i + 1]; ++w) {
      if (wants[w] < 0 || wants[w] >= counts[i])
        return fail(kRuleBroken, "entry " + std::to_string(i) + ": wanted place " + std::to_string(wants[w]) +
                                     " is outside its " + std::to_string(counts[i]) + " tokens");
      logit_rows[w] = q_start[i] + (int)wants[w];
    }
  }
  q_start[b] = (int)at;
  (void)m;
  return kOk;
}


// ---- the scheduler's decisions -----------------------------------------------------------------
// Which requests run, what the next step holds, when a request ends, whom to preempt.  The
// planner keeps counts only (how many tokens a request has, how many are in the cache, how many
// it has generated); the Python front keeps the token ids and does what the planner decides
// (opens and closes requests in the engine, runs the step, samples).  It reads the cache
// manager it was made over for free pages and slots and never changes it.
//
// One step's batch: one token for every decoding request, then portions of prompts in arrival
// order until the token budget is used (max_batch_tokens for the step, prefill_chunk for a
// request); with prefill_first decode rows are held back while any running request has prompt
// left.  The reference dispatches per request with a budget of min(remaining_prefill,
// prefill_chunk_tokens) or a decode quantum (crates/leone/src/scheduler.rs:341-378).
// Page policies: 0 "reserve": admitted only if ceil((prompt + max_new - 1) / page_tokens) pages
// can be set aside for its whole life (crates/leone/src/scheduler.rs:652-667); 1 "optimistic":
// admitted when its first portion fits, the youngest running request is preempted when a step
// cannot get its pages.  max_new counts the token sampled from the prompt, so N new tokens need
// the cache for P + N - 1 positions (crates/leone/src/runtime.rs:3602-3607).
namespace {

enum SchedState { kWaiting = 0, kRunning = 1, kFinished = 2, kCancelled = 3 };
enum Reject { kDuplicate = 1, kEmptyPrompt, kOutputLimit, kTokenId, kPromptLimit, kKvCapacity, kQueueLimit };
enum Finish { kNotFinished = 0, kEos = 1, kLength = 2, kMaxPositions = 3 };

struct SchedRequest {
  long long n_tokens = 0;       // prompt + generated: what the cache must come to hold
  long long computed = 0;       // tokens already in the cache
  long long generated = 0;
  long long max_new = 0;
  long long arrival = 0;
  long long reserved_pages = 0;  // the largest of `needs` (what a caller is shown)
  std::vector<long long> needs;  // pages set aside per cache group under the reserve policy
  long long preemptions = 0;
  int state = kWaiting;
  bool cancel = false;
  bool decoding() const { return generated > 0 && computed == n_tokens - 1; }
};

struct Planner {
  Manager* cache;
  long long max_running, max_waiting, max_batch_tokens, prefill_chunk;
  int policy, prefill_first;
  long long vocab, max_positions;
  long long decode_quantum = 1;  // most decode steps reserved in one call
  std::vector<long long> reserved_by_group;
  std::deque<long long> waiting;
  std::vector<long long> running;
  std::unordered_map<long long, SchedRequest> requests;
  long long arrivals = 0, reserved_total = 0;
  long long admitted = 0, finished = 0, cancelled = 0, preemptions = 0;

  bool has_groups() const { return cache != nullptr && !cache->groups.empty(); }
  // The most tokens one request brings to a step: a prompt portion, or a decode quantum.
  long long step_tokens() const { return std::max(std::min(prefill_chunk, max_batch_tokens), decode_quantum); }
  // The most pages one request holds at a time in group g when it comes to hold `total` tokens.
  // A full group keeps every page.  A window group holds, during a step from length c to
  // c + portion, the blocks from first_live_block(c) to blocks_for(c + portion); past the
  // window that count depends on c only through c mod page_tokens.
  long long group_need(const Group& g, long long total) const {
    const long long all = g.blocks_for(total);
    if (g.kind != 1) return all;
    long long most = 0;
    for (long long c = g.window; c < g.window + g.page_tokens; ++c)
      most = std::max(most, g.blocks_for(c + step_tokens()) - g.first_live_block(c));
    return std::min(all, most);
  }
  // Per group, the request's need; false if some group's pool is too small even when empty.
  bool fits_empty_pool(long long total, std::string* why) const {
    for (size_t i = 0; i < cache->groups.size(); ++i) {
      const Group& g = cache->groups[i];
      if (group_need(g, total) > g.pool.n) {
        *why = "the request needs " + std::to_string(group_need(g, total)) + " pages; the pool has " +
               std::to_string(g.pool.n) + " even when empty";
        return false;
      }
    }
    return true;
  }
  SchedRequest* find(long long rid) {
    auto it = requests.find(rid);
    return it == requests.end() ? nullptr : &it->second;
  }
  void leave_running(long long rid) { running.erase(std::find(running.begin(), running.end(), rid)); }
  void retire(long long rid, SchedRequest* r, bool was_cancelled) {
    leave_running(rid);
    reserved_total -= r->reserved_pages;
    r->reserved_pages = 0;
    for (size_t i = 0; i < r->needs.size() && i < reserved_by_group.size(); ++i) reserved_by_group[i] -= r->needs[i];
    r->needs.clear();
    r->state = was_cancelled ? kCancelled : kFinished;
    ++(was_cancelled ? cancelled : finished);
  }
};

}  // namespace

void* leone_sched_create(void* cache, long long max_running, long long max_waiting, long long max_batch_tokens,
                         long long prefill_chunk, int policy, int prefill_first, long long vocab,
                         long long max_positions) {
  if (max_running <= 0 || max_batch_tokens <= 0 || prefill_chunk <= 0 || policy < 0 || policy > 1) return nullptr;
  Planner* p = new Planner();
  p->cache = static_cast<Manager*>(cache);
  p->max_running = max_running;
  p->max_waiting = max_waiting;
  p->max_batch_tokens = max_batch_tokens;
  p->prefill_chunk = prefill_chunk;
  p->policy = policy;
  p->prefill_first = prefill_first;
  p->vocab = vocab;
  p->max_positions = max_positions;
  return p;
}
// The most decode steps the caller will reserve in one call (a window group's worst case counts it).
void leone_sched_set_decode_quantum(void* h, long long quantum) {
  static_cast<Planner*>(h)->decode_quantum = std::max(1ll, quantum);
}
void leone_sched_destroy(void* h) { delete static_cast<Planner*>(h); }

// A new request joins the queue.  Returns 0, or why it can never run (a Reject code; the
// reference's AdmissionReject, crates/leone/src/scheduler.rs:101-110) with a message.
int leone_sched_add(void* h, long long rid, const long long* prompt, long long n, long long max_new) {
  Planner* p = static_cast<Planner*>(h);
  SchedRequest* old = p->find(rid);
  if (old != nullptr && (old->state == kWaiting || old->state == kRunning))
    return fail((Code)kDuplicate, "request id is already in flight");
  if (n <= 0) return fail((Code)kEmptyPrompt, "a request needs at least one prompt token");
  if (max_new <= 0) return fail((Code)kOutputLimit, "max_new_tokens must be positive");
  std::string bad;
  int n_bad = 0;
  for (long long i = 0; i < n && n_bad < 8; ++i)
    if (prompt[i] < 0 || prompt[i] >= p->vocab) bad += (n_bad++ ? ", " : "") + std::to_string(prompt[i]);
  if (n_bad)
    return fail((Code)kTokenId, "token ids [" + bad + "] are outside the vocabulary of " + std::to_string(p->vocab));
  const long long need_positions = n + max_new - 1;
  if (need_positions > p->max_positions)
    return fail((Code)kPromptLimit, "prompt (" + std::to_string(n) + ") + max_new_tokens (" + std::to_string(max_new) +
                                        ") - 1 exceeds the model's " + std::to_string(p->max_positions) + " positions");
  std::string why;
  if (p->has_groups() && !p->fits_empty_pool(need_positions, &why)) return fail((Code)kKvCapacity, why);
  if ((long long)p->waiting.size() >= p->max_waiting)
    return fail((Code)kQueueLimit, std::to_string(p->max_waiting) + " requests are already waiting");
  SchedRequest r;
  r.n_tokens = n;
  r.max_new = max_new;
  r.arrival = p->arrivals++;
  p->requests[rid] = r;
  p->waiting.push_back(rid);
  return kOk;
}

// Queued: leaves at once (returns 1).  Running: marked, leaves at the next step boundary
// (returns 2; crates/leone/src/scheduler.rs:540-554).  Otherwise 0.
int leone_sched_cancel(void* h, long long rid) {
  Planner* p = static_cast<Planner*>(h);
  SchedRequest* r = p->find(rid);
  if (r == nullptr || r->state == kFinished || r->state == kCancelled) return 0;
  if (r->state == kWaiting) {
    p->waiting.erase(std::find(p->waiting.begin(), p->waiting.end(), rid));
    r->state = kCancelled;
    ++p->cancelled;
    return 1;
  }
  r->cancel = true;
  return 2;
}

// The running requests that were cancelled leave; the caller closes them.  Returns how many.
int leone_sched_drop_cancelled(void* h, long long* out, int cap) {
  Planner* p = static_cast<Planner*>(h);
  int n = 0;
  const std::vector<long long> now = p->running;
  for (long long rid : now) {
    SchedRequest* r = p->find(rid);
    if (r->cancel && n < cap) {
      p->retire(rid, r, true);
      out[n++] = rid;
    }
  }
  return n;
}

// Moves requests from the queue to running, in arrival order, while they fit.  The caller
// opens them (each takes a state slot, which this call counts ahead).  Returns how many.
int leone_sched_admit(void* h, long long* out, int cap) {
  Planner* p = static_cast<Planner*>(h);
  int n = 0;
  long long slots_free = p->cache != nullptr ? p->cache->slots.num_free() : (1ll << 30);
  while (!p->waiting.empty() && (long long)p->running.size() < p->max_running && n < cap) {
    const long long rid = p->waiting.front();
    SchedRequest* r = p->find(rid);
    if (slots_free == 0) break;
    if (p->policy == 0) {
      // every group must be able to set aside what the request holds there at its largest
      // (crates/leone/src/scheduler.rs:652-667 reserves prompt + output, rounded up to pages)
      const long long total = r->n_tokens + (r->max_new - r->generated) - 1;
      std::vector<long long> needs;
      bool fits = true;
      if (p->has_groups()) {
        p->reserved_by_group.resize(p->cache->groups.size(), 0);
        for (size_t i = 0; i < p->cache->groups.size(); ++i) {
          needs.push_back(p->group_need(p->cache->groups[i], total));
          fits = fits && p->reserved_by_group[i] + needs[i] <= p->cache->groups[i].pool.n;
        }
      }
      if (!fits) break;
      r->reserved_pages = 0;
      for (size_t i = 0; i < needs.size(); ++i) {
        p->reserved_by_group[i] += needs[i];
        r->reserved_pages = std::max(r->reserved_pages, needs[i]);
      }
      r->needs = needs;
      p->reserved_total += r->reserved_pages;
    } else {
      // the first portion must fit every group's free pages (nothing is released before a commit)
      const long long first = std::min(r->n_tokens, p->prefill_chunk);
      bool fits = true;
      if (!p->running.empty() && p->has_groups())
        for (const Group& g : p->cache->groups) fits = fits && g.blocks_for(first) <= g.pool.num_free();
      if (!fits) break;
    }
    p->waiting.pop_front();
    r->state = kRunning;
    r->computed = 0;
    p->running.push_back(rid);
    ++p->admitted;
    --slots_free;
    out[n++] = rid;
  }
  return n;
}

// The next step's entries: request, index of its first token, count.  Returns how many.
int leone_sched_plan(void* h, long long* rids, long long* starts, long long* counts, int cap) {
  Planner* p = static_cast<Planner*>(h);
  long long budget = p->max_batch_tokens;
  int n = 0;
  bool hold_decodes = false;
  if (p->prefill_first)
    for (long long rid : p->running) hold_decodes = hold_decodes || !p->find(rid)->decoding();
  if (!hold_decodes)
    for (long long rid : p->running) {              // decode rows first
      const SchedRequest* r = p->find(rid);
      if (r->decoding() && budget > 0 && n < cap) {
        rids[n] = rid, starts[n] = r->computed, counts[n] = 1;
        ++n, --budget;
      }
    }
  for (long long rid : p->running) {                // then prompt portions, oldest first
    if (budget <= 0 || n >= cap) break;
    const SchedRequest* r = p->find(rid);
    const long long left = r->n_tokens - r->computed;
    if (left >= 1 && !(left == 1 && r->generated > 0)) {
      const long long count = std::min(std::min(left, p->prefill_chunk), budget);
      rids[n] = rid, starts[n] = r->computed, counts[n] = count;
      ++n, budget -= count;
    }
  }
  return n;
}

// `count` more of the request's tokens are in the cache.
int leone_sched_computed(void* h, long long rid, long long count) {
  Planner* p = static_cast<Planner*>(h);
  SchedRequest* r = p->find(rid);
  if (r == nullptr || r->state != kRunning) return fail(kRuleBroken, "request " + std::to_string(rid) + " is not running");
  if (count < 0 || r->computed + count > r->n_tokens)
    return fail(kRuleBroken, "request " + std::to_string(rid) + ": more tokens computed than it has");
  r->computed += count;
  return kOk;
}

// The request emitted a token.  Returns why it ends now (a Finish code; it has then left the
// running list and the caller closes it) or 0.  Finished when eos or no tokens remain
// (crates/leone/src/scheduler.rs:1341-1343).
int leone_sched_emitted(void* h, long long rid, int is_eos) {
  Planner* p = static_cast<Planner*>(h);
  SchedRequest* r = p->find(rid);
  if (r == nullptr || r->state != kRunning) return -1;
  ++r->generated;
  ++r->n_tokens;
  int reason = kNotFinished;
  if (is_eos) reason = kEos;
  else if (r->generated >= r->max_new) reason = kLength;
  else if (r->n_tokens > p->max_positions) reason = kMaxPositions;
  if (reason != kNotFinished) p->retire(rid, r, false);
  return reason;
}

// One decode step's tokens for n running requests: each has one more token in the cache and has
// emitted one (is_eos[i]: it was the request's stop token).  reasons[i] as leone_sched_emitted.
int leone_sched_decoded(void* h, int n, const long long* rids, const int* is_eos, int* reasons) {
  for (int i = 0; i < n; ++i) {
    const int r = leone_sched_computed(h, rids[i], 1);
    if (r != kOk) return r;
    reasons[i] = leone_sched_emitted(h, rids[i], is_eos[i]);
  }
  return kOk;
}

// A finished or cancelled request is forgotten (its id may be used again).  Returns 1 if it was
// known and is gone now, 0 otherwise (unknown, or still waiting or running).
int leone_sched_forget(void* h, long long rid) {
  Planner* p = static_cast<Planner*>(h);
  SchedRequest* r = p->find(rid);
  if (r == nullptr || r->state == kWaiting || r->state == kRunning) return 0;
  p->requests.erase(rid);
  return 1;
}

// The youngest running request other than `keep` (-1: none kept) goes back to the front of the
// queue, to be recomputed from its first token; the caller closes it.  Returns 1 and the
// victim, or 0 if nobody can be preempted.
int leone_sched_preempt_youngest(void* h, long long keep, long long* victim) {
  Planner* p = static_cast<Planner*>(h);
  long long best = -1, best_arrival = -1;
  for (long long rid : p->running) {
    if (rid == keep) continue;
    const SchedRequest* r = p->find(rid);
    if (r->arrival > best_arrival) best = rid, best_arrival = r->arrival;
  }
  if (best < 0) return 0;
  SchedRequest* r = p->find(best);
  p->leave_running(best);
  r->state = kWaiting;
  r->computed = 0;
  ++r->preemptions;
  ++p->preemptions;
  p->waiting.push_front(best);
  *victim = best;
  return 1;
}

// The running request that arrived first, or -1.
long long leone_sched_oldest_running(void* h) {
  Planner* p = static_cast<Planner*>(h);
  long long best = -1, best_arrival = 1ll << 62;
  for (long long rid : p->running) {
    const SchedRequest* r = p->find(rid);
    if (r->arrival < best_arrival) best = rid, best_arrival = r->arrival;
  }
  return best;
}

// How many decode steps these requests can take together without the host: at most `quantum`,
// what each may still emit, and what the model's positions leave.
long long leone_sched_decode_quantum(void* h, int n, const long long* rids, long long quantum) {
  Planner* p = static_cast<Planner*>(h);
  long long q = quantum;
  for (int i = 0; i < n; ++i) {
    const SchedRequest* r = p->find(rids[i]);
    if (r == nullptr) continue;
    q = std::min(q, r->max_new - r->generated);
    q = std::min(q, p->max_positions - r->n_tokens + 1);
  }
  return std::max(1ll, q);
}

// what: 0 tokens, 1 computed, 2 generated, 3 state, 4 reserved pages, 5 preemptions, 6 arrival,
// 7 cancel requested.  -1 for an unknown request.
long long leone_sched_get(void* h, long long rid, int what) {
  const SchedRequest* r = static_cast<Planner*>(h)->find(rid);
  if (r == nullptr) return -1;
  switch (what) {
    case 0: return r->n_tokens;
    case 1: return r->computed;
    case 2: return r->generated;
    case 3: return r->state;
    case 4: return r->reserved_pages;
    case 5: return r->preemptions;
    case 6: return r->arrival;
    case 7: return r->cancel ? 1 : 0;
  }
  return -1;
}

// what: 0 waiting, 1 running, 2 admitted, 3 finished, 4 cancelled, 5 preemptions, 6 pages set aside.
long long leone_sched_count(void* h, int what) {
  const Planner* p = static_cast<Planner*>(h);
  switch (what) {
    case 0: return (long long)p->waiting.size();
    case 1: return (long long)p->running.size();
    case 2: return p->admitted;
    case 3: return p->finished;
    case 4: return p->cancelled;
    case 5: return p->preemptions;
    case 6: return p->reserved_total;
  }
  return -1;
}

// The queue (which 0) or the running list (which 1), in order.  Returns how many.
int leone_sched_list(void* h, int which, long long* out, int cap) {
  const Planner* p = static_cast<Planner*>(h);
  int n = 0;
  if (which == 0) {
    for (long long rid : p->waiting)
      if (n < cap) out[n++] = rid;
  } else {
    for (long long rid : p->running)
      if (n < cap) out[n++] = rid;
  }
  return n;
}

}  // extern "C"
