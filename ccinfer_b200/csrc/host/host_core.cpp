// Host core of ccinfer_b200: cache manager, request slots and the arrays of a step, behind the C interface of
// ccinfer.h.
//
// The decisions are those of 7QiC/ccInfer where it has them: pages of a fixed number of tokens with a FIFO free
// list (src/cache/kv_cache_manager.cpp:78-82, 242-244), pages taken on demand just before a step
// (src/worker/batch_translator.cpp:196-211), everything of a sequence given back when it ends
// (src/worker/worker.cpp:317-326), validate-then-mutate release with double-free detection
// (src/cache/kv_cache_manager.cpp:216-230), and a transactional step: what a failed step took is returned
// (src/worker/batch_translator.cpp:72-75, 579-589).  Beyond the reference: cache groups (layers that read all
// keys, or a window of them, each group with a pool and block tables of its own; a window group gives pages
// back while a sequence runs), state slots, and ONE buffer at fixed offsets for all arrays of a step instead of
// seven fresh device allocations (src/worker/batch_translator.cpp:241-431), so that a step is one or two
// copies and a decode step can be replayed from a CUDA graph.  No prefix sharing, reference counts or LRU:
// a page has exactly one owner.
#include "ccinfer.h"

#include <algorithm>
#include <cstring>
#include <deque>
#include <map>
#include <string>
#include <unordered_map>
#include <unordered_set>
#include <utility>
#include <vector>

namespace {

struct Failure {
  int code;
  std::string message;
};

[[noreturn]] void fail(int code, std::string message) { throw Failure{code, std::move(message)}; }

std::string str(long long v) { return std::to_string(v); }

// ---------------------------------------------------------------------------------------------
// pools
// ---------------------------------------------------------------------------------------------
constexpr int64_t kNoOwner = INT64_MIN;

class PagePool {
 public:
  explicit PagePool(int num_pages) : num_pages_(num_pages), owner_(num_pages > 0 ? num_pages : 0, kNoOwner) {
    if (num_pages <= 0) fail(CCINFER_INVALID_ARGUMENT, "a page pool needs at least one page");
    for (int p = 0; p < num_pages; ++p) free_.push_back(p);
  }
  int num_pages() const { return num_pages_; }
  int free_pages() const { return (int)free_.size(); }
  int used_pages() const { return num_pages_ - (int)free_.size(); }
  int high_water() const { return high_water_; }
  const std::deque<int>& free_list() const { return free_; }
  int64_t owner_of(int page) const { return owner_[page]; }

  void take(int64_t owner, int n, int* out) {
    if (n < 0) fail(CCINFER_INVALID_ARGUMENT, "cannot take a negative number of pages");
    if (owner == kNoOwner) fail(CCINFER_INVALID_ARGUMENT, "this owner id is reserved");
    if (n > (int)free_.size())
      fail(CCINFER_KV_BLOCK_EXHAUSTED, str(n) + " pages wanted, " + str(free_.size()) + " free of " + str(num_pages_));
    for (int i = 0; i < n; ++i) {
      const int p = free_.front();
      free_.pop_front();
      owner_[p] = owner;
      out[i] = p;
    }
    high_water_ = std::max(high_water_, used_pages());
  }

  // all or nothing: every page is checked before any is freed
  void give_back(int64_t owner, const int* pages, int n) {
    std::unordered_set<int> seen;
    for (int i = 0; i < n; ++i) {
      const int p = pages[i];
      if (p < 0 || p >= num_pages_)
        fail(CCINFER_KV_INVALID_BLOCK_TABLE, "page id " + str(p) + " is outside the pool of " + str(num_pages_));
      if (!seen.insert(p).second) fail(CCINFER_KV_BLOCK_DOUBLE_FREE, "page " + str(p) + " is named twice in one release");
      if (owner_[p] == kNoOwner) fail(CCINFER_KV_BLOCK_DOUBLE_FREE, "page " + str(p) + " is already free");
      if (owner_[p] != owner)
        fail(CCINFER_KV_INVALID_BLOCK_TABLE, "page " + str(p) + " belongs to another owner (" + str(owner_[p]) + ")");
    }
    for (int i = 0; i < n; ++i) {
      owner_[pages[i]] = kNoOwner;
      free_.push_back(pages[i]);
    }
  }

 private:
  int num_pages_;
  std::deque<int> free_;
  std::vector<int64_t> owner_;
  int high_water_ = 0;
};

class SlotPool {
 public:
  explicit SlotPool(int n) : used_(n > 0 ? n : 0, false) {
    if (n <= 0) fail(CCINFER_INVALID_ARGUMENT, "at least one state slot is needed");
    for (int s = 0; s < n; ++s) free_.push_back(s);
  }
  int num_slots() const { return (int)used_.size(); }
  int free_slots() const { return (int)free_.size(); }
  int take() {
    if (free_.empty()) fail(CCINFER_SEQUENCE_LIMIT_REACHED, "all " + str(used_.size()) + " request slots are in use");
    const int s = free_.front();
    free_.pop_front();
    used_[s] = true;
    return s;
  }
  void give_back(int slot) {
    if (slot < 0 || slot >= (int)used_.size())
      fail(CCINFER_INVALID_ARGUMENT, "slot " + str(slot) + " is outside the pool of " + str(used_.size()));
    if (!used_[slot]) fail(CCINFER_KV_BLOCK_DOUBLE_FREE, "slot " + str(slot) + " is already free");
    used_[slot] = false;
    free_.push_back(slot);
  }

 private:
  std::deque<int> free_;
  std::vector<bool> used_;
};

// ---------------------------------------------------------------------------------------------
// sequences
// ---------------------------------------------------------------------------------------------
struct Sequence {
  int64_t id = 0;
  int slot = -1;
  int ctx_len = 0;
  std::vector<std::vector<int>> tables;   // per group: logical page -> physical page, -1 = none / given back
  std::vector<int> taken;                 // per group: pages appended by the reservation that is not committed yet
  int reserved_tokens = 0;
};

struct Layout {
  ccinfer_layout c{};
  static Layout make(int cap_tokens, int cap_entries, int n_groups, int stride) {
    Layout l;
    int off = 0;
    auto region = [&off](int n) {
      const int start = off;
      off += (n + 3) / 4 * 4;   // every region starts on a 16-byte boundary
      return start;
    };
    l.c.capacity_tokens = cap_tokens;
    l.c.capacity_entries = cap_entries;
    l.c.token_ids = region(cap_tokens);
    l.c.positions = region(cap_tokens);
    l.c.entry_of_token = region(cap_tokens);
    l.c.logit_rows = region(cap_tokens);
    l.c.row_slot = region(cap_tokens);
    l.c.cu_q = region(cap_entries + 1);
    l.c.pos0 = region(cap_entries);
    l.c.ctx_after = region(cap_entries);
    l.c.state_slot = region(cap_entries);
    l.c.n_groups = n_groups;
    l.c.block_table_stride = stride;
    for (int g = 0; g < n_groups; ++g) l.c.slot_map[g] = region(cap_tokens);
    // block tables last: the rows in use are a prefix of each, so a step copies [0, first table) and a prefix
    // of every table, not the whole buffer
    for (int g = 0; g < n_groups; ++g) l.c.block_table[g] = region(cap_entries * stride);
    l.c.size_words = off;
    return l;
  }
};

}  // namespace

struct ccinfer_engine {
  std::vector<ccinfer_group> groups;
  std::vector<PagePool> pools;
  SlotPool slots;
  std::unordered_map<int64_t, Sequence> seqs;
  int max_seqs, max_tokens, max_context;
  Layout small, large;
  ccinfer_runner runner = nullptr;
  void* runner_user = nullptr;
  long long steps = 0;
  mutable std::string last_error;
  // per step buffer (by address) and group: how many block-table entries each row held when it was last written
  std::map<const void*, std::vector<std::vector<int>>> row_len;
  std::vector<int> order_scratch;

  ccinfer_engine(const ccinfer_options& o) : slots(o.max_seqs), max_seqs(o.max_seqs), max_tokens(o.max_tokens_per_step),
                                             max_context(o.max_context) {
    if (o.n_groups < 0 || o.n_groups > CCINFER_MAX_GROUPS)
      fail(CCINFER_INVALID_ARGUMENT, "0 to " + str(CCINFER_MAX_GROUPS) + " cache groups");
    if (o.max_tokens_per_step < o.max_seqs)
      fail(CCINFER_INVALID_ARGUMENT, "max_tokens_per_step (" + str(o.max_tokens_per_step) + ") is below max_seqs (" +
                                         str(o.max_seqs) + "): a step of one token per sequence must fit");
    if (o.max_context <= 0) fail(CCINFER_INVALID_ARGUMENT, "max_context must be > 0");
    int stride = 1;
    for (int g = 0; g < o.n_groups; ++g) {
      if (o.groups[g].page_size <= 0) fail(CCINFER_INVALID_ARGUMENT, "page_size must be > 0");
      groups.push_back(o.groups[g]);
      pools.emplace_back(o.groups[g].num_pages);
      stride = std::max(stride, (o.max_context + o.groups[g].page_size - 1) / o.groups[g].page_size);
    }
    small = Layout::make(o.max_seqs, o.max_seqs, o.n_groups, stride);
    large = Layout::make(o.max_tokens_per_step, o.max_seqs, o.n_groups, stride);
  }

  Sequence& seq(int64_t id) {
    auto it = seqs.find(id);
    if (it == seqs.end()) fail(CCINFER_INVALID_ARGUMENT, "sequence " + str(id) + " is not open");
    return it->second;
  }
  const Sequence& seq(int64_t id) const { return const_cast<ccinfer_engine*>(this)->seq(id); }

  int pages_needed(const Sequence& s, int g, int n_new) const {
    const int P = groups[g].page_size;
    return std::max(0, (s.ctx_len + n_new + P - 1) / P - (int)s.tables[g].size());
  }

  // logical index of the first page a query at position >= ctx_len can still read
  int first_needed_page(int g, int ctx_len) const {
    if (groups[g].window <= 0) return 0;
    return std::max(0, ctx_len - groups[g].window + 1) / groups[g].page_size;
  }

  void undo(Sequence& s) {
    for (size_t g = 0; g < groups.size(); ++g) {
      const int n = s.taken.empty() ? 0 : s.taken[g];
      if (n == 0) continue;
      auto& t = s.tables[g];
      pools[g].give_back(s.id, t.data() + (t.size() - n), n);   // they are the tail of the table
      t.resize(t.size() - n);
    }
    s.taken.assign(groups.size(), 0);
    s.reserved_tokens = 0;
  }

  void reserve(Sequence& s, int n_new) {
    if (n_new <= 0) fail(CCINFER_INVALID_ARGUMENT, "a step brings at least one token per sequence");
    if (s.reserved_tokens) fail(CCINFER_INVALID_ARGUMENT, "sequence " + str(s.id) + " has an uncommitted reservation");
    s.taken.assign(groups.size(), 0);
    std::vector<int> fresh;
    try {
      for (size_t g = 0; g < groups.size(); ++g) {
        const int n = pages_needed(s, (int)g, n_new);
        fresh.resize(n);
        pools[g].take(s.id, n, fresh.data());
        s.tables[g].insert(s.tables[g].end(), fresh.begin(), fresh.end());
        s.taken[g] = n;
      }
    } catch (const Failure&) {
      undo(s);   // either every group gets its pages or none keeps any
      throw;
    }
    s.reserved_tokens = n_new;
  }

  void commit(Sequence& s) {
    if (!s.reserved_tokens) fail(CCINFER_INVALID_ARGUMENT, "sequence " + str(s.id) + " has nothing reserved");
    s.ctx_len += s.reserved_tokens;
    s.reserved_tokens = 0;
    s.taken.assign(groups.size(), 0);
    std::vector<int> stale;
    for (size_t g = 0; g < groups.size(); ++g) {
      if (groups[g].window <= 0) continue;
      auto& t = s.tables[g];
      const int first = std::min(first_needed_page((int)g, s.ctx_len), (int)t.size());
      stale.clear();
      for (int i = 0; i < first; ++i)
        if (t[i] >= 0) stale.push_back(t[i]);
      if (stale.empty()) continue;
      pools[g].give_back(s.id, stale.data(), (int)stale.size());   // every later query has passed them
      for (int i = 0; i < first; ++i) t[i] = -1;
    }
  }
};

namespace {

thread_local std::string g_create_error;

template <typename F>
int guarded(const ccinfer_engine* e, F&& f) {
  try {
    f();
    return CCINFER_OK;
  } catch (const Failure& x) {
    if (e != nullptr) e->last_error = x.message;
    else g_create_error = x.message;
    return x.code;
  } catch (const std::exception& x) {
    if (e != nullptr) e->last_error = x.what();
    else g_create_error = x.what();
    return CCINFER_INVALID_STATE;
  }
}

void need(const void* p, const char* what) {
  if (p == nullptr) fail(CCINFER_INVALID_ARGUMENT, std::string(what) + " is null");
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// C interface
// ---------------------------------------------------------------------------------------------
extern "C" {

int ccinfer_create(const ccinfer_options* options, ccinfer_engine** out) {
  return guarded(nullptr, [&] {
    need(options, "options");
    need(out, "out");
    if (options->n_groups > 0) need(options->groups, "options.groups");
    *out = new ccinfer_engine(*options);
  });
}

void ccinfer_destroy(ccinfer_engine* e) { delete e; }

const char* ccinfer_last_error(const ccinfer_engine* e) { return e != nullptr ? e->last_error.c_str() : g_create_error.c_str(); }

int ccinfer_get_layout(const ccinfer_engine* e, int which, ccinfer_layout* out) {
  return guarded(e, [&] {
    need(e, "engine");
    need(out, "out");
    if (which != 0 && which != 1) fail(CCINFER_INVALID_ARGUMENT, "layout 0 (small) or 1 (large)");
    *out = which == 0 ? e->small.c : e->large.c;
  });
}

int ccinfer_stats(const ccinfer_engine* e, ccinfer_stats_t* out) {
  return guarded(e, [&] {
    need(e, "engine");
    need(out, "out");
    std::memset(out, 0, sizeof(*out));
    out->seqs = (int)e->seqs.size();
    out->slots_total = e->slots.num_slots();
    out->slots_free = e->slots.free_slots();
    out->n_groups = (int)e->groups.size();
    for (size_t g = 0; g < e->groups.size(); ++g) {
      out->pages_total[g] = e->pools[g].num_pages();
      out->pages_free[g] = e->pools[g].free_pages();
      out->pages_high_water[g] = e->pools[g].high_water();
    }
    out->steps = e->steps;
  });
}

int ccinfer_get_groups(const ccinfer_engine* e, ccinfer_group* out, int capacity, int* n) {
  return guarded(e, [&] {
    need(e, "engine");
    need(n, "n");
    *n = (int)e->groups.size();
    for (int g = 0; g < std::min(capacity, *n); ++g) {
      need(out, "out");
      out[g] = e->groups[g];
    }
  });
}

int ccinfer_check(const ccinfer_engine* e) {
  return guarded(e, [&] {
    need(e, "engine");
    for (size_t g = 0; g < e->groups.size(); ++g) {
      const PagePool& pool = e->pools[g];
      std::unordered_map<int, int64_t> held;
      for (const auto& kv : e->seqs)
        for (int p : kv.second.tables[g]) {
          if (p < 0) continue;
          if (p >= pool.num_pages()) fail(CCINFER_INVALID_STATE, "group " + str(g) + ": a table holds page " + str(p));
          if (!held.emplace(p, kv.first).second)
            fail(CCINFER_INVALID_STATE, "group " + str(g) + ": page " + str(p) + " is held twice");
        }
      std::unordered_set<int> free_set;
      for (int p : pool.free_list()) {
        if (!free_set.insert(p).second) fail(CCINFER_INVALID_STATE, "group " + str(g) + ": page " + str(p) + " is on the free list twice");
        if (held.count(p)) fail(CCINFER_INVALID_STATE, "group " + str(g) + ": page " + str(p) + " is both free and held");
      }
      // pages taken through ccinfer_pool_take directly have an owner and sit in no table
      int direct = 0;
      for (int p = 0; p < pool.num_pages(); ++p)
        if (pool.owner_of(p) != kNoOwner && !held.count(p)) {
          if (e->seqs.count(pool.owner_of(p))) fail(CCINFER_INVALID_STATE, "group " + str(g) + ": page " + str(p) + " is lost");
          ++direct;
        }
      if ((int)free_set.size() + (int)held.size() + direct != pool.num_pages())
        fail(CCINFER_INVALID_STATE, "group " + str(g) + ": pages lost");
      for (const auto& kv : held)
        if (pool.owner_of(kv.first) != kv.second)
          fail(CCINFER_INVALID_STATE, "group " + str(g) + ": page " + str(kv.first) + " owner mismatch");
    }
  });
}

int ccinfer_alloc_seq(ccinfer_engine* e, int64_t id, int* slot) {
  return guarded(e, [&] {
    need(e, "engine");
    if (id == kNoOwner) fail(CCINFER_INVALID_ARGUMENT, "this sequence id is reserved");
    if (e->seqs.count(id)) fail(CCINFER_INVALID_ARGUMENT, "sequence " + str(id) + " is already open");
    Sequence s;
    s.id = id;
    s.slot = e->slots.take();
    s.tables.resize(e->groups.size());
    s.taken.assign(e->groups.size(), 0);
    if (slot != nullptr) *slot = s.slot;
    e->seqs.emplace(id, std::move(s));
  });
}

int ccinfer_free_seq(ccinfer_engine* e, int64_t id) {
  return guarded(e, [&] {
    need(e, "engine");
    Sequence& s = e->seq(id);
    std::vector<int> pages;
    for (size_t g = 0; g < e->groups.size(); ++g) {
      pages.clear();
      for (int p : s.tables[g])
        if (p >= 0) pages.push_back(p);
      e->pools[g].give_back(id, pages.data(), (int)pages.size());
      s.tables[g].clear();
    }
    e->slots.give_back(s.slot);
    e->seqs.erase(id);
  });
}

int ccinfer_seq_state(const ccinfer_engine* e, int64_t id, int* slot, int* ctx_len, int* reserved_tokens) {
  return guarded(e, [&] {
    need(e, "engine");
    const Sequence& s = e->seq(id);
    if (slot != nullptr) *slot = s.slot;
    if (ctx_len != nullptr) *ctx_len = s.ctx_len;
    if (reserved_tokens != nullptr) *reserved_tokens = s.reserved_tokens;
  });
}

int ccinfer_seq_block_table(const ccinfer_engine* e, int64_t id, int group, int* out, int capacity, int* len) {
  return guarded(e, [&] {
    need(e, "engine");
    need(len, "len");
    const Sequence& s = e->seq(id);
    if (group < 0 || group >= (int)e->groups.size()) fail(CCINFER_INVALID_ARGUMENT, "no such cache group");
    const auto& t = s.tables[group];
    *len = (int)t.size();
    if (out != nullptr) std::memcpy(out, t.data(), sizeof(int) * std::min<size_t>(t.size(), capacity > 0 ? capacity : 0));
  });
}

int ccinfer_pages_needed(const ccinfer_engine* e, int64_t id, int n_new, int* per_group) {
  return guarded(e, [&] {
    need(e, "engine");
    need(per_group, "per_group");
    const Sequence& s = e->seq(id);
    for (size_t g = 0; g < e->groups.size(); ++g) per_group[g] = e->pages_needed(s, (int)g, n_new);
  });
}

int ccinfer_reserve(ccinfer_engine* e, int64_t id, int n_new) {
  return guarded(e, [&] { need(e, "engine"); e->reserve(e->seq(id), n_new); });
}
int ccinfer_commit(ccinfer_engine* e, int64_t id) {
  return guarded(e, [&] { need(e, "engine"); e->commit(e->seq(id)); });
}
int ccinfer_rollback(ccinfer_engine* e, int64_t id) {
  return guarded(e, [&] { need(e, "engine"); e->undo(e->seq(id)); });
}

int ccinfer_pool_take(ccinfer_engine* e, int group, int64_t owner, int n, int* pages_out) {
  return guarded(e, [&] {
    need(e, "engine");
    if (group < 0 || group >= (int)e->groups.size()) fail(CCINFER_INVALID_ARGUMENT, "no such cache group");
    if (n > 0) need(pages_out, "pages_out");
    if (e->seqs.count(owner)) fail(CCINFER_INVALID_ARGUMENT, "owner " + str(owner) + " is an open sequence: its pages come with its steps");
    e->pools[group].take(owner, n, pages_out);
  });
}
int ccinfer_pool_give_back(ccinfer_engine* e, int group, int64_t owner, const int* pages, int n) {
  return guarded(e, [&] {
    need(e, "engine");
    if (group < 0 || group >= (int)e->groups.size()) fail(CCINFER_INVALID_ARGUMENT, "no such cache group");
    if (e->seqs.count(owner)) fail(CCINFER_INVALID_ARGUMENT, "owner " + str(owner) + " is an open sequence: free it instead");
    e->pools[group].give_back(owner, pages, n);
  });
}
int ccinfer_pool_owner(const ccinfer_engine* e, int group, int page, int64_t* owner, int* is_free) {
  return guarded(e, [&] {
    need(e, "engine");
    if (group < 0 || group >= (int)e->groups.size()) fail(CCINFER_INVALID_ARGUMENT, "no such cache group");
    if (page < 0 || page >= e->pools[group].num_pages()) fail(CCINFER_KV_INVALID_BLOCK_TABLE, "page outside the pool");
    const int64_t o = e->pools[group].owner_of(page);
    if (is_free != nullptr) *is_free = o == kNoOwner;
    if (owner != nullptr) *owner = o == kNoOwner ? 0 : o;
  });
}
int ccinfer_slot_take(ccinfer_engine* e, int* slot) {
  return guarded(e, [&] { need(e, "engine"); need(slot, "slot"); *slot = e->slots.take(); });
}
int ccinfer_slot_give_back(ccinfer_engine* e, int slot) {
  return guarded(e, [&] { need(e, "engine"); e->slots.give_back(slot); });
}

int ccinfer_set_runner(ccinfer_engine* e, ccinfer_runner run, void* user) {
  return guarded(e, [&] {
    need(e, "engine");
    e->runner = run;
    e->runner_user = user;
  });
}

int ccinfer_forward(ccinfer_engine* e, int n_entries, const int64_t* seq_ids, const int* counts, const int* tokens,
                    const int* want_counts, const int* wants, int pad_to, int32_t* small_buffer,
                    int32_t* large_buffer, ccinfer_step_info* info_out) {
  std::vector<Sequence*> reserved;
  const int rc = guarded(e, [&] {
    need(e, "engine");
    need(seq_ids, "seqs");
    need(counts, "counts");
    need(tokens, "tokens");
    need(want_counts, "want_counts");
    need(info_out, "info_out");
    // ---- validation, once, on the host (src/worker/batch_translator.cpp:18-41, 94-96, 191-194) ----
    const int B = n_entries;
    if (B <= 0) fail(CCINFER_INVALID_ARGUMENT, "a step needs at least one entry");
    if (B > e->max_seqs) fail(CCINFER_INVALID_ARGUMENT, str(B) + " entries in a step, at most " + str(e->max_seqs));
    std::vector<Sequence*> given(B);
    std::vector<int> tok_begin(B + 1, 0), want_begin(B + 1, 0);
    {
      std::unordered_set<int64_t> seen;
      for (int i = 0; i < B; ++i) {
        if (!seen.insert(seq_ids[i]).second) fail(CCINFER_INVALID_ARGUMENT, "sequence " + str(seq_ids[i]) + " appears twice in one step");
        given[i] = &e->seq(seq_ids[i]);
        if (counts[i] <= 0) fail(CCINFER_INVALID_ARGUMENT, "sequence " + str(seq_ids[i]) + " brings no tokens");
        if (want_counts[i] < 0) fail(CCINFER_INVALID_ARGUMENT, "a negative number of wanted places");
        tok_begin[i + 1] = tok_begin[i] + counts[i];
        want_begin[i + 1] = want_begin[i] + want_counts[i];
        if (given[i]->ctx_len + counts[i] > e->max_context)
          fail(CCINFER_REQUEST_TOO_LONG, "sequence " + str(seq_ids[i]) + ": " + str(given[i]->ctx_len) + " cached + " +
                                             str(counts[i]) + " new tokens exceed the limit of " + str(e->max_context));
        for (int j = tok_begin[i]; j < tok_begin[i + 1]; ++j)
          if (tokens[j] < 0 && !(counts[i] == 1 && tokens[j] == -1))
            fail(CCINFER_INVALID_ARGUMENT, "sequence " + str(seq_ids[i]) + ": token ids are non-negative (-1 stands alone, for the token last sampled)");
        if (want_counts[i] > 0) need(wants, "wants");
        for (int j = want_begin[i]; j < want_begin[i + 1]; ++j)
          if (wants[j] < 0 || wants[j] >= counts[i])
            fail(CCINFER_INVALID_ARGUMENT, "sequence " + str(seq_ids[i]) + ": wanted place " + str(wants[j]) + " is outside its " + str(counts[i]) + " tokens");
      }
    }
    const int T = tok_begin[B];
    if (T > e->max_tokens) fail(CCINFER_INVALID_ARGUMENT, str(T) + " tokens in a step, at most " + str(e->max_tokens));
    if (want_begin[B] > e->max_tokens)
      fail(CCINFER_INVALID_ARGUMENT, str(want_begin[B]) + " logits rows wanted in a step, at most " + str(e->max_tokens));
    const int Bp = std::max(B, pad_to);
    if (pad_to > 0) {
      if (T != B) fail(CCINFER_INVALID_ARGUMENT, "only a step of single tokens can be padded");
      if (Bp > e->max_seqs) fail(CCINFER_INVALID_ARGUMENT, "padding beyond max_seqs");
    }
    const int Tp = T + (Bp - B);
    const int R = pad_to > 0 ? Bp : want_begin[B];
    // ---- pages for the step: all entries or none ----
    for (int i = 0; i < B; ++i) {
      e->reserve(*given[i], counts[i]);
      reserved.push_back(given[i]);
    }
    // ---- layout: single-token entries first (kernels treat the two kinds of rows differently) ----
    std::vector<int>& order = e->order_scratch;
    order.resize(B);
    for (int i = 0; i < B; ++i) order[i] = i;
    std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return (counts[a] != 1) < (counts[b] != 1); });
    const bool use_small = Tp <= e->small.c.capacity_tokens && R <= e->small.c.capacity_tokens;
    const ccinfer_layout& L = use_small ? e->small.c : e->large.c;
    int32_t* buf = use_small ? small_buffer : large_buffer;
    need(buf, use_small ? "small_buffer" : "large_buffer");
    std::vector<int> cu(B + 1, 0), place(B);
    int n_single = 0, max_q = 0, max_ctx = 0;
    for (int k = 0; k < B; ++k) {
      const int i = order[k];
      place[i] = k;
      cu[k + 1] = cu[k] + counts[i];
      n_single += counts[i] == 1;
      max_q = std::max(max_q, counts[i]);
      max_ctx = std::max(max_ctx, given[i]->ctx_len + counts[i]);
    }
    int32_t* tok = buf + L.token_ids;
    int32_t* pos = buf + L.positions;
    int32_t* eot = buf + L.entry_of_token;
    for (int k = 0; k < B; ++k) {
      const int i = order[k];
      const Sequence& s = *given[i];
      for (int j = 0; j < counts[i]; ++j) {
        const int t = cu[k] + j;
        const int id = tokens[tok_begin[i] + j];
        tok[t] = id >= 0 ? id : -1 - s.slot;   // resolved on the device from the token last sampled for the slot
        pos[t] = s.ctx_len + j;
        eot[t] = k;
      }
      buf[L.cu_q + k] = cu[k];
      buf[L.pos0 + k] = s.ctx_len;
      buf[L.ctx_after + k] = s.ctx_len + counts[i];
      buf[L.state_slot + k] = s.slot;
    }
    buf[L.cu_q + B] = T;
    for (int t = T; t < Tp; ++t) {   // padding rows: they cache nothing and attend to nothing
      tok[t] = 0;
      pos[t] = 0;
      eot[t] = -1;
    }
    for (int k = B; k < Bp; ++k) {
      buf[L.cu_q + k + 1] = T + (k - B) + 1;
      buf[L.pos0 + k] = 0;
      buf[L.ctx_after + k] = 0;
      buf[L.state_slot + k] = -1;
    }
    // rows whose logits are wanted, in the order of the caller's entries and of their wants
    if (pad_to > 0) {
      for (int k = 0; k < Bp; ++k) {
        buf[L.logit_rows + k] = k;
        buf[L.row_slot + k] = k < B ? given[order[k]]->slot : -1;
      }
    } else {
      int r = 0;
      for (int i = 0; i < B; ++i)
        for (int j = want_begin[i]; j < want_begin[i + 1]; ++j, ++r) {
          buf[L.logit_rows + r] = cu[place[i]] + wants[j];
          buf[L.row_slot + r] = given[i]->slot;
        }
    }
    // per group: where each token's cached tensors go, and each entry's block table
    auto& lens = e->row_len[buf];
    if (lens.size() != e->groups.size()) lens.assign(e->groups.size(), std::vector<int>(L.capacity_entries, 0));
    const int stride = L.block_table_stride;
    for (size_t g = 0; g < e->groups.size(); ++g) {
      const int P = e->groups[g].page_size;
      int32_t* sm = buf + L.slot_map[g];
      int32_t* bt = buf + L.block_table[g];
      for (int k = 0; k < B; ++k) {
        const Sequence& s = *given[order[k]];
        const auto& table = s.tables[g];
        const int n = std::min<int>((int)table.size(), stride);
        int32_t* row = bt + (size_t)k * stride;
        std::memcpy(row, table.data(), sizeof(int32_t) * n);
        for (int j = n; j < lens[g][k]; ++j) row[j] = -1;   // what an earlier, longer sequence left in this row
        lens[g][k] = n;
        for (int t = cu[k]; t < cu[k + 1]; ++t) {
          const int p = pos[t];
          sm[t] = table[p / P] * P + p % P;
        }
      }
      for (int t = T; t < Tp; ++t) sm[t] = -1;
    }
    // ---- what the runner has to know ----
    ccinfer_step_info& info = *info_out;
    info.layout = use_small ? 0 : 1;
    info.n_tokens = Tp;
    info.n_entries = Bp;
    info.n_real_tokens = T;
    info.n_real_entries = B;
    info.n_logit_rows = R;
    info.n_single = n_single == B ? n_single + (Bp - B) : n_single;   // padding rows are single rows too
    info.max_q_len = max_q;
    info.max_ctx = max_ctx;
    info.order = order.data();
    info.n_copies = 0;
    auto add_copy = [&info](int off, int words) {
      if (words <= 0) return;
      if (info.n_copies > 0 && info.copy_offset[info.n_copies - 1] + info.copy_words[info.n_copies - 1] == off) {
        info.copy_words[info.n_copies - 1] += words;   // adjacent: one copy
        return;
      }
      info.copy_offset[info.n_copies] = off;
      info.copy_words[info.n_copies] = words;
      ++info.n_copies;
    };
    add_copy(0, e->groups.empty() ? L.size_words : L.block_table[0]);
    for (size_t g = 0; g < e->groups.size(); ++g) add_copy(L.block_table[g], Bp * stride);
    // ---- the device work, then the step counts ----
    if (e->runner != nullptr) {
      const int r = e->runner(e->runner_user, &info);
      if (r != 0) fail(CCINFER_RUNNER_FAILED, "the runner reported " + str(r));
    }
    for (Sequence* s : reserved) e->commit(*s);
    reserved.clear();
    ++e->steps;
  });
  if (rc != CCINFER_OK) {
    for (Sequence* s : reserved) {   // give back what the step took; nothing has moved
      try {
        e->undo(*s);
      } catch (const Failure&) {
      }
    }
  }
  return rc;
}

}  // extern "C"
