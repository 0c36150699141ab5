// Continuous batching above the step function, behind the scheduler calls of ccinfer.h.
//
// The decisions are those of 7QiC/ccInfer's scheduler (src/scheduler/scheduler.cpp:398-598): requests are
// admitted first come first served; a step is built under a token budget and the free pages of the cache;
// requests that are decoding come first, one token each; then portions of prompts, at most prefill_chunk_size
// tokens (0 = whole prompts), shrunk to what the free pages hold; a new prompt starts only while fewer than
// max_running requests have started; whoever ran goes to the back of the order (round robin,
// src/scheduler/scheduler.cpp:600-615).  The first new token comes from a prompt's last portion.  A request
// ends at max_tokens or at the longest context (the reference never stops at an end-of-sequence token,
// src/model/model_runner.h:242; here eos_token_id may be given).
//
// When pages run out (src/scheduler/scheduler.cpp:225-268, 811-845) the reference suspends every blocked
// request and replays it; here ONE request gives way, the one that started last, so that older requests keep
// going: all its pages are given back, its prompt becomes prompt + generated[:-1] and is computed again
// without sampling, then decoding goes on from its last token.  A request's draw depends only on (seed, number
// of tokens it has produced), so a request that gave way produces the same tokens as an undisturbed one.
//
// Unlike the reference (one SamplingParams per batch, requests that differ are skipped, :489-498), every
// request keeps its own parameters and greedy and temperature requests share a step.
//
// Running ahead (the reference's loop waits for every step, src/scheduler/scheduler.cpp:206-284): a step is
// launched before the tokens of the step before it have been read.  A decoding request's item then names its
// token by -1; the step function finds it on the device, where the sampling kernel left it.  Everything that
// decides a step is known without the tokens (lengths, pages, how many tokens a request has produced), except
// an end-of-sequence stop: a request that stops that way has one more step in flight, whose token is dropped.
// The events of a step are queued by the call after it; before a request gives way or is cancelled the step in
// flight is read first, so those never see a token that is still on the device.
//
// This file uses the engine through the public calls of ccinfer.h only.
#include "ccinfer.h"

#include <algorithm>
#include <deque>
#include <memory>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

namespace {

struct Failure {
  int code;
  std::string message;
};

[[noreturn]] void fail(int code, std::string message) { throw Failure{code, std::move(message)}; }
std::string str(long long v) { return std::to_string(v); }

constexpr int kPending = -1;   // in place of a token that the sampling kernel left on the device

struct Request {
  int64_t id = 0;
  int64_t seq = 0;                 // the engine's sequence that holds its cache
  std::vector<int> initial_prompt;
  std::vector<int> prompt;         // what has to be in the cache before decoding (grows when it gives way)
  ccinfer_sampling_params params{};
  std::vector<int> generated;
  int cursor = 0;                  // tokens of `prompt` already cached
  bool opened = false;             // holds a slot in the engine
  long long started_at = -1;       // order of first scheduling (who gives way)
  bool replaying = false;          // the prompt's last portion does not sample
  bool finished = false;
  int pending = 0;                 // tokens drawn in a step whose results have not been read yet

  int n_out() const { return (int)generated.size() + pending; }   // those still on the device included
  bool prefill_done() const { return cursor >= (int)prompt.size(); }
};
using RequestPtr = std::shared_ptr<Request>;

struct Item {
  RequestPtr r;
  std::vector<int> tokens;
  bool sample;
  bool prefill;
};

struct InFlight {
  std::vector<RequestPtr> reqs;   // the requests that sampled, in item order
  int64_t ticket;
};

}  // namespace

struct ccinfer_scheduler {
  ccinfer_engine* engine;
  ccinfer_scheduler_options opt;
  ccinfer_scheduler_hooks hooks;
  std::vector<ccinfer_group> groups;
  std::deque<RequestPtr> waiting;
  std::unordered_map<int64_t, RequestPtr> active;
  std::vector<int64_t> order;               // round-robin order of the active requests
  std::vector<int64_t> blocked;             // requests of the last plan that found no pages
  long long start_counter = 0, preemptions = 0, steps = 0;
  int64_t next_ticket = 1;
  std::unique_ptr<InFlight> inflight;
  std::deque<ccinfer_event> events;
  mutable std::string last_error;
  // the plan handed to the run hook
  std::vector<int64_t> p_reqs;
  std::vector<int> p_counts, p_tokens, p_sample, p_out_index, tokens_scratch;
  std::vector<ccinfer_sampling_params> p_params;

  // -- the engine, through its public calls ------------------------------------------------
  void ok(int rc) const {
    if (rc != CCINFER_OK) fail(rc, ccinfer_last_error(engine));
  }
  ccinfer_stats_t engine_stats() const {
    ccinfer_stats_t st;
    ok(ccinfer_stats(engine, &st));
    return st;
  }
  int ctx_len(const Request& r) const {
    int slot, ctx, reserved;
    ok(ccinfer_seq_state(engine, r.seq, &slot, &ctx, &reserved));
    return ctx;
  }
  void pages_needed(const Request& r, int n_new, int* per_group) const { ok(ccinfer_pages_needed(engine, r.seq, n_new, per_group)); }
  int table_len(const Request& r, int g) const {
    int n;
    ok(ccinfer_seq_block_table(engine, r.seq, g, nullptr, 0, &n));
    return n;
  }
  void hook(int rc, const char* what) const {
    if (rc != CCINFER_OK) fail(rc >= CCINFER_INVALID_ARGUMENT && rc <= CCINFER_RUNNER_FAILED ? rc : CCINFER_RUNNER_FAILED,
                               std::string("the ") + what + " hook failed");
  }
  void open(Request& r) {
    if (hooks.open != nullptr) {
      hook(hooks.open(hooks.user, r.id, &r.seq), "open");
    } else {
      int slot;
      ok(ccinfer_alloc_seq(engine, r.id, &slot));
      r.seq = r.id;
    }
    r.opened = true;
  }
  void close(Request& r) {
    if (!r.opened) return;
    r.opened = false;
    if (hooks.close != nullptr) hook(hooks.close(hooks.user, r.id), "close");
    else ok(ccinfer_free_seq(engine, r.seq));
  }

  // -- requests ------------------------------------------------------------------------------
  void add(int64_t id, const int* prompt, int n, const ccinfer_sampling_params& sp) {
    if (sp.top_k < 0) fail(CCINFER_INVALID_ARGUMENT, "top_k must be 0 (off) or a positive count");
    if (!(sp.top_p > 0.0f)) fail(CCINFER_INVALID_ARGUMENT, "top_p must be above 0 (1 or more = off)");
    bool known = active.count(id) > 0;
    for (const auto& w : waiting) known = known || w->id == id;
    if (known) fail(CCINFER_INVALID_ARGUMENT, "request " + str(id) + " is already known");
    if (n <= 0) fail(CCINFER_INVALID_ARGUMENT, "a prompt needs at least one token");
    for (int i = 0; i < n; ++i)
      if (prompt[i] < 0) fail(CCINFER_INVALID_ARGUMENT, "token ids are non-negative integers");
    if (n > opt.max_context)
      fail(CCINFER_REQUEST_TOO_LONG, "a prompt of " + str(n) + " tokens exceeds the longest context " + str(opt.max_context));
    // a group that keeps every token must be able to hold the prompt (a window group gives pages back as the
    // request moves on: its pool bounds the size of a portion, not the length of a prompt)
    long long pool_tokens = -1;
    for (const auto& g : groups)
      if (g.window <= 0) {
        const long long t = (long long)g.num_pages * g.page_size;
        pool_tokens = pool_tokens < 0 ? t : std::min(pool_tokens, t);
      }
    if (pool_tokens >= 0 && n > pool_tokens)
      fail(CCINFER_REQUEST_TOO_LONG, "a prompt of " + str(n) + " tokens can never fit the cache pool of " + str(pool_tokens) + " tokens");
    auto r = std::make_shared<Request>();
    r->id = id;
    r->initial_prompt.assign(prompt, prompt + n);
    r->prompt = r->initial_prompt;
    r->params = sp;
    waiting.push_back(std::move(r));
  }

  void retire(const RequestPtr& r) {
    r->finished = true;
    close(*r);
    active.erase(r->id);
    order.erase(std::remove(order.begin(), order.end(), r->id), order.end());
  }

  bool cancel(int64_t id) {
    for (auto it = waiting.begin(); it != waiting.end(); ++it)
      if ((*it)->id == id) {
        waiting.erase(it);
        return true;
      }
    if (active.count(id)) resolve();   // its last token may still be on the device
    auto it = active.find(id);
    if (it == active.end()) return false;
    RequestPtr r = it->second;
    retire(r);
    return true;
  }

  bool has_work() const { return !waiting.empty() || !active.empty() || inflight != nullptr || !events.empty(); }

  // -- building a step -----------------------------------------------------------------------
  // moves waiting requests into the active set while slots are free (first come first served)
  void admit() {
    while (!waiting.empty() && engine_stats().slots_free > 0) {
      RequestPtr r = waiting.front();
      waiting.pop_front();
      if (r->params.max_tokens <= 0) {   // finished at once (src/scheduler/scheduler.cpp:309-314)
        events.push_back({r->id, -1, 1, CCINFER_REASON_MAX_TOKENS});
        continue;
      }
      open(*r);
      active[r->id] = r;
      order.push_back(r->id);
    }
  }

  // the most tokens (<= n) of a portion whose pages fit what is free in every group
  int largest_fit(const Request& r, int n, const int* free) const {
    long long best = n;
    const int ctx = ctx_len(r);
    for (size_t g = 0; g < groups.size(); ++g) {
      const long long room = ((long long)table_len(r, (int)g) + free[g]) * groups[g].page_size - ctx;
      best = std::min(best, room);
    }
    return (int)std::max(0LL, best);
  }

  std::vector<Item> plan() {
    const ccinfer_stats_t st = engine_stats();
    int free[CCINFER_MAX_GROUPS], need[CCINFER_MAX_GROUPS];
    const int G = (int)groups.size();
    for (int g = 0; g < G; ++g) free[g] = st.pages_free[g];
    int budget = opt.max_tokens_per_step;
    std::vector<Item> items;
    blocked.clear();
    auto fits = [&] {
      for (int g = 0; g < G; ++g)
        if (need[g] > free[g]) return false;
      return true;
    };
    auto take = [&] {
      for (int g = 0; g < G; ++g) free[g] -= need[g];
    };
    // decoding requests first, one token each
    for (int64_t id : order) {
      const RequestPtr& r = active.at(id);
      if (!r->prefill_done() || budget <= 0) continue;
      if (r->pending && (r->n_out() >= r->params.max_tokens || ctx_len(*r) + 1 > opt.max_context))
        continue;   // it ends when its token has been read
      pages_needed(*r, 1, need);
      if (!fits()) {
        blocked.push_back(id);
        continue;
      }
      take();
      budget -= 1;
      items.push_back({r, {r->pending ? kPending : r->generated.back()}, true, false});
    }
    // then portions of prompts
    int started = 0;
    for (const auto& kv : active) started += kv.second->started_at >= 0;
    for (int64_t id : order) {
      const RequestPtr& r = active.at(id);
      if (r->prefill_done() || budget <= 0) continue;
      if (r->started_at < 0 && started >= opt.max_running) continue;
      const int remaining = (int)r->prompt.size() - r->cursor;
      int n = opt.prefill_chunk_size == 0 ? remaining : std::min(remaining, opt.prefill_chunk_size);
      n = std::min(n, budget);
      pages_needed(*r, n, need);
      if (!fits()) {
        n = largest_fit(*r, n, free);
        if (n <= 0) {
          blocked.push_back(id);
          continue;
        }
        pages_needed(*r, n, need);
      }
      take();
      budget -= n;
      const bool last = r->cursor + n >= (int)r->prompt.size();
      items.push_back({r, std::vector<int>(r->prompt.begin() + r->cursor, r->prompt.begin() + r->cursor + n),
                       last && !r->replaying, true});
      if (r->started_at < 0) {
        r->started_at = start_counter++;
        ++started;
      }
    }
    return items;
  }

  // frees the pages of the request that started last (it will be computed again); false if none can give way
  bool preempt_one() {
    std::vector<RequestPtr> victims;
    for (const auto& kv : active)
      if (kv.second->started_at >= 0 && ctx_len(*kv.second) > 0) victims.push_back(kv.second);
    bool blocked_other = false;
    for (int64_t b : blocked) {
      bool among = false;
      for (const auto& v : victims) among = among || v->id == b;
      blocked_other = blocked_other || !among;
    }
    if (victims.size() <= 1 && !blocked_other) return false;
    if (victims.empty()) return false;
    RequestPtr v = *std::max_element(victims.begin(), victims.end(),
                                     [](const RequestPtr& a, const RequestPtr& b) { return a->started_at < b->started_at; });
    close(*v);
    open(*v);
    if (!v->generated.empty()) {
      v->prompt = v->initial_prompt;
      v->prompt.insert(v->prompt.end(), v->generated.begin(), v->generated.end() - 1);
      v->replaying = true;
    }
    v->cursor = 0;
    v->started_at = -1;
    order.erase(std::remove(order.begin(), order.end(), v->id), order.end());   // it queues behind the others
    order.push_back(v->id);
    ++preemptions;
    return true;
  }

  // a request whose next token would not fit the longest context ends (src/scheduler/scheduler.cpp:477-481)
  void finish_exhausted() {
    std::vector<RequestPtr> done;
    for (int64_t id : order) {
      const RequestPtr& r = active.at(id);
      if (r->pending) continue;   // after its token has been read
      if (r->prefill_done() && ctx_len(*r) + 1 > opt.max_context) done.push_back(r);
    }
    for (const auto& r : done) {
      events.push_back({r->id, -1, 1, CCINFER_REASON_MAX_CONTEXT});
      retire(r);
    }
  }

  // -- running a step ------------------------------------------------------------------------
  void read(const InFlight& rec) {
    const int n = (int)rec.reqs.size();
    tokens_scratch.assign(std::max(1, n), 0);
    hook(hooks.read(hooks.user, rec.ticket, n, tokens_scratch.data()), "read");
    for (int i = 0; i < n; ++i) {
      const RequestPtr& r = rec.reqs[i];
      if (r->finished) continue;   // it ended while this step was in flight; the token is dropped
      const int tok = tokens_scratch[i];
      r->pending -= 1;
      r->generated.push_back(tok);
      int reason = CCINFER_REASON_NONE;
      if ((int)r->generated.size() >= r->params.max_tokens) reason = CCINFER_REASON_MAX_TOKENS;
      else if (opt.eos_token_id >= 0 && tok == opt.eos_token_id) reason = CCINFER_REASON_EOS;
      events.push_back({r->id, tok, reason != CCINFER_REASON_NONE, reason});
      if (reason != CCINFER_REASON_NONE) retire(r);
    }
  }

  // reads the tokens of the step in flight, if there is one
  void resolve() {
    std::unique_ptr<InFlight> previous = std::move(inflight);
    inflight.reset();
    if (previous) read(*previous);
  }

  void step() {
    admit();
    finish_exhausted();
    std::vector<Item> items;
    if (!active.empty()) items = plan();
    if (items.empty() && inflight) {
      // nothing to launch before the tokens in flight are known (requests at their last token, or pages that
      // only an ending request gives back)
      resolve();
      admit();
      finish_exhausted();
      if (!active.empty()) items = plan();
    }
    if (active.empty()) return;
    size_t guard = 0;
    while (items.empty()) {
      // nothing fits: give one request's pages to the others, or fail if there is nothing to give
      ++guard;
      if (guard > active.size() + 1 || !preempt_one())
        fail(CCINFER_KV_BLOCK_EXHAUSTED,
             "no request can make progress: the cache pool is too small for the requests that are running");
      items = plan();
    }
    // the plan, as plain arrays
    p_reqs.clear(), p_counts.clear(), p_tokens.clear(), p_sample.clear(), p_out_index.clear(), p_params.clear();
    std::vector<RequestPtr> sampled;
    for (const Item& it : items) {
      p_reqs.push_back(it.r->id);
      p_counts.push_back((int)it.tokens.size());
      p_tokens.insert(p_tokens.end(), it.tokens.begin(), it.tokens.end());
      p_sample.push_back(it.sample ? 1 : 0);
      p_out_index.push_back(it.r->n_out());
      p_params.push_back(it.r->params);
      if (it.sample) sampled.push_back(it.r);
    }
    ccinfer_plan pl{};
    pl.n_items = (int)items.size();
    pl.reqs = p_reqs.data(), pl.counts = p_counts.data(), pl.tokens = p_tokens.data(), pl.sample = p_sample.data();
    pl.out_index = p_out_index.data(), pl.params = p_params.data();
    pl.n_sampled = (int)sampled.size();
    const int64_t ticket = next_ticket++;
    hook(hooks.run(hooks.user, &pl, ticket), "run");
    ++steps;
    // what is known at launch
    for (const Item& it : items) {
      Request& r = *it.r;
      if (it.prefill) {
        r.cursor += (int)it.tokens.size();
        if (r.prefill_done() && r.replaying) r.replaying = false;   // decoding goes on from the token it already has
      }
      if (it.sample) r.pending += 1;
    }
    // whoever ran goes to the back
    std::vector<int64_t> keep;
    for (int64_t id : order)
      if (std::find(p_reqs.begin(), p_reqs.end(), id) == p_reqs.end()) keep.push_back(id);
    keep.insert(keep.end(), p_reqs.begin(), p_reqs.end());
    order = std::move(keep);
    std::unique_ptr<InFlight> previous = std::move(inflight);
    inflight.reset();
    if (!sampled.empty()) inflight.reset(new InFlight{std::move(sampled), ticket});
    if (previous) read(*previous);
    if (!opt.run_ahead) resolve();
  }
};

namespace {

thread_local std::string g_create_error;

template <typename F>
int guarded(const ccinfer_scheduler* s, F&& f) {
  try {
    f();
    return CCINFER_OK;
  } catch (const Failure& x) {
    (s != nullptr ? s->last_error : g_create_error) = x.message;
    return x.code;
  } catch (const std::exception& x) {
    (s != nullptr ? s->last_error : g_create_error) = x.what();
    return CCINFER_INVALID_STATE;
  }
}

void need(const void* p, const char* what) {
  if (p == nullptr) fail(CCINFER_INVALID_ARGUMENT, std::string(what) + " is null");
}

}  // namespace

extern "C" {

int ccinfer_scheduler_create(ccinfer_engine* e, const ccinfer_scheduler_options* options,
                             const ccinfer_scheduler_hooks* hooks, ccinfer_scheduler** out) {
  return guarded(nullptr, [&] {
    need(e, "engine"), need(options, "options"), need(hooks, "hooks"), need(out, "out");
    if (hooks->run == nullptr || hooks->read == nullptr) fail(CCINFER_INVALID_ARGUMENT, "the run and read hooks are required");
    if (options->prefill_chunk_size < 0 || options->max_tokens_per_step <= 0 || options->max_running <= 0)
      fail(CCINFER_INVALID_ARGUMENT, "prefill_chunk_size >= 0, max_tokens_per_step > 0, max_running > 0");
    if (options->max_context <= 0) fail(CCINFER_INVALID_ARGUMENT, "max_context must be > 0");
    std::unique_ptr<ccinfer_scheduler> s(new ccinfer_scheduler());
    s->engine = e;
    s->opt = *options;
    s->hooks = *hooks;
    s->groups.resize(CCINFER_MAX_GROUPS);
    int n = 0;
    if (ccinfer_get_groups(e, s->groups.data(), CCINFER_MAX_GROUPS, &n) != CCINFER_OK) fail(CCINFER_INVALID_ARGUMENT, ccinfer_last_error(e));
    s->groups.resize(n);
    *out = s.release();
  });
}

void ccinfer_scheduler_destroy(ccinfer_scheduler* s) { delete s; }

const char* ccinfer_scheduler_last_error(const ccinfer_scheduler* s) {
  return s != nullptr ? s->last_error.c_str() : g_create_error.c_str();
}

int ccinfer_scheduler_stats(const ccinfer_scheduler* s, ccinfer_scheduler_stats_t* out) {
  return guarded(s, [&] {
    need(s, "scheduler"), need(out, "out");
    out->steps = s->steps;
    out->preemptions = s->preemptions;
    out->waiting = (int)s->waiting.size();
    out->active = (int)s->active.size();
    out->prefilling = 0;
    for (const auto& kv : s->active) out->prefilling += !kv.second->prefill_done();
    out->in_flight = s->inflight != nullptr;
    out->events = (int)s->events.size();
  });
}

int ccinfer_scheduler_active(const ccinfer_scheduler* s, int64_t* out, int capacity, int* n) {
  return guarded(s, [&] {
    need(s, "scheduler"), need(n, "n");
    *n = (int)s->order.size();
    for (int i = 0; i < std::min(capacity, *n); ++i) {
      need(out, "out");
      out[i] = s->order[i];
    }
  });
}

int ccinfer_add_request(ccinfer_scheduler* s, int64_t req, const int* prompt, int n_prompt,
                        const ccinfer_sampling_params* params) {
  return guarded(s, [&] {
    need(s, "scheduler"), need(params, "params");
    if (n_prompt > 0) need(prompt, "prompt");
    s->add(req, prompt, n_prompt, *params);
  });
}

int ccinfer_cancel(ccinfer_scheduler* s, int64_t req, int* found) {
  return guarded(s, [&] {
    need(s, "scheduler");
    const bool f = s->cancel(req);
    if (found != nullptr) *found = f;
  });
}

int ccinfer_has_work(const ccinfer_scheduler* s, int* yes) {
  return guarded(s, [&] {
    need(s, "scheduler"), need(yes, "yes");
    *yes = s->has_work();
  });
}

int ccinfer_step(ccinfer_scheduler* s) {
  return guarded(s, [&] {
    need(s, "scheduler");
    s->step();
  });
}

int ccinfer_drain(ccinfer_scheduler* s) {
  return guarded(s, [&] {
    need(s, "scheduler");
    s->resolve();
  });
}

int ccinfer_pop_events(ccinfer_scheduler* s, ccinfer_event* out, int capacity, int* n) {
  return guarded(s, [&] {
    need(s, "scheduler"), need(n, "n");
    *n = 0;
    while (*n < capacity && !s->events.empty()) {
      need(out, "out");
      out[(*n)++] = s->events.front();
      s->events.pop_front();
    }
  });
}

}  // extern "C"
