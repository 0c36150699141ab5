/* C interface of the host core of ccinfer_b200: cache manager, request slots, the arrays of a step.
 *
 * What 7QiC/ccInfer keeps in src/cache/kv_cache_manager.cpp (pages, FIFO free list, validate-then-mutate
 * release), src/worker/batch_translator.cpp (the arrays of a step, pages taken on demand, commit or roll back)
 * and src/worker/worker.cpp (sequences and their slots) lives here in C++ behind plain C types; every call
 * returns an error code (0 = ok) and ccinfer_last_error() gives the message of the last failure.
 *
 * The model itself (layers put together from parts, kernel launches) is not in this library: a step's device
 * work is done by a runner that the owner of the engine registers (the Python package registers its model's
 * forward pass).  ccinfer_forward() = validate -> take pages -> fill the step arrays -> runner -> commit, or
 * give the pages back if anything failed.  Above it, a scheduler (ccinfer_scheduler_create, ccinfer_add_request,
 * ccinfer_cancel, ccinfer_step): which requests run in the next step, which portions of their prompts, who
 * gives way when pages run out, when a request ends.  It runs a step and reads its sampled tokens through hooks
 * that the owner registers (the Python package's hooks call its step function and its sampling kernels).
 *
 * Not thread-safe: one thread drives an engine.
 */
#ifndef CCINFER_B200_HOST_H
#define CCINFER_B200_HOST_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CCINFER_API __attribute__((visibility("default")))

/* error codes; the names are those of 7QiC/ccInfer's src/base/error_code.h where it has one */
enum {
  CCINFER_OK = 0,
  CCINFER_INVALID_ARGUMENT = 1,
  CCINFER_KV_BLOCK_EXHAUSTED = 2,
  CCINFER_KV_BLOCK_DOUBLE_FREE = 3,
  CCINFER_KV_INVALID_BLOCK_TABLE = 4,
  CCINFER_SEQUENCE_LIMIT_REACHED = 5,
  CCINFER_REQUEST_TOO_LONG = 6,
  CCINFER_INVALID_STATE = 7,
  CCINFER_RUNNER_FAILED = 8
};

typedef struct ccinfer_engine ccinfer_engine;

/* one cache group: layers whose mixers read the same keys share a page pool and block tables */
typedef struct ccinfer_group {
  int window;     /* <= 0: every earlier token; W > 0: the last W tokens (pages behind the window are given back) */
  int page_size;  /* tokens per page */
  int num_pages;  /* pages of the pool */
} ccinfer_group;

typedef struct ccinfer_options {
  int n_groups;
  const ccinfer_group* groups;
  int max_seqs;             /* live sequences = state slots */
  int max_tokens_per_step;
  int max_context;          /* longest sequence; sizes the block-table rows */
} ccinfer_options;

/* Fixed offsets (in 32-bit words) of the step arrays inside a step buffer.  Two buffers exist: the small one
 * for steps of at most max_seqs token rows (every pure decode step), the large one for max_tokens_per_step. */
#define CCINFER_MAX_GROUPS 8
typedef struct ccinfer_layout {
  int capacity_tokens, capacity_entries, size_words;
  int token_ids, positions, entry_of_token, logit_rows, row_slot; /* [capacity_tokens] each */
  int cu_q;                                                        /* [capacity_entries + 1] */
  int pos0, ctx_after, state_slot;                                 /* [capacity_entries] each */
  int n_groups;
  int slot_map[CCINFER_MAX_GROUPS];                                /* [capacity_tokens] each */
  int block_table[CCINFER_MAX_GROUPS];                             /* [capacity_entries][block_table_stride] */
  int block_table_stride;
} ccinfer_layout;

/* what ccinfer_forward tells the runner about the step it has laid out */
typedef struct ccinfer_step_info {
  int layout;         /* 0: the small buffer, 1: the large one */
  int n_tokens;       /* token rows, padding included */
  int n_entries;      /* entries, padding included */
  int n_real_tokens, n_real_entries;
  int n_logit_rows;
  int n_single;       /* the first n_single entries (and rows) bring one token each */
  int max_q_len, max_ctx;
  int n_copies;       /* ranges of the buffer that hold this step's data: what must reach the device */
  int copy_offset[CCINFER_MAX_GROUPS + 1], copy_words[CCINFER_MAX_GROUPS + 1];
  const int* order;   /* [n_real_entries]: order[k] = index (in the caller's list) of the entry laid out k-th */
} ccinfer_step_info;

typedef int (*ccinfer_runner)(void* user, const ccinfer_step_info* info);

typedef struct ccinfer_stats_t {
  int seqs, slots_total, slots_free, n_groups;
  int pages_total[CCINFER_MAX_GROUPS], pages_free[CCINFER_MAX_GROUPS], pages_high_water[CCINFER_MAX_GROUPS];
  long long steps;
} ccinfer_stats_t;

CCINFER_API int ccinfer_create(const ccinfer_options* options, ccinfer_engine** out);
CCINFER_API void ccinfer_destroy(ccinfer_engine* e);
/* message of the last failed call on this engine (of the last failed ccinfer_create when e is NULL) */
CCINFER_API const char* ccinfer_last_error(const ccinfer_engine* e);
CCINFER_API int ccinfer_get_layout(const ccinfer_engine* e, int which, ccinfer_layout* out);
CCINFER_API int ccinfer_stats(const ccinfer_engine* e, ccinfer_stats_t* out);
/* the groups the engine was created with: copies min(capacity, n) of them and returns n */
CCINFER_API int ccinfer_get_groups(const ccinfer_engine* e, ccinfer_group* out, int capacity, int* n);
/* every page is free or in exactly one table of its owner, no page is lost; CCINFER_INVALID_STATE otherwise */
CCINFER_API int ccinfer_check(const ccinfer_engine* e);

/* sequences */
CCINFER_API int ccinfer_alloc_seq(ccinfer_engine* e, int64_t seq, int* slot);
CCINFER_API int ccinfer_free_seq(ccinfer_engine* e, int64_t seq);
CCINFER_API int ccinfer_seq_state(const ccinfer_engine* e, int64_t seq, int* slot, int* ctx_len, int* reserved_tokens);
/* copies the block table of a group (logical page -> physical page, -1 = none) and returns its length */
CCINFER_API int ccinfer_seq_block_table(const ccinfer_engine* e, int64_t seq, int group, int* out, int capacity, int* len);
CCINFER_API int ccinfer_pages_needed(const ccinfer_engine* e, int64_t seq, int n_new, int* per_group);
/* the three halves of a step for callers that run the device work themselves */
CCINFER_API int ccinfer_reserve(ccinfer_engine* e, int64_t seq, int n_new);
CCINFER_API int ccinfer_commit(ccinfer_engine* e, int64_t seq);
CCINFER_API int ccinfer_rollback(ccinfer_engine* e, int64_t seq);

/* pools, as they are (tests; owners are the caller's numbers) */
CCINFER_API int ccinfer_pool_take(ccinfer_engine* e, int group, int64_t owner, int n, int* pages_out);
CCINFER_API int ccinfer_pool_give_back(ccinfer_engine* e, int group, int64_t owner, const int* pages, int n);
CCINFER_API int ccinfer_pool_owner(const ccinfer_engine* e, int group, int page, int64_t* owner, int* is_free);
CCINFER_API int ccinfer_slot_take(ccinfer_engine* e, int* slot);
CCINFER_API int ccinfer_slot_give_back(ccinfer_engine* e, int slot);

/* a step */
CCINFER_API int ccinfer_set_runner(ccinfer_engine* e, ccinfer_runner run, void* user);
/* Lays out a step of n_entries (sequence, its next tokens, the places among them whose logits are wanted) in
 * `small_buffer` or `large_buffer` (pinned host memory of the sizes ccinfer_get_layout names), takes the pages
 * it needs, calls the runner and commits; on any failure the pages taken for the step are given back and no
 * sequence has moved.  A token of -1 in a one-token entry stands for "the token last sampled for this
 * sequence" and reaches the device as -1 - slot.  pad_to > 0: a step of single tokens padded with rows that
 * cache nothing and attend to nothing up to pad_to entries (a CUDA graph's size); logits rows are then one
 * per entry, padding included. */
CCINFER_API int ccinfer_forward(ccinfer_engine* e, int n_entries, const int64_t* seqs, const int* counts,
                                const int* tokens, const int* want_counts, const int* wants, int pad_to,
                                int32_t* small_buffer, int32_t* large_buffer, ccinfer_step_info* info_out);

/* ------------------------------------------------------------------------------------------------------
 * the scheduler: continuous batching above ccinfer_forward (or above any step function, through the hooks)
 * ------------------------------------------------------------------------------------------------------ */
typedef struct ccinfer_scheduler ccinfer_scheduler;

/* names, meanings and defaults of 7QiC/ccInfer's SamplingParams (src/base/types.h:54-60) */
typedef struct ccinfer_sampling_params {
  int max_tokens;      /* generation limit */
  int top_k;           /* 0 = off */
  float top_p;         /* >= 1 = off */
  float temperature;   /* <= 0 = greedy */
  uint64_t seed;
} ccinfer_sampling_params;

typedef struct ccinfer_scheduler_options {
  int prefill_chunk_size;    /* most prompt tokens of one request in a step; 0 = whole prompts */
  int max_tokens_per_step;   /* the token budget of a step */
  int max_running;           /* requests whose prompts have started */
  int max_context;           /* a request ends when its next token would not fit */
  int eos_token_id;          /* < 0 = off */
  int run_ahead;             /* 1: a step is launched before the tokens of the step before it have been read */
} ccinfer_scheduler_options;

/* one step as the scheduler decided it: items in the order they run */
typedef struct ccinfer_plan {
  int n_items;
  const int64_t* reqs;       /* [n_items] */
  const int* counts;         /* [n_items] tokens of each item */
  const int* tokens;         /* all items' tokens; -1 in a one-token item = the token last sampled for the request,
                                which may still be on the device */
  const int* sample;         /* [n_items] 1: a token is drawn from the item's last position */
  const int* out_index;      /* [n_items] tokens the request has produced so far (keys the draw) */
  const ccinfer_sampling_params* params; /* [n_items] */
  int n_sampled;             /* items with sample = 1 */
} ccinfer_plan;

typedef struct ccinfer_scheduler_hooks {
  /* a request enters the engine (again, after it gave way); *seq = the sequence that holds its cache.
   * NULL: ccinfer_alloc_seq(engine, req), seq = req. */
  int (*open)(void* user, int64_t req, int64_t* seq);
  /* the request leaves: everything it holds is given back.  NULL: ccinfer_free_seq. */
  int (*close)(void* user, int64_t req);
  /* run the step (cache pages, forward pass) and launch the sampling of its n_sampled rows; their tokens are
   * asked for later by ticket.  Required. */
  int (*run)(void* user, const ccinfer_plan* plan, int64_t ticket);
  /* the tokens of an earlier run, in the order of its sampled items; waits for them.  Required. */
  int (*read)(void* user, int64_t ticket, int n, int* tokens_out);
  void* user;
} ccinfer_scheduler_hooks;

enum { CCINFER_REASON_NONE = 0, CCINFER_REASON_MAX_TOKENS = 1, CCINFER_REASON_MAX_CONTEXT = 2, CCINFER_REASON_EOS = 3 };

typedef struct ccinfer_event {
  int64_t req;
  int token;       /* -1: none (a request that ended without a new token) */
  int finished;
  int reason;      /* CCINFER_REASON_* when finished */
} ccinfer_event;

typedef struct ccinfer_scheduler_stats_t {
  long long steps, preemptions;
  int waiting, active, prefilling;   /* prefilling: active requests whose prompt is not yet all in the cache */
  int in_flight;                     /* 1: a step's tokens have not been read yet */
  int events;                        /* events not yet popped */
} ccinfer_scheduler_stats_t;

CCINFER_API int ccinfer_scheduler_create(ccinfer_engine* e, const ccinfer_scheduler_options* options,
                                         const ccinfer_scheduler_hooks* hooks, ccinfer_scheduler** out);
CCINFER_API void ccinfer_scheduler_destroy(ccinfer_scheduler* s);
CCINFER_API const char* ccinfer_scheduler_last_error(const ccinfer_scheduler* s);
CCINFER_API int ccinfer_scheduler_stats(const ccinfer_scheduler* s, ccinfer_scheduler_stats_t* out);
/* ids of the active requests in their running order: copies min(capacity, n) and returns n */
CCINFER_API int ccinfer_scheduler_active(const ccinfer_scheduler* s, int64_t* out, int capacity, int* n);
/* queues a request (first come first served) */
CCINFER_API int ccinfer_add_request(ccinfer_scheduler* s, int64_t req, const int* prompt, int n_prompt,
                                    const ccinfer_sampling_params* params);
/* ends a request wherever it is; *found = 0 if it is not known (or ended while its last token was read) */
CCINFER_API int ccinfer_cancel(ccinfer_scheduler* s, int64_t req, int* found);
CCINFER_API int ccinfer_has_work(const ccinfer_scheduler* s, int* yes);
/* admits, decides and runs one step; what it produced waits in the event queue */
CCINFER_API int ccinfer_step(ccinfer_scheduler* s);
/* reads the step in flight, if any */
CCINFER_API int ccinfer_drain(ccinfer_scheduler* s);
CCINFER_API int ccinfer_pop_events(ccinfer_scheduler* s, ccinfer_event* out, int capacity, int* n);

#ifdef __cplusplus
}
#endif
#endif
