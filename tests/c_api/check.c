/* The host core driven from plain C, with no Python in the process: an engine of two cache groups, a
 * scheduler whose run hook takes the pages of every item through ccinfer_reserve / ccinfer_commit and whose
 * read hook makes up tokens, five requests through a pool too small for all of them.  Prints "ok" and exits
 * 0 when the books balance.  Built and run by tests/test_c_api.py. */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "ccinfer.h"

#define CHECK(x)                                                                                     \
  do {                                                                                               \
    int rc_ = (x);                                                                                   \
    if (rc_ != CCINFER_OK) {                                                                         \
      fprintf(stderr, "%s:%d: %s -> %d (%s / %s)\n", __FILE__, __LINE__, #x, rc_, ccinfer_last_error(g_engine), \
              g_sched ? ccinfer_scheduler_last_error(g_sched) : "");                                 \
      return 1;                                                                                      \
    }                                                                                                \
  } while (0)

static ccinfer_engine* g_engine = NULL;
static ccinfer_scheduler* g_sched = NULL;
static int g_last_sampled = 0;   /* sampled items of the step that is in flight */
static long long g_tokens_run = 0;

static int run_hook(void* user, const ccinfer_plan* plan, int64_t ticket) {
  (void)user;
  (void)ticket;
  for (int i = 0; i < plan->n_items; ++i) {
    int rc = ccinfer_reserve(g_engine, plan->reqs[i], plan->counts[i]);
    if (rc != CCINFER_OK) {
      for (int j = 0; j < i; ++j) ccinfer_rollback(g_engine, plan->reqs[j]);
      return rc;
    }
  }
  for (int i = 0; i < plan->n_items; ++i) {
    if (ccinfer_commit(g_engine, plan->reqs[i]) != CCINFER_OK) return CCINFER_INVALID_STATE;
    g_tokens_run += plan->counts[i];
  }
  g_last_sampled = plan->n_sampled;
  return CCINFER_OK;
}

static int read_hook(void* user, int64_t ticket, int n, int* tokens_out) {
  (void)user;
  if (n != g_last_sampled) return CCINFER_INVALID_STATE;
  for (int i = 0; i < n; ++i) tokens_out[i] = (int)((ticket * 31 + i * 7) % 1000);
  return CCINFER_OK;
}

int main(void) {
  ccinfer_group groups[2] = {{0, 4, 14}, {6, 4, 14}};   /* all keys; a window of six */
  ccinfer_options opt = {2, groups, 4, 32, 64};
  CHECK(ccinfer_create(&opt, &g_engine));
  ccinfer_scheduler_options so = {8, 32, 4, 64, -1, 0};
  ccinfer_scheduler_hooks hooks = {NULL, NULL, run_hook, read_hook, NULL};
  CHECK(ccinfer_scheduler_create(g_engine, &so, &hooks, &g_sched));
  int prompt[40];
  for (int i = 0; i < 40; ++i) prompt[i] = i + 1;
  const int lens[5] = {9, 17, 5, 30, 12}, news[5] = {6, 12, 1, 9, 20};
  for (int r = 0; r < 5; ++r) {
    ccinfer_sampling_params sp = {news[r], 0, 1.0f, r % 2 ? 0.7f : 0.0f, (uint64_t)r};
    CHECK(ccinfer_add_request(g_sched, 100 + r, prompt, lens[r], &sp));
  }
  if (ccinfer_add_request(g_sched, 100, prompt, 3, &(ccinfer_sampling_params){1, 0, 1.0f, 0.0f, 0}) != CCINFER_INVALID_ARGUMENT) {
    fprintf(stderr, "a second request 100 was not refused\n");
    return 1;
  }
  int produced[5] = {0, 0, 0, 0, 0}, finished = 0, yes = 1, guard = 0;
  while (yes) {
    CHECK(ccinfer_step(g_sched));
    ccinfer_event ev[16];
    int n = 0;
    do {
      CHECK(ccinfer_pop_events(g_sched, ev, 16, &n));
      for (int i = 0; i < n; ++i) {
        const int r = (int)(ev[i].req - 100);
        if (r < 0 || r > 4) return 1;
        if (ev[i].token >= 0) produced[r] += 1;
        if (ev[i].finished) {
          finished += 1;
          if (ev[i].reason != CCINFER_REASON_MAX_TOKENS) return 1;
        }
      }
    } while (n == 16);
    CHECK(ccinfer_check(g_engine));
    CHECK(ccinfer_has_work(g_sched, &yes));
    if (++guard > 2000) {
      fprintf(stderr, "the scheduler does not come to an end\n");
      return 1;
    }
  }
  ccinfer_scheduler_stats_t st;
  ccinfer_stats_t es;
  CHECK(ccinfer_scheduler_stats(g_sched, &st));
  CHECK(ccinfer_stats(g_engine, &es));
  for (int r = 0; r < 5; ++r)
    if (produced[r] != news[r]) {
      fprintf(stderr, "request %d produced %d of %d tokens\n", r, produced[r], news[r]);
      return 1;
    }
  if (finished != 5 || es.seqs != 0 || es.slots_free != 4 || es.pages_free[0] != 14 || es.pages_free[1] != 14 ||
      st.active != 0 || st.waiting != 0) {
    fprintf(stderr, "something is left: finished %d, sequences %d, slots %d, pages %d / %d\n", finished, es.seqs,
            es.slots_free, es.pages_free[0], es.pages_free[1]);
    return 1;
  }
  printf("ok steps %lld preemptions %lld tokens %lld high water %d / %d\n", st.steps, st.preemptions, g_tokens_run,
         es.pages_high_water[0], es.pages_high_water[1]);
  ccinfer_scheduler_destroy(g_sched);
  ccinfer_destroy(g_engine);
  return 0;
}
