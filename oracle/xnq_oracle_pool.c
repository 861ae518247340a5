/*
 * A small persistent worker pool for the CPU oracle / timed CPU baseline. TEST INFRASTRUCTURE ONLY.
 * Stands in for xn-core/src/threadpool.rs: workers spin for a while on a generation counter, then
 * park on a condition variable; the publisher takes part as participant 0 and joins at the end.
 */
#include "xnq_oracle.h"
#include "xnq_oracle_internal.h"

#include <pthread.h>
#include <stdatomic.h>
#include <stdlib.h>
#include <unistd.h>

#define MAX_WORKERS 255
#define SPIN_BUDGET 20000

static pthread_mutex_t g_run_lock = PTHREAD_MUTEX_INITIALIZER; /* one job at a time */
static pthread_mutex_t g_mu = PTHREAD_MUTEX_INITIALIZER;
static pthread_cond_t g_cv = PTHREAD_COND_INITIALIZER;
static pthread_t g_threads[MAX_WORKERS];
static int g_nworkers = 0;
static atomic_uint g_generation;
static atomic_int g_pending;
static xnqo_pool_fn g_fn;
static void *g_arg;
static int g_nth;

static void *worker_main(void *p) {
  const int id = (int)(intptr_t)p; /* participant index id+1 */
  unsigned seen = 0;
  for (;;) {
    unsigned gen = atomic_load_explicit(&g_generation, memory_order_acquire);
    int spins = 0;
    while (gen == seen) {
      if (++spins > SPIN_BUDGET) {
        pthread_mutex_lock(&g_mu);
        while ((gen = atomic_load_explicit(&g_generation, memory_order_acquire)) == seen) pthread_cond_wait(&g_cv, &g_mu);
        pthread_mutex_unlock(&g_mu);
        break;
      }
      __builtin_ia32_pause();
      gen = atomic_load_explicit(&g_generation, memory_order_acquire);
    }
    seen = gen;
    if (id + 1 < g_nth) {
      g_fn(id + 1, g_nth, g_arg);
      atomic_fetch_sub_explicit(&g_pending, 1, memory_order_acq_rel);
    }
  }
  return NULL;
}

int xnqo_hw_threads(void) {
  long n = sysconf(_SC_NPROCESSORS_ONLN);
  return n < 1 ? 1 : (int)n;
}

void xnqo_pool_run(xnqo_pool_fn fn, void *arg, int nth) {
  if (nth <= 0) nth = xnqo_hw_threads();
  if (nth > MAX_WORKERS + 1) nth = MAX_WORKERS + 1;
  if (nth == 1) {
    fn(0, 1, arg);
    return;
  }
  pthread_mutex_lock(&g_run_lock);
  while (g_nworkers < nth - 1) {
    if (pthread_create(&g_threads[g_nworkers], NULL, worker_main, (void *)(intptr_t)g_nworkers) != 0) break;
    g_nworkers++;
  }
  if (nth > g_nworkers + 1) nth = g_nworkers + 1;
  g_fn = fn;
  g_arg = arg;
  g_nth = nth;
  atomic_store_explicit(&g_pending, nth - 1, memory_order_release);
  pthread_mutex_lock(&g_mu);
  atomic_fetch_add_explicit(&g_generation, 1, memory_order_acq_rel);
  pthread_cond_broadcast(&g_cv);
  pthread_mutex_unlock(&g_mu);
  fn(0, nth, arg);
  while (atomic_load_explicit(&g_pending, memory_order_acquire) > 0) __builtin_ia32_pause();
  pthread_mutex_unlock(&g_run_lock);
}
