/* Threaded team API for the timed CPU baseline: a persistent pool of
 * NUM_CORES-1 workers plus the caller, released and joined through two
 * barriers per fork; pi_cl_team_barrier is a third, real barrier because
 * mm_manager synchronises inside a forked region
 * (lib/sources/pulp_train_utils_fp32.c:1673).  TEST INFRASTRUCTURE ONLY. */
#define _GNU_SOURCE
#include "pmsis.h"
#include <pthread.h>

__thread int oracle_shim_core_id = 0;

static pthread_barrier_t g_go, g_done, g_team;
static pthread_t g_threads[256];
static int g_pool = 0;
static void (*volatile g_fn)(void *);
static void *volatile g_arg;
static volatile int g_quit = 0;
static volatile int g_active = 0;      /* a fork is in flight: forks issued from inside it run inline */

static void *pool_main(void *p)
{
    oracle_shim_core_id = (int)(intptr_t)p;
    for (;;) {
        pthread_barrier_wait(&g_go);
        if (g_quit) return NULL;
        g_fn(g_arg);
        pthread_barrier_wait(&g_done);
    }
}

static void pool_start(int n)
{
    pthread_barrier_init(&g_go, NULL, (unsigned)n);
    pthread_barrier_init(&g_done, NULL, (unsigned)n);
    pthread_barrier_init(&g_team, NULL, (unsigned)n);
    for (int i = 1; i < n; i++) pthread_create(&g_threads[i], NULL, pool_main, (void *)(intptr_t)i);
    g_pool = n;
}

void pi_cl_team_fork(int n, void (*fn)(void *), void *arg)
{
    if (oracle_shim_core_id != 0 || g_active || n <= 1) { fn(arg); return; }   /* nested or single core */
    if (g_pool == 0) pool_start(n);
    if (g_pool != n) {                          /* pool is sized once; other widths run in turn */
        for (int i = 0; i < n; i++) { oracle_shim_core_id = i; fn(arg); }
        oracle_shim_core_id = 0;
        return;
    }
    g_fn = fn; g_arg = arg; g_active = 1;
    pthread_barrier_wait(&g_go);
    fn(arg);
    pthread_barrier_wait(&g_done);
    g_active = 0;
}

void pi_cl_team_barrier(void)
{
    if (g_pool > 1) pthread_barrier_wait(&g_team);
}
#include "shim_common.inc"
