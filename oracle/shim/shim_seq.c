/* Sequential team API: every "core" runs in turn on the caller's thread.
 * Results do not depend on NUM_CORES because the reference's static partitioning
 * never changes a per-output accumulation order.  TEST INFRASTRUCTURE ONLY. */
#include "pmsis.h"
__thread int oracle_shim_core_id = 0;
void pi_cl_team_fork(int n, void (*fn)(void *), void *arg)
{
    int outer = oracle_shim_core_id;
    if (outer != 0) { fn(arg); return; }          /* nested fork: run inline on this core */
    for (int i = 0; i < n; i++) { oracle_shim_core_id = i; fn(arg); }
    oracle_shim_core_id = 0;
}
void pi_cl_team_barrier(void) {}
#include "shim_common.inc"
