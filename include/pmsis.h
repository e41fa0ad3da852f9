/*
 * pmsis.h - stand-in for the PULP runtime header that code written for PULP-TrainLib
 * includes (lib/include/pulp_train.h:29 of the reference).  It declares the part of
 * the PMSIS surface such code uses; libtrainlib_b200.so defines it.
 *
 * pi_cl_team_fork(n, fn, arg): on PULP this runs fn on n cores, each taking a slice
 * by pi_core_id().  Here a library worker (any exported pulp_* / mm* function) is run
 * ONCE - it performs the whole-tensor operation in one GPU launch - while a
 * user-defined fn is run n times on the host with pi_core_id() = 0..n-1.
 */
#ifndef TRAINLIB_B200_PMSIS_H
#define TRAINLIB_B200_PMSIS_H
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef __cplusplus
extern "C" {
#endif

#ifndef NUM_CORES
#define NUM_CORES 1
#endif
#define PI_L1
#define PI_L2
#define PI_CL_DMA_DIR_EXT2LOC 1
#define PI_CL_DMA_DIR_LOC2EXT 0
/* performance-counter events named by the reference's stats.h (tools/TrainLib_Deployer/deployer_utils/srcfiles/stats.h:57-75);
 * only the two cycle counters have a meaning here, the others read 0 */
#define PI_PERF_CYCLES 0
#define PI_PERF_INSTR  1
#define PI_PERF_LD_STALL 2
#define PI_PERF_JR_STALL 3
#define PI_PERF_IMISS 4
#define PI_PERF_LD 5
#define PI_PERF_ST 6
#define PI_PERF_JUMP 7
#define PI_PERF_BRANCH 8
#define PI_PERF_BTAKEN 9
#define PI_PERF_RVC 10
#define PI_PERF_LD_EXT 12
#define PI_PERF_ST_EXT 13
#define PI_PERF_LD_EXT_CYC 14
#define PI_PERF_ST_EXT_CYC 15
#define PI_PERF_TCDM_CONT 16
#define PI_PERF_ACTIVE_CYCLES 17

#ifndef __CUDACC__
typedef _Float16 float16alt;
typedef _Float16 float16;
typedef short v2s __attribute__((vector_size(4)));
#endif

typedef struct { int dir, merge, stride, length, size, id; uintptr_t ext, loc; } pi_cl_dma_copy_2d_t;
typedef struct { int dir, merge, size, id; uintptr_t ext, loc; } pi_cl_dma_copy_t;
typedef struct { int id; } pi_cl_dma_cmd_t;

int  pi_core_id(void);
void pi_cl_team_fork(int n, void (*fn)(void *), void *arg);
void pi_cl_team_barrier(void);

/* cluster DMA: plain (strided) memcpy between host arrays */
void pi_cl_dma_cmd(uintptr_t ext, uintptr_t loc, int size, int dir, pi_cl_dma_cmd_t *cmd);
void pi_cl_dma_cmd_2d(uintptr_t ext, uintptr_t loc, int size, int stride, int length, int dir, pi_cl_dma_cmd_t *cmd);
void pi_cl_dma_cmd_wait(pi_cl_dma_cmd_t *cmd);

/* performance counters: "cycles" are elapsed nanoseconds on the library's stream */
void pi_perf_conf(unsigned events);
void pi_perf_reset(void);
void pi_perf_start(void);
void pi_perf_stop(void);
unsigned pi_perf_read(int event);

void *pi_l2_malloc(int bytes);
void  pi_l2_free(void *p, int bytes);

/* Cluster bring-up as the reference's main.c files do it (tests/test_conv2d_fp32/main.c:27-46 of the reference):
 * configure, open, send one task, close, exit.  There is no cluster to power up here: opening initialises the CUDA
 * device (non-zero = no device), sending a task calls its entry function once on the calling thread and returns when
 * the GPU work it queued has finished, pmsis_exit ends the process with the given status. */
struct pi_device { void *config; void *data; };
struct pi_cluster_conf { int id; int device_type; };
struct pi_cluster_task { void (*entry)(void *); void *arg; unsigned stack_size, slave_stack_size; };
void pi_cluster_conf_init(struct pi_cluster_conf *conf);
void pi_open_from_conf(struct pi_device *device, void *conf);
int  pi_cluster_open(struct pi_device *device);
int  pi_cluster_close(struct pi_device *device);
struct pi_cluster_task *pi_cluster_task(struct pi_cluster_task *task, void (*entry)(void *), void *arg);
int  pi_cluster_send_task_to_cl(struct pi_device *device, struct pi_cluster_task *task);
void pmsis_exit(int status);

#ifdef __cplusplus
}
#endif
#endif
