/*
 * Host stand-in for the PULP "pmsis.h" runtime header.  TEST INFRASTRUCTURE ONLY:
 * it exists so that the reference library's C sources (lib/sources/*.c, which
 * include "pmsis.h" through lib/include/pulp_train.h:29) compile unmodified with
 * gcc on x86-64 and can serve as the checker and the timed CPU baseline.
 *
 * Two implementations of the team API live beside this header:
 *   shim_seq.c - pi_cl_team_fork runs the worker NUM_CORES times, one core id
 *                after the other, on the calling thread (bit-reproducible checker);
 *   shim_mt.c  - a persistent pthread pool with a real barrier (timed baseline).
 */
#ifndef ORACLE_PMSIS_SHIM_H
#define ORACLE_PMSIS_SHIM_H
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>

#ifndef NUM_CORES
#define NUM_CORES 1
#endif

/* lib/include/pulp_train_defines.h:32 typedefs fp16 from float16alt (bfloat16 on
 * PULP).  IEEE binary16 is the default here; -DSHIM_BF16 selects bfloat16. */
#ifdef SHIM_BF16
typedef __bf16 float16alt;
#else
typedef _Float16 float16alt;
#endif
typedef _Float16 float16;
typedef short v2s __attribute__((vector_size(4)));

#define PI_L1
#define PI_L2
#define PI_CL_DMA_DIR_EXT2LOC 1
#define PI_CL_DMA_DIR_LOC2EXT 0

typedef struct { int dir, merge, stride, length, size, id; uintptr_t ext, loc; } pi_cl_dma_copy_2d_t;
typedef struct { int dir, merge, size, id; uintptr_t ext, loc; } pi_cl_dma_copy_t;
typedef struct { int id; } pi_cl_dma_cmd_t;
typedef struct { int id; } pi_cl_fs_req_t;
typedef struct { int id; } pi_fs_file_t;

extern __thread int oracle_shim_core_id;
static inline int pi_core_id(void) { return oracle_shim_core_id; }

void pi_cl_team_fork(int n, void (*fn)(void *), void *arg);
void pi_cl_team_barrier(void);

/* DMA paths of the reference cast pointers to uint32_t and cannot run on a
 * 64-bit host; these exist only so that the sources link. */
void pi_cl_dma_memcpy_2d(pi_cl_dma_copy_2d_t *c);
void pi_cl_dma_memcpy(pi_cl_dma_copy_t *c);
void pi_cl_dma_wait(void *c);
void pi_cl_dma_cmd_2d(uintptr_t ext, uintptr_t loc, int size, int stride, int length, int dir, pi_cl_dma_cmd_t *c);
void pi_cl_dma_cmd(uintptr_t ext, uintptr_t loc, int size, int dir, pi_cl_dma_cmd_t *c);
void pi_cl_dma_cmd_wait(pi_cl_dma_cmd_t *c);
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
void pi_perf_conf(unsigned events);
void pi_perf_reset(void);
void pi_perf_start(void);
void pi_perf_stop(void);
unsigned pi_perf_read(int event);
/* cluster bring-up of the reference's main.c files: the task's entry function is called once */
struct pi_device { void *config; void *data; };
struct pi_cluster_conf { int id; int device_type; };
struct pi_cluster_task { void (*entry)(void *); void *arg; int stack_size; int slave_stack_size; };
void pi_cluster_conf_init(struct pi_cluster_conf *conf);
void pi_open_from_conf(struct pi_device *device, void *conf);
int  pi_cluster_open(struct pi_device *device);
int  pi_cluster_close(struct pi_device *device);
struct pi_cluster_task *pi_cluster_task(struct pi_cluster_task *task, void (*entry)(void *), void *arg);
int  pi_cluster_send_task_to_cl(struct pi_device *device, struct pi_cluster_task *task);
void pmsis_exit(int code);
void *pi_l2_malloc(int n);
void pi_l2_free(void *p, int n);
void pi_cl_fs_read(pi_fs_file_t *f, void *b, int n, pi_cl_fs_req_t *r);
void pi_cl_fs_wait(pi_cl_fs_req_t *r);
void pi_cl_fs_copy(pi_fs_file_t *f, uint32_t o, void *b, int n, int d, pi_cl_fs_req_t *r);
#endif
