/*
 * trainlib_b200.h - entry points of libtrainlib_b200.so that have no counterpart in
 * the reference library: device/memory management, error reporting, the batched
 * "streams" mode and timing.  Plain C ABI: pointers, sizes and ints only.
 */
#ifndef TRAINLIB_B200_H
#define TRAINLIB_B200_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- error state.  The reference reports errors with printf + return
 * (e.g. lib/sources/pulp_im2col_fp32.c:125-127); entry points here do the same and
 * also latch a code that the caller can read.  CUDA errors are sticky. */
enum {
    TL_OK = 0,
    TL_ERR_NO_DEVICE = 1,      /* no CUDA device / driver: there is no CPU fallback */
    TL_ERR_CUDA = 2,           /* a CUDA runtime call failed */
    TL_ERR_BAD_ARGS = 3,       /* inconsistent sizes, unsupported flag combination */
    TL_ERR_UNSUPPORTED = 4,    /* a branch the reference itself leaves unimplemented */
    TL_ERR_TOO_LARGE = 5,      /* request exceeds a fixed capacity */
    TL_ERR_TIMEOUT = 6,        /* a bounded device-side wait gave up: the kernel returned early, its output is invalid */
    TL_ERR_NO_MEMORY = 7       /* a device or pinned allocation failed; clearable, nothing else is affected */
};
int         trainlib_last_error(void);
const char *trainlib_last_error_string(void);
void        trainlib_clear_error(void);

/* ---- device.  One host thread drives one device; all work is queued on one stream,
 * so call order is execution order.  trainlib_init is implicit in every entry point. */
int   trainlib_init(int device);              /* returns TL_OK or an error code */
int   trainlib_device(void);
void  trainlib_set_stream(void *cuda_stream); /* NULL = the library's own stream */
void *trainlib_stream(void);
void  trainlib_synchronize(void);

/* ---- memory modes.  The reference's tensors are host arrays handed over through
 * struct blob.  Each pointer reaching an entry point is either
 *   - a device address (from trainlib_malloc, cudaMalloc or a torch CUDA tensor):
 *     used in place, nothing is copied, the call returns without synchronising; or
 *   - a host address: the bytes the call reads are copied to a device staging arena
 *     first, the bytes it writes are copied back before the call returns.
 * TL_MEM_AUTO asks the driver per pointer; TL_MEM_DEVICE / TL_MEM_HOST assert that all
 * pointers are of one kind and skip the query. */
enum { TL_MEM_AUTO = 0, TL_MEM_DEVICE = 1, TL_MEM_HOST = 2 };
void  trainlib_set_memory_mode(int mode);
int   trainlib_memory_mode(void);
void *trainlib_malloc(size_t bytes);          /* device memory, 256-byte aligned */
void  trainlib_free(void *dev_ptr);
void *trainlib_malloc_host(size_t bytes);     /* pinned host memory (fast staging) */
void  trainlib_free_host(void *host_ptr);
int   trainlib_memcpy_h2d(void *dev, const void *host, size_t bytes);
int   trainlib_memcpy_d2h(void *host, const void *dev, size_t bytes);
int   trainlib_memset(void *dev, int byte, size_t bytes);
/* Upload that overlaps the kernels already queued: for an input that the caller keeps in two device buffers
 * (slot 0 / 1, alternating).  The copy runs on a second stream after the work marked with
 * trainlib_mark_consumed(slot) has finished; everything queued on the library's stream after this call sees the
 * new data.  `host` should be pinned (trainlib_malloc_host), otherwise the copy is synchronous. */
int   trainlib_memcpy_h2d_overlapped(void *dev, const void *host, size_t bytes, int slot);
int   trainlib_mark_consumed(int slot);      /* "all work queued so far is the last reader of buffer `slot`" */

/* ---- streams mode.  With n > 1, every activation blob (input, output, and their
 * diffs) holds n independent batch-1 tensors back to back ([n][blob.dim]); weight
 * blobs stay single and weight gradients are the sum over the n streams, taken in
 * stream order inside one launch.  Losses write n values.  n = 1 is the reference's
 * behaviour.  Applies to conv2d, linear, instnorm/batchnorm, relu, residual,
 * avgpool, CrossEntropy/MSE and the SGD step. */
void  trainlib_set_streams(int n);
int   trainlib_streams(void);

/* ---- timing on the library's stream (CUDA events).  pi_perf_* map onto these. */
void   trainlib_timer_start(void);
double trainlib_timer_stop_ms(void);          /* synchronises; elapsed milliseconds */
long long trainlib_kernel_launches(void);     /* kernels launched by this library so far */

/* ---- per-kernel timing.  While on, every kernel launch is bracketed by CUDA events on the
 * library's stream; entries are keyed by kernel name.  Adds launch overhead: use it for a
 * profiling step, not inside a timed region. */
void        trainlib_profile(int on);          /* 1 = clear and start, 0 = stop */
int         trainlib_profile_entries(void);
const char *trainlib_profile_entry(int i, long long *launches, double *total_ms);
/* useful floating-point operations the convolution kernels of entry i were launched for (2 per multiply-add of the
 * operator's definition, full windows at the borders, no credit for zeros a kernel inserts); 0 for other kernels */
double      trainlib_profile_entry_flops(int i);

/* ---- layer norm and GELU beyond the reference, which has an fp32 layer-norm forward and GELU forwards only
 * [ref: lib/include/pulp_layernorm_fp32.h:26-34, lib/sources/pulp_act_fp32.c:714].  The first seven fields are
 * those of LayerNorm_args_fp32, so the same object also serves pulp_layerNorm_fp32_fw_cl.  Pointers are float * for
 * the fp32 entry points and fp16 * for the fp16 ones; eps points at one value of that type.  Backward: derivative of
 * the reference's forward formula; dx, dweight, dbias are written (not accumulated).  GELU backward: derivative of
 * the reference's rational tanh approximation, input.diff = output.diff * gelu'(input.data). */
struct trainlib_layernorm_args {
    void *x; void *weight; void *bias; void *output; void *eps; int size; int step_size;
    void *dy; void *dx; void *dweight; void *dbias;
};
void  trainlib_layernorm_fp16_fw_cl(void *trainlib_layernorm_args);
void  trainlib_layernorm_fp32_bw_cl(void *trainlib_layernorm_args);
void  trainlib_layernorm_fp16_bw_cl(void *trainlib_layernorm_args);
void  trainlib_gelu_fp32_bw_cl(void *act_args);
void  trainlib_gelu_fp16_bw_cl(void *act_args_fp16);

/* ---- Instance norm fused with what follows it in a residual network.  No counterpart in the reference, which runs
 * pulp_instnorm_*_fw_cl, pulp_residualconn_*_fw and pulp_relu_*_fw_cl one after the other
 * (lib/sources/pulp_instnorm_fp32.c:27, pulp_residual_fp32.c:26, pulp_act_fp32.c:83); results are those of that sequence,
 * bit for bit.  `norm` points at an InstNorm_args (fp32 entry points) or InstNorm_args_fp16.
 *   fw:  norm->output->data = relu(instnorm(norm->input->data) + skip->data); `skip` (a struct blob / blob_fp16 of the
 *        output's size) may be NULL and `relu` 0.  The running statistics are written as by the plain forward.
 *   bw:  norm->output->diff holds the gradient behind the ReLU (relu != 0, skip == NULL only): writes norm->input->diff
 *        and norm->coeff->diff like pulp_instnorm_*_bw_cl after pulp_relu_*_bw_cl.  norm->output->diff may be masked in
 *        place.  With a skip connection the ReLU's gradient has two readers, so mask it once with pulp_relu_*_bw_cl on the
 *        sum and call pulp_instnorm_*_bw_cl.
 *        `diff2` (backward only; NULL or an array of the output's size and type): the gradient that a second reader of the
 *        output left, e.g. an identity shortcut; it is added to norm->output->diff first, as pulp_sumnode_*_bw would
 *        (lib/sources/pulp_residual_fp32.c:59), without writing the sum back. */
struct trainlib_instnorm_act_args { void *norm; void *skip; int relu; void *diff2; };
void  trainlib_instnorm_act_fp32_fw_cl(void *trainlib_instnorm_act_args);
void  trainlib_instnorm_act_fp16_fw_cl(void *trainlib_instnorm_act_args);
void  trainlib_instnorm_act_fp32_bw_cl(void *trainlib_instnorm_act_args);
void  trainlib_instnorm_act_fp16_bw_cl(void *trainlib_instnorm_act_args);

/* ---- Input gradient of Conv2D added to what input->diff already holds (CHW only).  No counterpart in the reference, where a
 * shortcut convolution writes its input gradient to a buffer of its own and pulp_sumnode_*_bw adds it to the gradient of
 * the main branch (lib/sources/pulp_conv2d_fp32.c:454, pulp_residual_fp32.c:59); the values are those of that pair of calls.
 * A 1x1 strided convolution adds its samples in place and touches nothing between them. */
void  trainlib_conv2d_fp32_bw_input_grads_acc_cl(void *Conv2D_args);
void  trainlib_conv2d_fp16_bw_input_grads_acc_cl(void *Conv2D_args_fp16);

/* ---- Deferred reductions (off by default).  Weight gradients and norm-parameter gradients are produced as partial results
 * and then summed by a small kernel per call; a network of thousands of streams issues two dozen such sums per backward
 * pass.  While the mode is on, device-resident calls keep their partial results in a library-owned arena and the library
 * runs ALL pending sums as ONE launch when pulp_gradient_descent_*, trainlib_synchronize, trainlib_memcpy_d2h,
 * trainlib_timer_stop_ms, trainlib_graph_begin/_end or trainlib_set_stream is called, when the mode is switched off, or
 * on trainlib_flush_reductions().  Until then the gradient buffers of the deferred calls do not hold their values: flush
 * before anything outside the library (a collective, a kernel of your own, a cudaMemcpy) reads a gradient.  The values
 * are those of the immediate mode (same summation trees).  The arena is sized at a flush from what the calls since the
 * previous flush asked for: the first pass of a workload in this mode still sums at once, and so does any call whose
 * partial results do not fit (after a graph capture the arena is never moved again). */
void  trainlib_set_deferred_reductions(int on);
void  trainlib_flush_reductions(void);

/* ---- CUDA graphs.  Entry-point calls made between begin and end are recorded instead of executed (device pointers
 * only: a host pointer would need a synchronous copy); the handle replays them with one launch on the library's
 * stream.  The recorded launches keep the addresses they saw, including library scratch: run the same calls once
 * before capturing so that the scratch arena has its final size; it is never shrunk or moved afterwards.
 * trainlib_kernel_launches() advances by the number of recorded kernels on every replay. */
int   trainlib_graph_begin(void);
void *trainlib_graph_end(void);               /* NULL on failure (see trainlib_last_error) */
int   trainlib_graph_launch(void *graph);
void  trainlib_graph_destroy(void *graph);

/* ---- GEMM path selection for diagnostics and profiling.
 * 0 = automatic, 1 = force FFMA SIMT tiles, 2 = force the tcgen05 kernels whose operands are staged by threads
 * (convolutions: the tensor-core kernel at every size), 3 = force the TMA-fed tcgen05 GEMM for the mm family,
 * 4 = convolutions take the tensor-core kernel that builds its A operand in tensor memory also where the
 * row-slot kernel (operands read in place from the TMA-written rows) would qualify. */
void  trainlib_set_gemm_path(int path);
/* 0 while every tensor-core kernel so far finished normally; otherwise the id of the bounded
 * device-side wait that gave up (the kernel then returned early and its output is invalid). */
int   trainlib_tc_status(void);
int   trainlib_gemm_path(void);

/* ---- Linear input gradient for callers that must not allocate.  No counterpart in the reference
 * (it is a variant of pulp_linear_fp32_bw_input_grads_cl with plain arguments).
 * dx[in] = W[out x in]^T dy[out], all three DEVICE pointers; the kernels run on `cuda_stream`
 * (NULL = the default stream) and the call returns without synchronising.
 * Who needs it: hosts that gave the whole device to their own memory pool, loops with a memory budget
 * fixed at start-up, callers that cannot take the device-wide stall an allocation may cause.  The call
 * performs no cudaMalloc/cudaFree and uses no allocating library routine; its scratch is a fixed 4 MiB
 * array inside the library image (held by every GPU that loads the library until the process exits).
 * Limits and rules:
 *   - `in` may be at most 1 048 576; larger layers are refused with TL_ERR_TOO_LARGE (nothing runs);
 *   - the first call on a device looks up the array's device address; make that first call before
 *     starting any stream capture;
 *   - all calls share the one array: calls that overlap on the GPU (different streams) race, serialise them;
 *   - the array keeps the last call's partial sums; each call overwrites every entry it reads.
 * Returns TL_OK or the error code it also latches. */
int trainlib_linear_fp32_bw_input_grads_noalloc(const float *W, const float *dy, float *dx, int out, int in, void *cuda_stream);

#ifdef __cplusplus
}
#endif
#endif /* TRAINLIB_B200_H */
