// Launchers of the device kernels (one declaration per operation; defined in the tl_*.cu files).
#pragma once
#include "tl_common.h"

namespace tl {

// ---------------------------------------------------------------- GEMM
// C[i][j] (+)= alpha * sum_k A(i,k) * B(k,j) (+ bias), i < N, j < M, k < K, per batch b:
//   A(i,k) = A[b*a_bs + i*a_rs + k*a_cs],  B(k,j) = B[b*b_bs + k*b_rs + j*b_cs],
//   C(i,j) = C[b*c_bs + i*c_rs + j*c_cs].
// Accumulation is fp32 for every storage type.
template <class T> struct GemmDesc {
    const T *A = nullptr; const T *B = nullptr; T *C = nullptr;
    int N = 0, M = 0, K = 0;
    long long a_rs = 0, a_cs = 1, b_rs = 0, b_cs = 1, c_rs = 0, c_cs = 1;
    int batch = 1; long long a_bs = 0, b_bs = 0, c_bs = 0;
    float alpha = 1.f;
    bool accumulate = false;        // C += result instead of C = result
    const T *bias = nullptr;        // added after the product
    int bias_mode = 0;              // 1: bias[i] (per row), 2: bias[j] (per column)
};
template <class T> void gemm(const GemmDesc<T> &d);
// Up to three products of one shape whose operands are separate allocations (the q, k, v projections of an attention layer)
// as one launch: `shape` gives sizes, strides, alpha, accumulate and bias_mode; A, B, C and bias come from the list.
template <class T> struct GemmList { const T *A[3]; const T *B[3]; const T *bias[3]; T *C[3]; };
template <class T> void gemm_list(const GemmDesc<T> &shape, const GemmList<T> &l, int count);

// Reference-contract product: C[N x M] = A[N x K] * B, B is [K x M] or (trans_B) [M x K].
template <class T> void mm_contract(const T *A, const T *B, T *C, int N, int K, int M, int trans_B, bool accumulate);

// Batch-1 Linear kernels (HBM-bound): y = W x (+b), dW = dy (x) x, dx = W^T dy.
template <class T> void linear_fw_gemv(const T *W, const T *x, const T *bias, T *y, int out, int in);
template <class T> void linear_wg_outer(const T *dy, const T *x, T *dW, int out, int in);
template <class T> bool linear_wg_streams(Scope &sc, const T *dy, const T *x, T *dW, int n, int out, int in);
template <class T> void linear_ig_gemv(Scope &sc, const T *W, const T *dy, T *dx, int out, int in);
// dW and dX of a batch-1 layer in one launch; false = not covered, nothing launched
template <class T> bool linear_bw_fused(Scope &sc, const T *W, const T *dy, const T *x, T *dW, T *dx, int out, int in);

// ---------------------------------------------------------------- convolution
struct ConvGeom {
    int Cin, Hin, Win, Cout, Hk, Wk, Hout, Wout;
    int sh, sw, padU, padL;
    int n;                 // independent streams
    bool depthwise;        // Cout == Cin, one filter per channel
    bool hwc;              // activations HWC, weights [Cout][Hk][Wk][Cin]
};
template <class T> void conv_fw(Scope &sc, const ConvGeom &g, const T *x, const T *w, const T *bias, T *y);
template <class T> void conv_wg(Scope &sc, const ConvGeom &g, const T *x, const T *dy, T *dw, T *dbias);
template <class T> void conv_ig(Scope &sc, const ConvGeom &g, const T *dy, const T *w, T *dx);
template <class T> void conv_ig_accumulate(Scope &sc, const ConvGeom &g, const T *dy, const T *w, T *dx);   // dx += input gradient
// tensor-core implicit GEMM (tl_conv_tc.cu); false = geometry does not qualify, use the FFMA kernels
// One parity class of a strided input gradient as a stride-1 convolution over dY (see tl_conv_tc.cu)
// One parity class of a strided input gradient.  up = 1 (row-slot kernel only): both column parities of a row parity in one
// launch; accumulator column b holds filter column kw = b and the epilogue writes pixel pairs (see tl_conv_mn.cu).
struct ConvTcClass { int kstep, kh_r, kh_m, kw_r, kw_m, w_Hk, w_Wk; int oH, oW, osy, osx, oy0, ox0; int up; };
bool conv_tc_run(Scope &sc, const float *src, const float *w, const float *bias, float *dst,
                 int n, int C_src, int H_src, int W_src, int C_dst, int H_dst, int W_dst,
                 int Hk, int Wk, int sh, int sw, int padU, int padL, int Cout_w, int Cin_w, bool flip, bool dry_run = false,
                 const ConvTcClass *cls = nullptr);
int conv_tc_status();
#ifdef __CUDACC__
// Fixed-order sum of `groups` partial results (each n floats) for the four consecutive elements i .. i + 3, by a CTA of 1024
// threads = 8 slices x 128 element quads: thread (slice, quad) adds the groups slice, slice + 8, ... with 16-byte loads
// (every load of a thread is independent of the others: the memory system sees them all at once), the eight slice sums
// are then added in slice order.  `used` = false skips the loads of a quad nobody needs.  True in the threads of slice 0
// that hold a result (`t`; components at or past n are zero).  Every kernel that sums weight-gradient partials goes through
// this function, so the immediate and the deferred reductions give the same bits.
static constexpr int PSUM_ELEMS = 512;                  // elements per CTA
__device__ __forceinline__ bool partial_sums_quad(const float *__restrict__ part, long long n, int groups, long long i, bool used, float4 &t, float4 (*sm)[128])
{
    const int q = threadIdx.x & 127, sl = threadIdx.x >> 7;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (used && i < n) {
        if ((n & 3) == 0 && (((uintptr_t)part) & 15) == 0) {
#pragma unroll 4
            for (int g = sl; g < groups; g += 8) {
                const float4 v = __ldcs(reinterpret_cast<const float4 *>(part + (long long)g * n + i));
                acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
        } else {
            for (int g = sl; g < groups; g += 8) {
                const float *src = part + (long long)g * n + i;
                acc.x += src[0];
                if (i + 1 < n) acc.y += src[1];
                if (i + 2 < n) acc.z += src[2];
                if (i + 3 < n) acc.w += src[3];
            }
        }
    }
    sm[sl][q] = acc;
    __syncthreads();
    if (sl != 0 || !used || i >= n) return false;
    t = sm[0][q];
#pragma unroll
    for (int k = 1; k < 8; k++) { const float4 v = sm[k][q]; t.x += v.x; t.y += v.y; t.z += v.z; t.w += v.w; }
    return true;
}
// element e (one of the four of a quad) of the accumulator layout of conv_wgt_kernel -> its place in dW[co][ci][kh][kw], or -1
__device__ __forceinline__ long long wgt_partial_index(long long e, int Cin, int Cout, int s2, int xg, int cigs, int ncopy)
{
    const int NBc = ncopy * Cout;
    const int row = (int)(e / NBc), col = (int)(e % NBc);
    const int grp = row / 8, ci8 = row & 7;                             // row = m * 128 + lane of the accumulator: 16 groups of 8 per M block
    if (grp >= 3 * xg) return -1;                                       // padding rows of the last M block (never written)
    const int a = grp / xg, par = (grp % xg) / cigs, ci = (grp % cigs) * 8 + ci8;
    const int b = col / Cout, co = col % Cout;
    // copy b of the dY row holds dY[x - b + 1], which pairs X[x] with filter column kw = b;
    // stride 2: even pixels with dY[x] are column 1, odd pixels with dY[x] column 2, with dY[x + 1] column 0
    const int kw = !s2 ? b : (par == 0 ? (b == 1 ? 1 : -1) : (b == 1 ? 2 : 0));
    return kw >= 0 ? ((long long)co * Cin + ci) * 9 + a * 3 + kw : -1;
}
#endif

// Partial results of an fp32 reduction: from the deferred-reduction arena when that mode is on and every buffer of the call
// is device-resident (`deferred` = true: the caller notes the sum with defer_*), else scratch of the call (the caller sums at once).
template <class T> inline float *partials_alloc(Scope &sc, size_t floats, bool &deferred)
{
    deferred = false;
    if (sizeof(T) == 4 && sc.may_defer()) {
        float *p = defer_alloc(floats);
        if (p) { deferred = true; return p; }
    }
    return sc.scratch<float>(floats);
}
// 1x1 strided convolutions (tl_conv1x1.cu); false = geometry not covered, nothing launched
bool conv1x1s_fw(const ConvGeom &g, const float *x, const float *w, const float *bias, float *y);
bool conv1x1s_ig(const ConvGeom &g, const float *dy, const float *w, float *dx);   // dX += gradient
bool conv1x1s_wg(const ConvGeom &g, const float *x, const float *dy, float *part, int part_groups, int *groups_out, bool dry_run);
// tensor-core weight gradient (tl_conv_wgt.cu): partial results per CTA into `part`; false = geometry not covered
bool conv_wgt_run(const float *x, const float *dy, float *part, int part_groups, int *groups_out, long long *group_floats_out, int n, int Cin, int Cout, int H,
                  int W, int stride, bool dry_run);
void conv_wgt_reduce(const float *part, float *dw, int groups, int Cin, int Cout, int stride, bool deferred);   // deferred: noted for the batched launch
template <class T> void im2row(const T *src, T *buf, int C, int H, int W, int Hk, int Wk, int Ho, int Wo,
                               int sh, int sw, int padU, int padL, int mode_ig, int hwc, int transposed_buf);
template <class T> void blocktransp(const T *w, T *bt, int Cin, int Cout, int Hk, int Wk, int hwc);

// ---------------------------------------------------------------- elementwise / reductions
enum ActKind { ACT_RELU = 0, ACT_LEAKY = 1, ACT_SIGMOID = 2, ACT_GELU = 3 };
template <class T> void act_fw(int kind, const T *x, T *y, long long n, float slope);
template <class T> void act_bw(int kind, const T *x, const T *y, const T *dy, T *dx, long long n, float slope);
template <class T> void softmax_fw(const T *in, T *out, T *maxes, T *sums, int rows, int width, int batch);
template <class T> void softmax_bw(const T *out, const T *dout, T *din, T *sums, int rows, int width, int batch);
// groups = streams * channels, each of D contiguous elements.
template <class T> void instnorm_fw(const T *x, T *y, const T *gamma_beta, T *mean, T *var, T *stdev,
                                    int n, int C, int D, bool frozen, float eps);
template <class T> void instnorm_bw_input(const T *x, const T *dy, T *dx, const T *gamma, const T *mean,
                                          const T *var, const T *stdev, int n, int C, int D);
template <class T> void instnorm_bw_param(Scope &sc, const T *x, const T *dy, T *dgamma_beta, const T *mean,
                                          const T *stdev, int n, int C, int D);
template <class T> void instnorm_bw_both(Scope &sc, const T *x, const T *dy, T *dx, T *dgamma_beta, const T *gamma, const T *mean,
                                         const T *var, const T *stdev, int n, int C, int D);
// y = relu(norm(x) + skip) in one pass (skip may be null, relu false), and the backward of y = relu(norm(x)) from dL/dy.
template <class T> void instnorm_act_fw(const T *x, T *y, const T *skip, const T *gamma_beta, T *mean, T *var, T *stdev,
                                        int n, int C, int D, bool frozen, float eps, bool relu);
template <class T> void instnorm_relu_bw(Scope &sc, const T *x, const T *y, T *dy, const T *dy2, T *dx, T *dgamma_beta, const T *gamma_beta, const T *mean,
                                         const T *var, const T *stdev, int n, int C, int D);
template <class T> void column_sum(Scope &sc, const T *in, T *out, int n, int dim);    // out[j] = sum_i in[i][j], fixed order
template <class T> void batchnorm_fw(const T *x, T *y, const T *w, const T *b, int n, int B, int C, int HW, float eps);
template <class T> void layernorm_fw(const T *x, T *y, const T *w, const T *b, int rows, int width, float eps);
template <class T> void layernorm_bw(Scope &sc, const T *x, const T *w, const T *dy, T *dx, T *dw, T *db, int rows, int width, float eps);
template <class T> void mse_fw(const T *y, const T *t, T *loss, int dim, int n);
template <class T> void mse_bw(const T *y, const T *t, T *dy, int dim, int n);
template <class T> void ce_fw(const T *z, const T *t, T *loss, int dim, int n);
template <class T> void ce_bw(const T *z, const T *t, T *dz, int dim, int n);
template <class T> void sgd(T *w, T *g, long long n, float lr, float lambda);
template <class T> void add(const T *a, const T *b, T *c, long long n);
template <class T> void copy_n(const T *from, T *to, long long n);
template <class T> void fill(T *to, float v, long long n);
template <class T> void scale(T *x, float s, long long n);
template <class T> void bias_add_rows(T *mat, const T *bias, int H, int W, int per_row);
template <class T> void avgpool_fw(const T *x, T *y, int n, int C, int H, int W, int Ho, int Wo, int Hk, int Wk, int sh, int sw);
template <class T> void avgpool_bw(const T *dy, T *dx, int n, int C, int H, int W, int Ho, int Wo, int Hk, int Wk, int sh, int sw);
template <class T> void transpose_nd(const T *in, T *out, const int *dims, const int *axes, int nd);
template <class T> void broadcast_add(const T *a, const T *b, T *c, const int *da, int na, const int *db, int nb);
template <class T> void pad2d(const T *src, T *dst, int C, int H, int W, int padL, int padR, int padU, int padD, int hwc);
template <class T> void row_max(const T *in, T *maxes, int rows, int width);
template <class T> void exp_sum(const T *in, T *out, const T *maxes, T *sums, int rows, int width);
template <class T> void row_div(T *io, const T *sums, int rows, int width);
template <class T> void mean_std(const T *x, T *mean, T *var, T *stdev, int D, float eps);
// the rest of the element-wise family (tl_family.cu)
template <class T> void l1_fw(const T *y, const T *t, T *loss, int dim, int n, bool berhu, float alpha);
template <class T> void l1_bw(const T *y, const T *t, T *dy, int dim, int n, bool berhu, float alpha);
template <class T> void maxpool_fw(const T *x, T *y, long long planes, int H, int W, int Ho, int Wo, int Hk, int Wk, int Hs, int Ws);
template <class T> void maxpool_bw(const T *x, const T *dy, T *dx, long long planes, int H, int W, int Ho, int Wo, int Hk, int Wk, int Hs, int Ws);
template <class T> void nonorm_fw(const T *x, const T *w, const T *b, T *y, long long rows, int width);
template <class T> void weighted_scaling(const T *x, const T *w, T *y, long long n, float sf, const T *sumsq);
template <class T> void sum_of_squares(const T *x, T *out, long long n);
template <class T> void swiglu(const T *a, const T *b, T *y, long long n);
template <class T> void vec_max(const T *x, T *out, long long n);
template <class T> void vec_exp_sum(const T *x, T *y, T *sum, long long n, float mx);
template <class T> void vector_softmax(const T *x, T *y, long long n);
template <class T> void vec_div(T *io, long long n, float d);
template <class T> void shift_sum(const T *x, const T *maxes, T *y, T *sums, int dim);
template <class T> void sm_bw_op1(const T *A, const T *B, T *S, int H, int W);
template <class T> void sm_bw_op2(const T *A, const T *B, const T *S, T *out, int H, int W);
void cast_h2f(const __half *src, float *dst, long long n);
void cast_f2h(const float *src, __half *dst, long long n);

// ---------------------------------------------------------------- attention
struct MhsaDims { int L, E, F, heads; };
struct MobileBertDims { int L, E, Kb, F, No, heads; };
template <class T> void mhsa_mobilebert_fw(Scope &sc, const MobileBertDims &d, const T *x, const T *xb, const T *wq, const T *wk, const T *wv,
                                           const T *bq, const T *bk, const T *bv, const T *wo, const T *bo,
                                           T *q, T *k, T *v, T *softmax, T *att, T *y);
template <class T> void mhsa_mobilebert_bw(Scope &sc, const MobileBertDims &d, const T *x, const T *xb, const T *wq, const T *wk, const T *wv, const T *wo,
                                           const T *q, const T *k, const T *v, const T *softmax, const T *att, const T *dy,
                                           T *dq, T *dk, T *dv, T *dsoftmax, T *datt, T *dwq, T *dwk, T *dwv, T *dwo, T *dx, T *dxb);
// fused attention core (tl_attn.cu): q, k, v, att are F x L with head h in rows h*H..; P, dP are heads x L x L
bool attn_fused_ok(int L, int H);
template <class T> void attn_fw(const T *q, const T *k, const T *v, T *P, T *att, int L, int H, int heads, float scaling);
template <class T> void attn_bw(const T *datt, const T *q, const T *k, const T *v, const T *P, T *dP, float *rowdot,
                                T *dq, T *dk, T *dv, int L, int H, int heads, float scaling);
template <class T> void mhsa_fw(Scope &sc, const MhsaDims &d, const T *x, const T *wq, const T *wk, const T *wv,
                                const T *bq, const T *bk, const T *bv, const T *wo,
                                T *q, T *k, T *v, T *softmax, T *att, T *y);
template <class T> void mhsa_bw(Scope &sc, const MhsaDims &d, const T *x, const T *wq, const T *wk, const T *wv,
                                const T *wo, const T *q, const T *k, const T *v, const T *softmax, const T *att,
                                const T *dy, T *dq, T *dk, T *dv, T *dsoftmax, T *datt, T *grad_scratch,
                                T *dwq, T *dwk, T *dwv, T *dwo, T *dx);

// ---------------------------------------------------------------- device scalar helpers
__device__ __forceinline__ float ld(const float *p) { return *p; }
__device__ __forceinline__ float ld(const __half *p) { return __half2float(*p); }
__device__ __forceinline__ void st(float *p, float v) { *p = v; }
__device__ __forceinline__ void st(__half *p, float v) { *p = __float2half_rn(v); }

} // namespace tl
