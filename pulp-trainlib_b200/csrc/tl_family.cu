// The rest of the bandwidth-bound family around the training step: L1 and berHu losses, max pooling, NoNorm,
// RMS norm and its two pieces, SwiGLU, and the per-row pieces the reference's softmax is assembled from.
// One stream's tensor per CTA row where a reduction is involved (fixed summation order), grid-stride elsewhere.
#include "tl_kernels.h"
#include "tl_reduce.cuh"

namespace tl {

static inline int fam_grid(long long n, int per_block = 256, int waves = 16)
{
    long long b = (n + per_block - 1) / per_block;
    long long cap = (long long)sm_count() * waves;
    if (b > cap) b = cap;
    return (int)(b < 1 ? 1 : b);
}
#define FAM_STRIDE(i, n) for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (n); i += (long long)gridDim.x * blockDim.x)

// ------------------------------------------------------------------ L1 and berHu losses
// L1: loss = sum_i (1/dim) |t_i - y_i|; dy_i = sign(y_i - t_i) / dim   [ref: lib/sources/pulp_losses_fp32.c:140-210]
// berHu: c = alpha * max_i |y_i - t_i|; term = |d| below c, (d^2 - c^2) / (2c) from c on; loss = (sum term) / dim;
// dy = sign(d) / dim below c, d / (dim c) from c on   [ref: lib/sources/pulp_losses_fp32.c:281-365]
template <class T, bool BERHU>
__global__ void __launch_bounds__(256) l1_fw_kernel(const T *__restrict__ y, const T *__restrict__ t, T *__restrict__ loss, int dim, float alpha)
{
    __shared__ float red[33];
    const T *yp = y + (long long)blockIdx.x * dim, *tp = t + (long long)blockIdx.x * dim;
    const float meanval = 1.0f / (float)dim;
    float s = 0.f;
    if (!BERHU) {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) s += __fmul_rn(meanval, fabsf(__fsub_rn(ld(tp + i), ld(yp + i))));
        s = block_sum(s, red);
    } else {
        float c = 0.f;
        for (int i = threadIdx.x; i < dim; i += blockDim.x) c = fmaxf(c, fabsf(__fsub_rn(ld(yp + i), ld(tp + i))));
        c = __fmul_rn(alpha, block_max(c, red));
        for (int i = threadIdx.x; i < dim; i += blockDim.x) {
            const float v = fabsf(__fsub_rn(ld(yp + i), ld(tp + i)));
            s += (v < c) ? v : __fdiv_rn(__fsub_rn(__fmul_rn(v, v), __fmul_rn(c, c)), __fmul_rn(2.f, c));
        }
        s = __fmul_rn(block_sum(s, red), meanval);
    }
    if (threadIdx.x == 0) st(loss + blockIdx.x, s);
}
template <class T, bool BERHU>
__global__ void __launch_bounds__(256) l1_bw_kernel(const T *__restrict__ y, const T *__restrict__ t, T *__restrict__ dy, int dim, float alpha)
{
    __shared__ float red[33];
    const long long base = (long long)blockIdx.x * dim;
    const float meanval = 1.0f / (float)dim;
    float c = 0.f;
    if (BERHU) {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) c = fmaxf(c, fabsf(__fsub_rn(ld(y + base + i), ld(t + base + i))));
        c = __fmul_rn(alpha, block_max(c, red));
    }
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
        const float d = __fsub_rn(ld(y + base + i), ld(t + base + i));
        float g = d > 0.f ? meanval : (d == 0.f ? 0.f : -meanval);
        if (BERHU && !(fabsf(d) < c)) g = __fdiv_rn(__fmul_rn(meanval, d), c);
        st(dy + base + i, g);
    }
}
template <class T> void l1_fw(const T *y, const T *t, T *loss, int dim, int n, bool berhu, float alpha)
{
    if (n <= 0) return;
    if (berhu) TL_LAUNCH((l1_fw_kernel<T, true>), n, 256, 0, y, t, loss, dim, alpha);
    else TL_LAUNCH((l1_fw_kernel<T, false>), n, 256, 0, y, t, loss, dim, alpha);
}
template <class T> void l1_bw(const T *y, const T *t, T *dy, int dim, int n, bool berhu, float alpha)
{
    if (n <= 0) return;
    if (berhu) TL_LAUNCH((l1_bw_kernel<T, true>), n, 256, 0, y, t, dy, dim, alpha);
    else TL_LAUNCH((l1_bw_kernel<T, false>), n, 256, 0, y, t, dy, dim, alpha);
}

// ------------------------------------------------------------------ max pooling
// Forward: the window maximum.  Backward: the gradient of an output pixel goes to the FIRST window position (row-major
// scan, strict >) that holds the maximum; windows may overlap, so every input pixel gathers from the windows that
// cover it, in window order  [ref: lib/sources/pulp_pooling_fp32.c:123-237].
template <class T>
__global__ void maxpool_fw_kernel(const T *__restrict__ x, T *__restrict__ y, long long total, int H, int W, int Ho, int Wo,
                                  int Hk, int Wk, int Hs, int Ws)
{
    FAM_STRIDE(i, total) {
        const int wo = (int)(i % Wo), ho = (int)((i / Wo) % Ho);
        const long long plane = i / ((long long)Wo * Ho);
        const T *p = x + plane * H * W + (long long)ho * Hs * W + (long long)wo * Ws;
        float m = ld(p);
        for (int a = 0; a < Hk; a++)
            for (int b = 0; b < Wk; b++) m = fmaxf(m, ld(p + a * W + b));
        st(y + i, m);
    }
}
template <class T>
__global__ void maxpool_bw_kernel(const T *__restrict__ x, const T *__restrict__ dy, T *__restrict__ dx, long long total, int H, int W,
                                  int Ho, int Wo, int Hk, int Wk, int Hs, int Ws)
{
    FAM_STRIDE(i, total) {
        const int w = (int)(i % W), h = (int)((i / W) % H);
        const long long plane = i / ((long long)W * H);
        const T *xp = x + plane * H * W;
        const float mine = ld(xp + h * W + w);
        // windows (ho, wo) with ho*Hs <= h < ho*Hs + Hk
        int ho_lo = h - Hk + 1; ho_lo = ho_lo <= 0 ? 0 : (ho_lo + Hs - 1) / Hs;
        int wo_lo = w - Wk + 1; wo_lo = wo_lo <= 0 ? 0 : (wo_lo + Ws - 1) / Ws;
        const int ho_hi = min(Ho - 1, h / Hs), wo_hi = min(Wo - 1, w / Ws);
        float acc = 0.f;
        for (int ho = ho_lo; ho <= ho_hi; ho++)
            for (int wo = wo_lo; wo <= wo_hi; wo++) {
                const T *p = xp + (long long)ho * Hs * W + (long long)wo * Ws;
                const int ra = h - ho * Hs, rb = w - wo * Ws;            // my place in the window
                bool first_max = true;
                for (int a = 0; a < Hk && first_max; a++)
                    for (int b = 0; b < Wk; b++) {
                        const float v = ld(p + a * W + b);
                        const bool before = a < ra || (a == ra && b < rb);
                        if (before ? (v >= mine) : (v > mine)) { first_max = false; break; }   // an earlier equal value wins
                    }
                if (first_max) acc = __fadd_rn(acc, ld(dy + plane * Ho * Wo + (long long)ho * Wo + wo));
            }
        st(dx + i, acc);
    }
}
template <class T> void maxpool_fw(const T *x, T *y, long long planes, int H, int W, int Ho, int Wo, int Hk, int Wk, int Hs, int Ws)
{
    const long long total = planes * Ho * Wo;
    if (total > 0) TL_LAUNCH((maxpool_fw_kernel<T>), fam_grid(total), 256, 0, x, y, total, H, W, Ho, Wo, Hk, Wk, Hs, Ws);
}
template <class T> void maxpool_bw(const T *x, const T *dy, T *dx, long long planes, int H, int W, int Ho, int Wo, int Hk, int Wk, int Hs, int Ws)
{
    const long long total = planes * H * W;
    if (total > 0) TL_LAUNCH((maxpool_bw_kernel<T>), fam_grid(total), 256, 0, x, dy, dx, total, H, W, Ho, Wo, Hk, Wk, Hs, Ws);
}

// ------------------------------------------------------------------ NoNorm, weighted scaling, SwiGLU
// NoNorm: out[i][j] = in[i][j] * coeff[j] + bias[j]   [ref: lib/sources/pulp_nonorm_fp32.c:30-58]
template <class T>
__global__ void nonorm_kernel(const T *__restrict__ x, const T *__restrict__ w, const T *__restrict__ b, T *__restrict__ y, long long total, int width)
{
    FAM_STRIDE(i, total) { const int j = (int)(i % width); st(y + i, __fadd_rn(__fmul_rn(ld(x + i), ld(w + j)), ld(b + j))); }
}
template <class T> void nonorm_fw(const T *x, const T *w, const T *b, T *y, long long rows, int width)
{
    const long long total = rows * width;
    if (total > 0) TL_LAUNCH((nonorm_kernel<T>), fam_grid(total), 256, 0, x, w, b, y, total, width);
}
// out[i] = w[i] * (sf * in[i]); sf is a value, or (RMS norm) derived on the device from a sum of squares:
// sf = 1 / sqrt(sum / size + 1e-5)   [ref: lib/sources/pulp_rmsnorm_fp32.c:29-60]
template <class T>
__global__ void weighted_scaling_kernel(const T *__restrict__ x, const T *__restrict__ w, T *__restrict__ y, long long n, float sf, const T *__restrict__ sumsq)
{
    if (sumsq) {
        float ss = __fdiv_rn(ld(sumsq), (float)n);
        ss = __fadd_rn(ss, 1e-5f);
        sf = __fdiv_rn(1.0f, __fsqrt_rn(ss));
        if (sizeof(T) == 2) sf = __half2float(__float2half_rn(sf));
    }
    FAM_STRIDE(i, n) st(y + i, __fmul_rn(ld(w + i), __fmul_rn(sf, ld(x + i))));
}
template <class T> void weighted_scaling(const T *x, const T *w, T *y, long long n, float sf, const T *sumsq)
{
    if (n > 0) TL_LAUNCH((weighted_scaling_kernel<T>), fam_grid(n), 256, 0, x, w, y, n, sf, sumsq);
}
// out[0] = sum in[i]^2 (the reference leaves one partial sum per core; this library is "one core")
// [ref: lib/sources/pulp_rmsnorm_fp32.c:78-95]
template <class T>
__global__ void __launch_bounds__(1024) sum_of_squares_kernel(const T *__restrict__ x, T *__restrict__ out, long long n)
{
    __shared__ float red[33];
    float s = 0.f;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) { const float v = ld(x + i); s = fmaf(v, v, s); }
    s = block_sum(s, red);
    if (threadIdx.x == 0) st(out, s);
}
template <class T> void sum_of_squares(const T *x, T *out, long long n)
{
    if (n > 0) TL_LAUNCH((sum_of_squares_kernel<T>), 1, 1024, 0, x, out, n);
}
// SwiGLU: out = in1 * (1 / (1 + exp(-in1))) * in2   [ref: lib/sources/pulp_act_fp32.c:688-712]
template <class T>
__global__ void swiglu_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ y, long long n)
{
    FAM_STRIDE(i, n) {
        float v = ld(a + i);
        v = __fmul_rn(v, __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-v))));
        if (sizeof(T) == 2) v = __half2float(__float2half_rn(v));
        st(y + i, __fmul_rn(v, ld(b + i)));
    }
}
template <class T> void swiglu(const T *a, const T *b, T *y, long long n)
{
    if (n > 0) TL_LAUNCH((swiglu_kernel<T>), fam_grid(n), 256, 0, a, b, y, n);
}

// ------------------------------------------------------------------ pieces of the reference's softmax
// maxes[0] = max of a W-long vector (one core's share = all of it)   [ref: lib/sources/pulp_train_utils_fp32.c:987-1006]
template <class T> __global__ void __launch_bounds__(1024) vec_max_kernel(const T *__restrict__ x, T *__restrict__ out, long long n)
{
    __shared__ float red[33];
    float m = -FLT_MAX;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, ld(x + i));
    m = block_max(m, red);
    if (threadIdx.x == 0) st(out, m);
}
template <class T> void vec_max(const T *x, T *out, long long n) { if (n > 0) TL_LAUNCH((vec_max_kernel<T>), 1, 1024, 0, x, out, n); }

// output[i] = exp(input[i] - max); sums[0] = their sum   [ref: lib/sources/pulp_train_utils_fp32.c:1730-1756]
template <class T> __global__ void __launch_bounds__(1024) vec_exp_sum_kernel(const T *__restrict__ x, T *__restrict__ y, T *__restrict__ sum, long long n, float mx)
{
    __shared__ float red[33];
    float s = 0.f;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) {
        float o = expf(__fsub_rn(ld(x + i), mx));
        if (sizeof(T) == 2) o = __half2float(__float2half_rn(o));
        st(y + i, o); s += o;
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) st(sum, s);
}
template <class T> void vec_exp_sum(const T *x, T *y, T *sum, long long n, float mx) { if (n > 0) TL_LAUNCH((vec_exp_sum_kernel<T>), 1, 1024, 0, x, y, sum, n, mx); }

// out = exp(in - max) / sum over one vector   [ref: lib/sources/pulp_act_fp32.c:651-685]
template <class T> __global__ void __launch_bounds__(1024) vector_softmax_kernel(const T *__restrict__ x, T *__restrict__ y, long long n)
{
    __shared__ float red[33];
    float m = -FLT_MAX;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, ld(x + i));
    m = block_max(m, red);
    float s = 0.f;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) s += expf(__fsub_rn(ld(x + i), m));
    s = block_sum(s, red);
    for (long long i = threadIdx.x; i < n; i += blockDim.x) st(y + i, __fdiv_rn(expf(__fsub_rn(ld(x + i), m)), s));
}
template <class T> void vector_softmax(const T *x, T *y, long long n) { if (n > 0) TL_LAUNCH((vector_softmax_kernel<T>), 1, 1024, 0, x, y, n); }
// io[i] /= d   [ref: lib/sources/pulp_train_utils_fp32.c:1250-1264]
template <class T> __global__ void vec_div_kernel(T *__restrict__ io, long long n, float d) { FAM_STRIDE(i, n) st(io + i, __fdiv_rn(ld(io + i), d)); }
template <class T> void vec_div(T *io, long long n, float d) { if (n > 0) TL_LAUNCH((vec_div_kernel<T>), fam_grid(n), 256, 0, io, n, d); }

// The reference's polynomial stand-in for 2^-x: 0 from 3.14 on   [ref: lib/sources/pulp_train_utils_fp32.c:1009-1027]
__device__ __forceinline__ float threshold_dev(float x)
{
    if (x >= 3.14f) return 0.0f;
    const float x2 = __fmul_rn(x, x), x3 = __fmul_rn(x2, x), x4 = __fmul_rn(x3, x), x5 = __fmul_rn(x4, x);
    float r = __fsub_rn(1.0f, __fmul_rn(0.6931471805599453f, x));
    r = __fadd_rn(r, __fmul_rn(__fmul_rn(0.5f, x2), 0.4804530139182014f));
    r = __fsub_rn(r, __fmul_rn(__fmul_rn(0.16f, x3), 0.3330246519889294f));
    r = __fadd_rn(r, __fmul_rn(__fmul_rn(0.0416f, x4), 0.2308350985830834f));
    r = __fsub_rn(r, __fmul_rn(__fmul_rn(0.008f, x5), 0.1600026977571413f));
    return r;
}
// output[i][j] = threshold(maxes[i] - input[i][j]); sums[i] = row sum, dim x dim   [ref: pulp_train_utils_fp32.c:1193-1220]
template <class T> __global__ void __launch_bounds__(128) shift_sum_kernel(const T *__restrict__ x, const T *__restrict__ maxes, T *__restrict__ y, T *__restrict__ sums, int dim)
{
    __shared__ float red[33];
    const long long row = blockIdx.x;
    const float m = ld(maxes + row);
    float s = 0.f;
    for (int j = threadIdx.x; j < dim; j += blockDim.x) { const float o = threshold_dev(__fsub_rn(m, ld(x + row * dim + j))); st(y + row * dim + j, o); s += o; }
    s = block_sum(s, red);
    if (threadIdx.x == 0) st(sums + row, s);
}
template <class T> void shift_sum(const T *x, const T *maxes, T *y, T *sums, int dim) { if (dim > 0) TL_LAUNCH((shift_sum_kernel<T>), dim, 128, 0, x, maxes, y, sums, dim); }

// S[i] = sum_j A[i][j] B[i][j];  out[i][j] = (A[i][j] - S[i]) B[i][j]   [ref: pulp_train_utils_fp32.c:1136-1189]
template <class T> __global__ void __launch_bounds__(128) sm_bw_op1_kernel(const T *__restrict__ A, const T *__restrict__ B, T *__restrict__ S, int W)
{
    __shared__ float red[33];
    const long long row = blockIdx.x;
    float s = 0.f;
    for (int j = threadIdx.x; j < W; j += blockDim.x) s = fmaf(ld(A + row * W + j), ld(B + row * W + j), s);
    s = block_sum(s, red);
    if (threadIdx.x == 0) st(S + row, s);
}
template <class T> __global__ void sm_bw_op2_kernel(const T *__restrict__ A, const T *__restrict__ B, const T *__restrict__ S, T *__restrict__ out, long long total, int W)
{
    FAM_STRIDE(i, total) st(out + i, __fmul_rn(__fsub_rn(ld(A + i), ld(S + i / W)), ld(B + i)));
}
template <class T> void sm_bw_op1(const T *A, const T *B, T *S, int H, int W) { if (H > 0 && W > 0) TL_LAUNCH((sm_bw_op1_kernel<T>), H, 128, 0, A, B, S, W); }
template <class T> void sm_bw_op2(const T *A, const T *B, const T *S, T *out, int H, int W)
{
    const long long total = (long long)H * W;
    if (total > 0) TL_LAUNCH((sm_bw_op2_kernel<T>), fam_grid(total), 256, 0, A, B, S, out, total, W);
}

#define INST(T)                                                                                                        \
    template void l1_fw<T>(const T *, const T *, T *, int, int, bool, float);                                         \
    template void l1_bw<T>(const T *, const T *, T *, int, int, bool, float);                                         \
    template void maxpool_fw<T>(const T *, T *, long long, int, int, int, int, int, int, int, int);                   \
    template void maxpool_bw<T>(const T *, const T *, T *, long long, int, int, int, int, int, int, int, int);        \
    template void nonorm_fw<T>(const T *, const T *, const T *, T *, long long, int);                                  \
    template void weighted_scaling<T>(const T *, const T *, T *, long long, float, const T *);                         \
    template void sum_of_squares<T>(const T *, T *, long long);                                                        \
    template void swiglu<T>(const T *, const T *, T *, long long);                                                     \
    template void vec_max<T>(const T *, T *, long long);                                                               \
    template void vec_exp_sum<T>(const T *, T *, T *, long long, float);                                               \
    template void vector_softmax<T>(const T *, T *, long long);                                                        \
    template void vec_div<T>(T *, long long, float);                                                                   \
    template void shift_sum<T>(const T *, const T *, T *, T *, int);                                                   \
    template void sm_bw_op1<T>(const T *, const T *, T *, int, int);                                                   \
    template void sm_bw_op2<T>(const T *, const T *, const T *, T *, int, int);
INST(float)
INST(__half)

} // namespace tl
