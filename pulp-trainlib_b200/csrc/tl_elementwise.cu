// Bandwidth-bound kernels around the matmul-centred training step: activations, softmax,
// instance / batch / layer norm, MSE and CrossEntropy, SGD, residual adds, average pooling
// and the index-shuffling helpers (transpose, pad, broadcast add).  Each kernel cites the
// reference loop it replaces; reductions use warp shuffles, streams use 16-byte accesses.
#include "tl_kernels.h"
#include "tl_reduce.cuh"
#include <cfloat>

namespace tl {

static inline int grid_for(long long n, int per_block = 256, int waves = 16)
{
    long long b = (n + per_block - 1) / per_block;
    long long cap = (long long)sm_count() * waves;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (int)b;
}

#define GRID_STRIDE(i, n) for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (n); i += (long long)gridDim.x * blockDim.x)

// ------------------------------------------------------------------ activations
// [ref: lib/sources/pulp_act_fp32.c:37-180 (sigmoid, relu, leaky relu), :714-746 (GELU, rational tanh)]
__device__ __forceinline__ float act_apply(int kind, float x, float slope)
{
    switch (kind) {
    case ACT_RELU: return x > 0.f ? x : 0.f;
    case ACT_LEAKY: return x > 0.f ? x : x * slope;
    case ACT_SIGMOID: return 1.f / (1.f + expf(-x));
    default: {
        float half_x = 0.5f * x;
        float val = __fmul_rn(__fadd_rn(__fmul_rn(__fmul_rn(__fmul_rn(x, x), x), 0.044715f), x), 0.7978f);
        float v2 = __fmul_rn(val, val);
        float a = __fmul_rn(__fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(__fadd_rn(v2, 378.0f), v2), 17325.0f), v2), 135135.0f), val);
        float b = __fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(__fadd_rn(__fmul_rn(28.0f, v2), 3150.0f), v2), 62370.0f), v2), 135135.0f);
        val = __fdiv_rn(a, b);
        val = val > 1.f ? 1.f : (val < -1.f ? -1.f : val);
        return __fadd_rn(__fmul_rn(val, half_x), half_x);
    }
    }
}

template <class T> __global__ void act_fw_kernel(int kind, const T *__restrict__ x, T *__restrict__ y, long long n, float slope)
{
    GRID_STRIDE(i, n) st(y + i, act_apply(kind, ld(x + i), slope));
}

// Backward of the reference activations.  GELU has no backward in the reference; the
// derivative of its own rational approximation is used (clamped region: 0.5 * (1 +- 1)).
template <class T>
__global__ void act_bw_kernel(int kind, const T *__restrict__ x, const T *__restrict__ y, const T *__restrict__ dy,
                              T *__restrict__ dx, long long n, float slope)
{
    GRID_STRIDE(i, n) {
        float g = ld(dy + i), r;
        if (kind == ACT_RELU) r = ld(x + i) > 0.f ? g : 0.f;
        else if (kind == ACT_LEAKY) r = ld(x + i) > 0.f ? g : g * slope;
        else if (kind == ACT_SIGMOID) { float s = ld(y + i); r = g * (s * (1.f - s)); }
        else {
            float xv = ld(x + i);
            float u = (xv * xv * xv * 0.044715f + xv) * 0.7978f;
            float du = (3.f * 0.044715f * xv * xv + 1.f) * 0.7978f;
            float u2 = u * u;
            float a = (((u2 + 378.0f) * u2 + 17325.0f) * u2 + 135135.0f) * u;
            float b = ((28.0f * u2 + 3150.0f) * u2 + 62370.0f) * u2 + 135135.0f;
            float da = ((7.f * u2 + 5.f * 378.0f) * u2 + 3.f * 17325.0f) * u2 + 135135.0f;
            float db = ((6.f * 28.0f * u2 + 4.f * 3150.0f) * u2 + 2.f * 62370.0f) * u;
            float t = a / b, dt = (da * b - a * db) / (b * b);
            if (t > 1.f) { t = 1.f; dt = 0.f; } else if (t < -1.f) { t = -1.f; dt = 0.f; }
            r = g * (0.5f * (1.f + t) + 0.5f * xv * dt * du);
        }
        st(dx + i, r);
    }
}

template <class T> void act_fw(int kind, const T *x, T *y, long long n, float slope)
{
    if (n <= 0) return;
    TL_LAUNCH((act_fw_kernel<T>), grid_for(n), 256, 0, kind, x, y, n, slope);
}
template <class T> void act_bw(int kind, const T *x, const T *y, const T *dy, T *dx, long long n, float slope)
{
    if (n <= 0) return;
    TL_LAUNCH((act_bw_kernel<T>), grid_for(n), 256, 0, kind, x, y, dy, dx, n, slope);
}

// ------------------------------------------------------------------ softmax
// Row softmax: max, Schraudolph exp of (x - max), divide by the row sum
// [ref: lib/sources/pulp_act_fp32.c:187-245; pieces pulp_train_utils_fp32.c:1046-1138].
// One CTA per row; maxes/sums (caller scratch in the reference API) are written when given.
template <class T>
__global__ void __launch_bounds__(128) softmax_fw_kernel(const T *__restrict__ in, T *__restrict__ out,
                                                         T *__restrict__ maxes, T *__restrict__ sums, int width, int rows_per_batch)
{
    __shared__ float red[33];
    const long long row = blockIdx.x;
    const T *ip = in + row * width;
    T *op = out + row * width;
    float m = -FLT_MAX;
    for (int j = threadIdx.x; j < width; j += blockDim.x) m = fmaxf(m, ld(ip + j));
    m = block_max(m, red);
    float s = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) s += fastexp_gist_dev(__fsub_rn(ld(ip + j), m));
    s = block_sum(s, red);
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        st(op + j, __fdiv_rn(fastexp_gist_dev(__fsub_rn(ld(ip + j), m)), s));
    if (threadIdx.x == 0 && blockIdx.x < rows_per_batch) {       // scratch rows are shared across heads
        if (maxes) st(maxes + row, m);
        if (sums) st(sums + row, s);
    }
}

// dIn = (dOut - sum_j dOut_j * Out_j) * Out   [ref: lib/sources/pulp_act_fp32.c:335-392]
template <class T>
__global__ void __launch_bounds__(128) softmax_bw_kernel(const T *__restrict__ out, const T *__restrict__ dout,
                                                         T *__restrict__ din, T *__restrict__ sums, int width, int rows_per_batch)
{
    __shared__ float red[33];
    const long long row = blockIdx.x;
    const T *op = out + row * width, *gp = dout + row * width;
    T *ip = din + row * width;
    float s = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) s = fmaf(ld(gp + j), ld(op + j), s);
    s = block_sum(s, red);
    for (int j = threadIdx.x; j < width; j += blockDim.x) st(ip + j, __fmul_rn(__fsub_rn(ld(gp + j), s), ld(op + j)));
    if (threadIdx.x == 0 && sums && blockIdx.x < rows_per_batch) st(sums + row, s);
}

template <class T> void softmax_fw(const T *in, T *out, T *maxes, T *sums, int rows, int width, int batch)
{
    if (rows <= 0 || width <= 0) return;
    TL_LAUNCH((softmax_fw_kernel<T>), rows * batch, 128, 0, in, out, maxes, sums, width, rows);
}
template <class T> void softmax_bw(const T *out, const T *dout, T *din, T *sums, int rows, int width, int batch)
{
    if (rows <= 0 || width <= 0) return;
    TL_LAUNCH((softmax_bw_kernel<T>), rows * batch, 128, 0, out, dout, din, sums, width, rows);
}

template <class T> __global__ void row_max_kernel(const T *__restrict__ in, T *__restrict__ maxes, int width)
{
    __shared__ float red[33];
    const T *ip = in + (long long)blockIdx.x * width;
    float m = ld(maxes + blockIdx.x);                  // reference semantics: running maximum
    for (int j = threadIdx.x; j < width; j += blockDim.x) m = fmaxf(m, ld(ip + j));
    m = block_max(m, red);
    if (threadIdx.x == 0) st(maxes + blockIdx.x, m);
}
template <class T> __global__ void exp_sum_kernel(const T *__restrict__ in, T *__restrict__ out, const T *__restrict__ maxes, T *__restrict__ sums, int width)
{
    __shared__ float red[33];
    const long long row = blockIdx.x;
    float m = ld(maxes + row), s = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        float o = fastexp_gist_dev(__fsub_rn(ld(in + row * width + j), m));
        st(out + row * width + j, o);
        s += o;
    }
    s = block_sum(s, red);
    if (threadIdx.x == 0) st(sums + row, ld(sums + row) + s);   // reference accumulates into sums
}
template <class T> __global__ void row_div_kernel(T *__restrict__ io, const T *__restrict__ sums, int width, long long n)
{
    GRID_STRIDE(i, n) st(io + i, __fdiv_rn(ld(io + i), ld(sums + i / width)));
}
template <class T> void row_max(const T *in, T *maxes, int rows, int width) { if (rows > 0) TL_LAUNCH((row_max_kernel<T>), rows, 128, 0, in, maxes, width); }
template <class T> void exp_sum(const T *in, T *out, const T *maxes, T *sums, int rows, int width) { if (rows > 0) TL_LAUNCH((exp_sum_kernel<T>), rows, 128, 0, in, out, maxes, sums, width); }
template <class T> void row_div(T *io, const T *sums, int rows, int width)
{
    long long n = (long long)rows * width;
    if (n > 0) TL_LAUNCH((row_div_kernel<T>), grid_for(n), 256, 0, io, sums, width, n);
}

// ------------------------------------------------------------------ instance norm
// One CTA per (stream, channel) plane of D elements.  mean = sum/D, var = sum(x^2)/D - mean^2 + eps
// (clamped to eps when negative), stdev = sqrt(var); y = gamma/stdev * (x - mean) + beta
// [ref: lib/sources/pulp_instnorm_fp32.c:33-115, pulp_train_utils_fp32.c:1685-1728].
template <class T>
__global__ void __launch_bounds__(256) instnorm_fw_kernel(const T *__restrict__ x, T *__restrict__ y, const T *__restrict__ gb,
                                                          T *__restrict__ mean_o, T *__restrict__ var_o, T *__restrict__ std_o,
                                                          int C, int D, int frozen, float eps)
{
    __shared__ float red[33];
    const long long plane = blockIdx.x;
    const int ch = (int)(plane % C);
    const T *xp = x + plane * D;
    T *yp = y + plane * D;
    float mean, var, sd;
    if (!frozen) {
        float s = 0.f, q = 0.f;
        for (int d = threadIdx.x; d < D; d += blockDim.x) { float t = ld(xp + d); s += t; q = fmaf(t, t, q); }
        s = block_sum(s, red);
        q = block_sum(q, red);
        const float inv = 1.f / (float)D;
        mean = s * inv;
        var = q * inv;
        var = __fsub_rn(var, __fmul_rn(mean, mean));
        var = var + eps;
        if (var < 0.f) var = eps;
        sd = sqrtf(var);
        if (threadIdx.x == 0) { st(mean_o + plane, mean); st(var_o + plane, var); st(std_o + plane, sd); }
    } else {
        mean = ld(mean_o + plane); var = ld(var_o + plane); sd = ld(std_o + plane);
    }
    const float gamma = __fdiv_rn(ld(gb + ch), sd), beta = ld(gb + C + ch);
    for (int d = threadIdx.x; d < D; d += blockDim.x)
        st(yp + d, __fadd_rn(__fmul_rn(gamma, __fsub_rn(ld(xp + d), mean)), beta));
}

// dx = (-(sum dy) - (sum (x-mean) dy) * (x-mean)/var + D*dy) * gamma / (D*stdev)
// [ref: lib/sources/pulp_instnorm_fp32.c:117-175]
template <class T>
__global__ void __launch_bounds__(256) instnorm_bw_input_kernel(const T *__restrict__ x, const T *__restrict__ dy, T *__restrict__ dx,
                                                                const T *__restrict__ gamma, const T *__restrict__ mean_i,
                                                                const T *__restrict__ var_i, const T *__restrict__ std_i, int C, int D)
{
    __shared__ float red[33];
    const long long plane = blockIdx.x;
    const int ch = (int)(plane % C);
    const T *xp = x + plane * D, *gp = dy + plane * D;
    T *dp = dx + plane * D;
    const float mean = ld(mean_i + plane), var = ld(var_i + plane), sd = ld(std_i + plane), gm = ld(gamma + ch);
    float s = 0.f, p = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) { float g = ld(gp + d); s -= g; p -= (ld(xp + d) - mean) * g; }
    s = block_sum(s, red);
    p = block_sum(p, red);
    const float fD = (float)D, denom = fD * sd;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float grad = s;
        float md = (ld(xp + d) - mean) / var;
        grad += p * md;
        grad += fD * ld(gp + d);
        st(dp + d, grad * gm / denom);
    }
}

// Per-plane partials of dgamma = sum dy (x-mean) / stdev and dbeta = sum dy
// [ref: lib/sources/pulp_instnorm_fp32.c:182-230]; summed over streams in stream order below.
template <class T>
__global__ void __launch_bounds__(256) instnorm_bw_param_kernel(const T *__restrict__ x, const T *__restrict__ dy, float *__restrict__ part,
                                                                const T *__restrict__ mean_i, const T *__restrict__ std_i, int D)
{
    __shared__ float red[33];
    const long long plane = blockIdx.x;
    const T *xp = x + plane * D, *gp = dy + plane * D;
    const float mean = ld(mean_i + plane), sd = ld(std_i + plane);
    float a = 0.f, b = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) { float g = ld(gp + d); a = fmaf(g, ld(xp + d) - mean, a); b += g; }
    a = block_sum(a, red);
    b = block_sum(b, red);
    if (threadIdx.x == 0) { part[2 * plane] = a / sd; part[2 * plane + 1] = b; }
}
// out[map(j)] = sum over the n rows of in[n][dim], always added in the same order.  First pass: the rows are cut into
// slices; a CTA takes 32 columns of one slice, its 8 warps the rows round-robin (each warp reads 32 consecutive floats), and
// adds the 8 sums in warp order.  Second pass: one thread per column adds the slice sums in slice order.
// pairs > 0: the columns are (a, b) pairs per channel and the output is [all a | all b] (instance-norm parameters).
template <class T>
__global__ void __launch_bounds__(256) column_partial_kernel(const T *__restrict__ in, float *__restrict__ part, int n, int dim, int rows_per_slice)
{
    __shared__ float sm[8][33];
    const int c = threadIdx.x & 31, r = threadIdx.x >> 5, j = blockIdx.x * 32 + c;
    const int begin = blockIdx.y * rows_per_slice, end = min(n, begin + rows_per_slice);
    float s = 0.f;
    if (j < dim)
        for (int i = begin + r; i < end; i += 8) s += ld(in + (long long)i * dim + j);
    sm[r][c] = s;
    __syncthreads();
    if (r == 0 && j < dim) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; k++) t += sm[k][c];
        part[(long long)blockIdx.y * dim + j] = t;
    }
}
// One pass for few rows: a single slice, the 8 warp sums go straight to the output (with the pair mapping of the second pass).
template <class TI, class TO>
__global__ void __launch_bounds__(1024) column_direct_kernel(const TI *__restrict__ in, TO *__restrict__ out, int n, int dim, int pairs)
{
    // 32 columns x 32 row lanes; a lane walks rows r, r + 32, ... four at a time (independent loads in flight, the four partial
    // sums are then added in a fixed order), the 32 lane sums of a column are added in lane order: one fixed summation tree.
    __shared__ float sm[32][33];
    const int c = threadIdx.x & 31, r = threadIdx.x >> 5, j = blockIdx.x * 32 + c;
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
    if (j < dim) {
        int i = r;
        for (; i + 96 < n; i += 128) {
            s0 += ld(in + (long long)i * dim + j); s1 += ld(in + (long long)(i + 32) * dim + j);
            s2 += ld(in + (long long)(i + 64) * dim + j); s3 += ld(in + (long long)(i + 96) * dim + j);
        }
        for (; i < n; i += 32) s0 += ld(in + (long long)i * dim + j);
    }
    sm[r][c] = (s0 + s1) + (s2 + s3);
    __syncthreads();
    if (r == 0 && j < dim) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 32; k++) t += sm[k][c];
        st(out + (pairs > 0 ? (j & 1) * pairs + (j >> 1) : j), t);
    }
}
template <class T>
__global__ void __launch_bounds__(128) column_final_kernel(const float *__restrict__ part, T *__restrict__ out, int slices, int dim, int pairs)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= dim) return;
    float s = 0.f;
    for (int k = 0; k < slices; k++) s += part[(long long)k * dim + j];
    st(out + (pairs > 0 ? (j & 1) * pairs + (j >> 1) : j), s);
}
template <class TI, class TO>
static bool column_sum_launch(Scope &sc, const TI *in, TO *out, int n, int dim, int pairs)
{
    if (n <= 0 || dim <= 0) return true;
    if (n <= 1024) {        // 128 rows per thread at most: one launch instead of two
        TL_LAUNCH((column_direct_kernel<TI, TO>), (unsigned)((dim + 31) / 32), 1024, 0, in, out, n, dim, pairs);
        return true;
    }
    const int rows_per_slice = n >= 4096 ? 64 : (n >= 256 ? 32 : 8), slices = (n + rows_per_slice - 1) / rows_per_slice;
    float *part = sc.scratch<float>((size_t)slices * dim);
    if (!part) return false;
    TL_LAUNCH((column_partial_kernel<TI>), dim3((unsigned)((dim + 31) / 32), (unsigned)slices), 256, 0, in, part, n, dim, rows_per_slice);
    TL_LAUNCH((column_final_kernel<TO>), (unsigned)((dim + 127) / 128), 128, 0, part, out, slices, dim, pairs);
    return true;
}
// dgb = [sum of a | sum of b] over the streams of part[n][C] (a, b) pairs
template <class T> static void instnorm_param_reduce(Scope &sc, const float *part, T *dgb, int n, int C, bool deferred = false)
{
    if (deferred) { defer_columns(part, reinterpret_cast<float *>(dgb), n, 2 * C, C); return; }     // deferred only ever with T = float
    column_sum_launch<float, T>(sc, part, dgb, n, 2 * C, C);
}
template <class T> void column_sum(Scope &sc, const T *in, T *out, int n, int dim) { column_sum_launch<T, T>(sc, in, out, n, dim, 0); }

// fp32 planes of up to 1024 elements (a multiple of 4): one warp per plane, the plane held in registers as NV 16-byte
// vectors per lane, so every element is read once and the reductions are warp shuffles without a CTA barrier.
// RELU / SKIP fuse what follows the norm in a residual network into the same pass: y = relu(norm(x) + skip), each part optional,
// with the operations (and so the bits) of the separate norm, sum and ReLU kernels.
__device__ __forceinline__ float relu_of(float v) { return v > 0.f ? v : 0.f; }
template <int NV, bool RELU, bool SKIP>
__global__ void __launch_bounds__(256) instnorm_fw_warp_kernel(const float *__restrict__ x, float *__restrict__ y, const float *__restrict__ gb,
                                                               float *__restrict__ mean_o, float *__restrict__ var_o, float *__restrict__ std_o,
                                                               long long planes, int C, int D, int frozen, float eps, const float *__restrict__ skip)
{
    const int lane = threadIdx.x & 31;
    const long long plane = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (plane >= planes) return;
    const int ch = (int)(plane % C), D4 = D >> 2;
    const float4 *xp = reinterpret_cast<const float4 *>(x + plane * D);
    float4 *yp = reinterpret_cast<float4 *>(y + plane * D);
    float4 v[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) v[i] = (lane + 32 * i < D4) ? xp[lane + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
    float mean, var, sd;
    if (!frozen) {
        float s = 0.f, q = 0.f;
#pragma unroll
        for (int i = 0; i < NV; i++) {
            s += (v[i].x + v[i].y) + (v[i].z + v[i].w);
            q = fmaf(v[i].x, v[i].x, q); q = fmaf(v[i].y, v[i].y, q); q = fmaf(v[i].z, v[i].z, q); q = fmaf(v[i].w, v[i].w, q);
        }
        s = warp_sum(s); q = warp_sum(q);
        const float inv = 1.f / (float)D;
        mean = s * inv;
        var = q * inv;
        var = __fsub_rn(var, __fmul_rn(mean, mean));
        var = var + eps;
        if (var < 0.f) var = eps;
        sd = sqrtf(var);
        if (lane == 0) { mean_o[plane] = mean; var_o[plane] = var; std_o[plane] = sd; }
    } else {
        mean = mean_o[plane]; var = var_o[plane]; sd = std_o[plane];
    }
    const float gamma = __fdiv_rn(gb[ch], sd), beta = gb[C + ch];
#pragma unroll
    for (int i = 0; i < NV; i++)
        if (lane + 32 * i < D4) {
            float4 o;
            o.x = __fadd_rn(__fmul_rn(gamma, __fsub_rn(v[i].x, mean)), beta); o.y = __fadd_rn(__fmul_rn(gamma, __fsub_rn(v[i].y, mean)), beta);
            o.z = __fadd_rn(__fmul_rn(gamma, __fsub_rn(v[i].z, mean)), beta); o.w = __fadd_rn(__fmul_rn(gamma, __fsub_rn(v[i].w, mean)), beta);
            if (SKIP) {
                const float4 k = reinterpret_cast<const float4 *>(skip + plane * D)[lane + 32 * i];
                o.x = __fadd_rn(k.x, o.x); o.y = __fadd_rn(k.y, o.y); o.z = __fadd_rn(k.z, o.z); o.w = __fadd_rn(k.w, o.w);
            }
            if (RELU) { o.x = relu_of(o.x); o.y = relu_of(o.y); o.z = relu_of(o.z); o.w = relu_of(o.w); }
            yp[lane + 32 * i] = o;
        }
}
// Backward of the same planes: both plane sums once, then dX and/or the per-plane (dgamma, dbeta) partials.
// GATE: dy is the gradient behind a ReLU that followed the norm; the norm's output is recomputed from x with the forward's own
// operations and dy counts only where that output is positive (gamma points at [gamma | beta] then).
// dy2: a second gradient of the same output (another reader of it), added to dy first; GATE kernels only.
// dx = (D dy - sum(dy) - (x - mean) sum((x - mean) dy) / var) * gamma / (D stdev), the two per-plane quotients taken once:
// ka = gamma / (D stdev), kb = sum((x - mean) dy) / var
__device__ __forceinline__ float dx_of(float dy, float xm, float s, float kb, float fD, float ka) { return (fmaf(fD, dy, -s) - kb * xm) * ka; }
__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w)); }
__device__ __forceinline__ float gated(float dy, float xm, float scale, float beta) { return __fadd_rn(__fmul_rn(scale, xm), beta) > 0.f ? dy : 0.f; }
template <int NV, bool DX, bool PART, bool GATE>
__global__ void __launch_bounds__(256) instnorm_bw_warp_kernel(const float *__restrict__ x, const float *__restrict__ dy, float *__restrict__ dx,
                                                               float *__restrict__ part, const float *__restrict__ gamma,
                                                               const float *__restrict__ mean_i, const float *__restrict__ var_i,
                                                               const float *__restrict__ std_i, long long planes, int C, int D, const float *__restrict__ dy2)
{
    const int lane = threadIdx.x & 31;
    const long long plane = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (plane >= planes) return;
    const int ch = (int)(plane % C), D4 = D >> 2;
    const float4 *xp = reinterpret_cast<const float4 *>(x + plane * D), *gp = reinterpret_cast<const float4 *>(dy + plane * D);
    const float mean = mean_i[plane], sd = std_i[plane];
    float4 v[NV], g[NV];
#pragma unroll
    for (int i = 0; i < NV; i++) {
        const bool in = lane + 32 * i < D4;
        v[i] = in ? xp[lane + 32 * i] : make_float4(mean, mean, mean, mean);
        g[i] = in ? gp[lane + 32 * i] : make_float4(0.f, 0.f, 0.f, 0.f);
        if (GATE && dy2 && in) g[i] = add4(g[i], reinterpret_cast<const float4 *>(dy2 + plane * D)[lane + 32 * i]);
    }
    float s = 0.f, p = 0.f;     // s = sum dy, p = sum (x - mean) dy
    const float gsc = GATE ? __fdiv_rn(gamma[ch], sd) : 0.f, gbeta = GATE ? gamma[C + ch] : 0.f;
#pragma unroll
    for (int i = 0; i < NV; i++) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        if (GATE) {
            g[i].x = gated(g[i].x, v[i].x, gsc, gbeta); g[i].y = gated(g[i].y, v[i].y, gsc, gbeta);
            g[i].z = gated(g[i].z, v[i].z, gsc, gbeta); g[i].w = gated(g[i].w, v[i].w, gsc, gbeta);
        }
        s += (g[i].x + g[i].y) + (g[i].z + g[i].w);
        p = fmaf(v[i].x, g[i].x, p); p = fmaf(v[i].y, g[i].y, p); p = fmaf(v[i].z, g[i].z, p); p = fmaf(v[i].w, g[i].w, p);
    }
    s = warp_sum(s); p = warp_sum(p);
    if (PART && lane == 0) { part[2 * plane] = p / sd; part[2 * plane + 1] = s; }
    if (DX) {
        const float var = var_i[plane], gm = gamma[ch], fD = (float)D, ka = gm / (fD * sd), kb = p / var;
        float4 *dp = reinterpret_cast<float4 *>(dx + plane * D);
#pragma unroll
        for (int i = 0; i < NV; i++)
            if (lane + 32 * i < D4) {
                float4 o;
                o.x = dx_of(g[i].x, v[i].x, s, kb, fD, ka); o.y = dx_of(g[i].y, v[i].y, s, kb, fD, ka);
                o.z = dx_of(g[i].z, v[i].z, s, kb, fD, ka); o.w = dx_of(g[i].w, v[i].w, s, kb, fD, ka);
                dp[lane + 32 * i] = o;
            }
    }
}
// Planes of up to 64 elements (8x8 images): half a warp per plane, one 16-byte vector per lane; the sums run over the 16 lanes
// of a half with xor shuffles that stay inside it.
__device__ __forceinline__ float half_warp_sum(float v)
{
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
template <bool RELU, bool SKIP>
__global__ void __launch_bounds__(256) instnorm_fw_half_kernel(const float *__restrict__ x, float *__restrict__ y, const float *__restrict__ gb,
                                                               float *__restrict__ mean_o, float *__restrict__ var_o, float *__restrict__ std_o,
                                                               long long planes, int C, int D, int frozen, float eps, const float *__restrict__ skip)
{
    const int l16 = threadIdx.x & 15;
    const long long plane = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const bool live = plane < planes;
    const int D4 = D >> 2;
    const bool in = live && l16 < D4;
    const float4 v = in ? reinterpret_cast<const float4 *>(x + plane * D)[l16] : make_float4(0.f, 0.f, 0.f, 0.f);
    float mean, var, sd;
    if (!frozen) {
        float s = (v.x + v.y) + (v.z + v.w), q = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
        s = half_warp_sum(s); q = half_warp_sum(q);
        const float inv = 1.f / (float)D;
        mean = s * inv;
        var = q * inv;
        var = __fsub_rn(var, __fmul_rn(mean, mean));
        var = var + eps;
        if (var < 0.f) var = eps;
        sd = sqrtf(var);
        if (live && l16 == 0) { mean_o[plane] = mean; var_o[plane] = var; std_o[plane] = sd; }
    } else if (live) {
        mean = mean_o[plane]; var = var_o[plane]; sd = std_o[plane];
    } else { mean = 0.f; var = 1.f; sd = 1.f; }
    if (!in) return;
    const int ch = (int)(plane % C);
    const float gamma = __fdiv_rn(gb[ch], sd), beta = gb[C + ch];
    float4 o;
    o.x = __fadd_rn(__fmul_rn(gamma, __fsub_rn(v.x, mean)), beta); o.y = __fadd_rn(__fmul_rn(gamma, __fsub_rn(v.y, mean)), beta);
    o.z = __fadd_rn(__fmul_rn(gamma, __fsub_rn(v.z, mean)), beta); o.w = __fadd_rn(__fmul_rn(gamma, __fsub_rn(v.w, mean)), beta);
    if (SKIP) {
        const float4 k = reinterpret_cast<const float4 *>(skip + plane * D)[l16];
        o.x = __fadd_rn(k.x, o.x); o.y = __fadd_rn(k.y, o.y); o.z = __fadd_rn(k.z, o.z); o.w = __fadd_rn(k.w, o.w);
    }
    if (RELU) { o.x = relu_of(o.x); o.y = relu_of(o.y); o.z = relu_of(o.z); o.w = relu_of(o.w); }
    reinterpret_cast<float4 *>(y + plane * D)[l16] = o;
}
template <bool DX, bool PART, bool GATE>
__global__ void __launch_bounds__(256) instnorm_bw_half_kernel(const float *__restrict__ x, const float *__restrict__ dy, float *__restrict__ dx,
                                                               float *__restrict__ part, const float *__restrict__ gamma,
                                                               const float *__restrict__ mean_i, const float *__restrict__ var_i,
                                                               const float *__restrict__ std_i, long long planes, int C, int D, const float *__restrict__ dy2)
{
    const int l16 = threadIdx.x & 15;
    const long long plane = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const bool live = plane < planes;
    const int D4 = D >> 2;
    const bool in = live && l16 < D4;
    const float mean = live ? mean_i[plane] : 0.f, sd = live ? std_i[plane] : 1.f;
    float4 v = in ? reinterpret_cast<const float4 *>(x + plane * D)[l16] : make_float4(mean, mean, mean, mean);
    float4 g = in ? reinterpret_cast<const float4 *>(dy + plane * D)[l16] : make_float4(0.f, 0.f, 0.f, 0.f);
    v.x -= mean; v.y -= mean; v.z -= mean; v.w -= mean;
    if (GATE && dy2 && in) g = add4(g, reinterpret_cast<const float4 *>(dy2 + plane * D)[l16]);
    if (GATE && in) {
        const int ch = (int)(plane % C);
        const float gsc = __fdiv_rn(gamma[ch], sd), gbeta = gamma[C + ch];
        g.x = gated(g.x, v.x, gsc, gbeta); g.y = gated(g.y, v.y, gsc, gbeta); g.z = gated(g.z, v.z, gsc, gbeta); g.w = gated(g.w, v.w, gsc, gbeta);
    }
    float s = (g.x + g.y) + (g.z + g.w), p = fmaf(v.x, g.x, fmaf(v.y, g.y, fmaf(v.z, g.z, v.w * g.w)));
    s = half_warp_sum(s); p = half_warp_sum(p);
    if (PART && live && l16 == 0) { part[2 * plane] = p / sd; part[2 * plane + 1] = s; }
    if (DX && in) {
        const float var = var_i[plane], gm = gamma[(int)(plane % C)], fD = (float)D, ka = gm / (fD * sd), kb = p / var;
        float4 o;
        o.x = dx_of(g.x, v.x, s, kb, fD, ka); o.y = dx_of(g.y, v.y, s, kb, fD, ka);
        o.z = dx_of(g.z, v.z, s, kb, fD, ka); o.w = dx_of(g.w, v.w, s, kb, fD, ka);
        reinterpret_cast<float4 *>(dx + plane * D)[l16] = o;
    }
}
// Planes of 513..1024 elements: two warps per plane (4 sixteen-byte vectors of x and of dY per lane instead of 8), which
// halves the registers per thread and doubles the warps in flight; the two warp sums meet in shared memory.
template <bool DX, bool PART, bool GATE>
__global__ void __launch_bounds__(256) instnorm_bw_pair_kernel(const float *__restrict__ x, const float *__restrict__ dy, float *__restrict__ dx,
                                                               float *__restrict__ part, const float *__restrict__ gamma,
                                                               const float *__restrict__ mean_i, const float *__restrict__ var_i,
                                                               const float *__restrict__ std_i, long long planes, int C, int D, const float *__restrict__ dy2)
{
    __shared__ float2 sums[4][2];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, slot = warp >> 1, half = warp & 1;
    const long long plane = (long long)blockIdx.x * 4 + slot;
    const bool live = plane < planes;
    const int D4 = D >> 2;
    float4 v[4], g[4];
    float mean = 0.f, sd = 1.f;
    if (live) {
        mean = mean_i[plane]; sd = std_i[plane];
        const float4 *xp = reinterpret_cast<const float4 *>(x + plane * D), *gp = reinterpret_cast<const float4 *>(dy + plane * D);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int idx = half * 128 + lane + 32 * i;
            const bool in = idx < D4;
            v[i] = in ? xp[idx] : make_float4(mean, mean, mean, mean);
            g[i] = in ? gp[idx] : make_float4(0.f, 0.f, 0.f, 0.f);
            if (GATE && dy2 && in) g[i] = add4(g[i], reinterpret_cast<const float4 *>(dy2 + plane * D)[idx]);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 4; i++) { v[i] = make_float4(0.f, 0.f, 0.f, 0.f); g[i] = v[i]; }
    }
    float s = 0.f, p = 0.f;
    float gsc = 0.f, gbeta = 0.f;
    if (GATE && live) { const int gch = (int)(plane % C); gsc = __fdiv_rn(gamma[gch], sd); gbeta = gamma[C + gch]; }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        v[i].x -= mean; v[i].y -= mean; v[i].z -= mean; v[i].w -= mean;
        if (GATE) {
            g[i].x = gated(g[i].x, v[i].x, gsc, gbeta); g[i].y = gated(g[i].y, v[i].y, gsc, gbeta);
            g[i].z = gated(g[i].z, v[i].z, gsc, gbeta); g[i].w = gated(g[i].w, v[i].w, gsc, gbeta);
        }
        s += (g[i].x + g[i].y) + (g[i].z + g[i].w);
        p = fmaf(v[i].x, g[i].x, p); p = fmaf(v[i].y, g[i].y, p); p = fmaf(v[i].z, g[i].z, p); p = fmaf(v[i].w, g[i].w, p);
    }
    s = warp_sum(s); p = warp_sum(p);
    if (lane == 0) sums[slot][half] = make_float2(s, p);
    __syncthreads();
    s = sums[slot][0].x + sums[slot][1].x; p = sums[slot][0].y + sums[slot][1].y;      // same order in both warps
    if (!live) return;
    if (PART && lane == 0 && half == 0) { part[2 * plane] = p / sd; part[2 * plane + 1] = s; }
    if (DX) {
        const int ch = (int)(plane % C);
        const float var = var_i[plane], gm = gamma[ch], fD = (float)D, ka = gm / (fD * sd), kb = p / var;
        float4 *dp = reinterpret_cast<float4 *>(dx + plane * D);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int idx = half * 128 + lane + 32 * i;
            if (idx < D4) {
                float4 o;
                o.x = dx_of(g[i].x, v[i].x, s, kb, fD, ka); o.y = dx_of(g[i].y, v[i].y, s, kb, fD, ka);
                o.z = dx_of(g[i].z, v[i].z, s, kb, fD, ka); o.w = dx_of(g[i].w, v[i].w, s, kb, fD, ka);
                dp[idx] = o;
            }
        }
    }
}
static inline bool aligned16(const void *a, const void *b, const void *c) { return ((((uintptr_t)a) | ((uintptr_t)b) | ((uintptr_t)c)) & 15) == 0; }
static inline int instnorm_nv(int D) { return (D % 4 != 0 || D > 1024) ? 0 : (D <= 128 ? 1 : (D <= 256 ? 2 : (D <= 512 ? 4 : 8))); }
#define TL_NV_SWITCH(nv, CALL)                                                                                         \
    do { if ((nv) == 1) { CALL(1); } else if ((nv) == 2) { CALL(2); } else if ((nv) == 4) { CALL(4); } else { CALL(8); } } while (0)

template <bool RELU, bool SKIP>
static void instnorm_fw_warp_launch(const float *x, float *y, const float *gb, float *mean, float *var, float *stdev, long long planes, int C, int D,
                                    bool frozen, float eps, const float *skip, int nv)
{
    if (D <= 64) {
        TL_LAUNCH((instnorm_fw_half_kernel<RELU, SKIP>), (unsigned)((planes + 15) / 16), 256, 0, x, y, gb, mean, var, stdev, planes, C, D, frozen ? 1 : 0, eps, skip);
        return;
    }
#define TL_CALL(NV) TL_LAUNCH((instnorm_fw_warp_kernel<NV, RELU, SKIP>), (unsigned)((planes + 7) / 8), 256, 0, x, y, gb, mean, var, stdev, planes, C, D, frozen ? 1 : 0, eps, skip)
    TL_NV_SWITCH(nv, TL_CALL);
#undef TL_CALL
}
static bool instnorm_fw_warp(const float *x, float *y, const float *gb, float *mean, float *var, float *stdev, int n, int C, int D, bool frozen, float eps,
                             const float *skip = nullptr, bool relu = false)
{
    const int nv = instnorm_nv(D);
    if (!nv || !aligned16(x, y, skip)) return false;
    const long long planes = (long long)n * C;
    if (relu && skip) instnorm_fw_warp_launch<true, true>(x, y, gb, mean, var, stdev, planes, C, D, frozen, eps, skip, nv);
    else if (relu) instnorm_fw_warp_launch<true, false>(x, y, gb, mean, var, stdev, planes, C, D, frozen, eps, skip, nv);
    else if (skip) instnorm_fw_warp_launch<false, true>(x, y, gb, mean, var, stdev, planes, C, D, frozen, eps, skip, nv);
    else instnorm_fw_warp_launch<false, false>(x, y, gb, mean, var, stdev, planes, C, D, frozen, eps, skip, nv);
    return true;
}
template <class T> static bool instnorm_fw_warp(const T *, T *, const T *, T *, T *, T *, int, int, int, bool, float, const T * = nullptr, bool = false) { return false; }
// dx and/or part may be null: the kernel variant is chosen accordingly
static bool instnorm_bw_warp(const float *x, const float *dy, float *dx, float *part, const float *gamma, const float *mean, const float *var,
                             const float *stdev, int n, int C, int D, bool gate = false, const float *dy2 = nullptr)
{
    const int nv = instnorm_nv(D);
    if (!nv || !aligned16(x, dy, dx)) return false;
    if (gate && !(dx && part)) return false;           // the gated form exists for the one-pass backward only
    if (dy2 && (!gate || (((uintptr_t)dy2) & 15) != 0)) return false;
    const long long planes = (long long)n * C;
#define TL_BW_VARIANTS(KERNEL, GRID, ...)                                                                              \
    do {                                                                                                               \
        if (gate) TL_LAUNCH((KERNEL<__VA_ARGS__ true, true, true>), GRID, 256, 0, x, dy, dx, part, gamma, mean, var, stdev, planes, C, D, dy2);         \
        else if (dx && part) TL_LAUNCH((KERNEL<__VA_ARGS__ true, true, false>), GRID, 256, 0, x, dy, dx, part, gamma, mean, var, stdev, planes, C, D, dy2);  \
        else if (dx) TL_LAUNCH((KERNEL<__VA_ARGS__ true, false, false>), GRID, 256, 0, x, dy, dx, part, gamma, mean, var, stdev, planes, C, D, dy2);    \
        else TL_LAUNCH((KERNEL<__VA_ARGS__ false, true, false>), GRID, 256, 0, x, dy, dx, part, gamma, mean, var, stdev, planes, C, D, dy2);            \
    } while (0)
    if (D <= 64) {
        TL_BW_VARIANTS(instnorm_bw_half_kernel, (unsigned)((planes + 15) / 16), );
        return true;
    }
    if (nv == 8) {
        TL_BW_VARIANTS(instnorm_bw_pair_kernel, (unsigned)((planes + 3) / 4), );
        return true;
    }
    const unsigned blocks = (unsigned)((planes + 7) / 8);
    if (nv == 1) TL_BW_VARIANTS(instnorm_bw_warp_kernel, blocks, 1, );
    else if (nv == 2) TL_BW_VARIANTS(instnorm_bw_warp_kernel, blocks, 2, );
    else TL_BW_VARIANTS(instnorm_bw_warp_kernel, blocks, 4, );
#undef TL_BW_VARIANTS
    return true;
}
template <class T> static bool instnorm_bw_warp(const T *, const T *, T *, float *, const T *, const T *, const T *, const T *, int, int, int, bool = false, const T * = nullptr) { return false; }

template <class T>
void instnorm_fw(const T *x, T *y, const T *gb, T *mean, T *var, T *stdev, int n, int C, int D, bool frozen, float eps)
{
    if (n * C <= 0) return;
    if (instnorm_fw_warp(x, y, gb, mean, var, stdev, n, C, D, frozen, eps)) return;
    TL_LAUNCH((instnorm_fw_kernel<T>), n * C, D >= 256 ? 256 : 64, 0, x, y, gb, mean, var, stdev, C, D, frozen ? 1 : 0, eps);
}
template <class T>
void instnorm_bw_input(const T *x, const T *dy, T *dx, const T *gamma, const T *mean, const T *var, const T *stdev, int n, int C, int D)
{
    if (n * C <= 0) return;
    if (instnorm_bw_warp(x, dy, dx, (float *)nullptr, gamma, mean, var, stdev, n, C, D)) return;
    TL_LAUNCH((instnorm_bw_input_kernel<T>), n * C, D >= 256 ? 256 : 64, 0, x, dy, dx, gamma, mean, var, stdev, C, D);
}
template <class T>
void instnorm_bw_param(Scope &sc, const T *x, const T *dy, T *dgb, const T *mean, const T *stdev, int n, int C, int D)
{
    if (n * C <= 0) return;
    bool deferred;
    float *part = partials_alloc<T>(sc, (size_t)2 * n * C, deferred);
    if (!part) return;
    if (!instnorm_bw_warp(x, dy, (T *)nullptr, part, (const T *)nullptr, mean, (const T *)nullptr, stdev, n, C, D))
        TL_LAUNCH((instnorm_bw_param_kernel<T>), n * C, D >= 256 ? 256 : 64, 0, x, dy, part, mean, stdev, D);
    instnorm_param_reduce<T>(sc, part, dgb, n, C, deferred);
}
// Both gradients of one layer in one pass over x and dy (falls back to the two separate passes).
template <class T>
void instnorm_bw_both(Scope &sc, const T *x, const T *dy, T *dx, T *dgb, const T *gamma, const T *mean, const T *var, const T *stdev, int n, int C, int D)
{
    if (n * C <= 0) return;
    bool deferred;
    float *part = partials_alloc<T>(sc, (size_t)2 * n * C, deferred);
    if (!part) return;
    if (instnorm_bw_warp(x, dy, dx, part, gamma, mean, var, stdev, n, C, D)) {
        instnorm_param_reduce<T>(sc, part, dgb, n, C, deferred);
        return;
    }
    instnorm_bw_param<T>(sc, x, dy, dgb, mean, stdev, n, C, D);
    instnorm_bw_input<T>(x, dy, dx, gamma, mean, var, stdev, n, C, D);
}

// y = relu(norm(x) + skip) with `skip` and the ReLU optional.  One pass where the plane shape has a warp kernel, otherwise the
// norm, sum and ReLU kernels one after the other (same values either way).
template <class T>
void instnorm_act_fw(const T *x, T *y, const T *skip, const T *gb, T *mean, T *var, T *stdev, int n, int C, int D, bool frozen, float eps, bool relu)
{
    if (n * C <= 0) return;
    if (instnorm_fw_warp(x, y, gb, mean, var, stdev, n, C, D, frozen, eps, skip, relu)) return;
    const long long total = (long long)n * C * D;
    instnorm_fw<T>(x, y, gb, mean, var, stdev, n, C, D, frozen, eps);
    if (skip) add<T>(skip, y, y, total);
    if (relu) act_fw<T>(ACT_RELU, y, y, total, 0.f);
}
// Backward of y = relu(norm(x)): both gradients of the norm from dL/dy (+ dy2, the gradient of a second reader of y, when
// given).  `y` (the forward output) is only read by the fallback, which sums and masks into dy in place.
template <class T>
void instnorm_relu_bw(Scope &sc, const T *x, const T *y, T *dy, const T *dy2, T *dx, T *dgb, const T *gb, const T *mean, const T *var, const T *stdev,
                      int n, int C, int D)
{
    if (n * C <= 0) return;
    bool deferred;
    float *part = partials_alloc<T>(sc, (size_t)2 * n * C, deferred);
    if (!part) return;
    if (instnorm_bw_warp(x, dy, dx, part, gb, mean, var, stdev, n, C, D, true, dy2)) {
        instnorm_param_reduce<T>(sc, part, dgb, n, C, deferred);
        return;
    }
    if (dy2) add<T>(dy2, dy, dy, (long long)n * C * D);
    act_bw<T>(ACT_RELU, y, (const T *)nullptr, dy, dy, (long long)n * C * D, 0.f);
    instnorm_bw_both<T>(sc, x, dy, dx, dgb, gb, mean, var, stdev, n, C, D);
}

// ------------------------------------------------------------------ batch norm / layer norm (forward)
// mean = S1/n; sqrt_var = sqrt((S2 - 2*S1*mean)/n + mean^2 + eps); y = (x-mean)/sqrt_var * w + b
// [ref: lib/sources/pulp_batchnorm_fp32.c:84-109, pulp_layernorm_fp32.c:60-77].
template <class T>
__global__ void __launch_bounds__(256) batchnorm_fw_kernel(const T *__restrict__ x, T *__restrict__ y, const T *__restrict__ w,
                                                           const T *__restrict__ b, int B, int C, int HW, float eps)
{
    __shared__ float red[33];
    const int c = blockIdx.x % C;
    const long long s = blockIdx.x / C;                  // stream
    const T *xs = x + s * (long long)B * C * HW;
    T *ys = y + s * (long long)B * C * HW;
    const int cnt = B * HW;
    float s1 = 0.f, s2 = 0.f;
    for (int e = threadIdx.x; e < cnt; e += blockDim.x) {
        float t = ld(xs + ((long long)(e / HW) * C + c) * HW + e % HW);
        s1 += t; s2 = fmaf(t, t, s2);
    }
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    const float mean = s1 / (float)cnt;
    const float sv = sqrtf(__fadd_rn(__fadd_rn(__fdiv_rn(__fsub_rn(s2, __fmul_rn(__fmul_rn(2.f, s1), mean)), (float)cnt), __fmul_rn(mean, mean)), eps));
    const float wc = ld(w + c), bc = ld(b + c);
    for (int e = threadIdx.x; e < cnt; e += blockDim.x) {
        long long idx = ((long long)(e / HW) * C + c) * HW + e % HW;
        st(ys + idx, __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(ld(xs + idx), mean), sv), wc), bc));
    }
}
template <class T> void batchnorm_fw(const T *x, T *y, const T *w, const T *b, int n, int B, int C, int HW, float eps)
{
    if (n * C <= 0) return;
    TL_LAUNCH((batchnorm_fw_kernel<T>), n * C, (B * HW) >= 256 ? 256 : 64, 0, x, y, w, b, B, C, HW, eps);
}

template <class T>
__global__ void __launch_bounds__(128) layernorm_fw_kernel(const T *__restrict__ x, T *__restrict__ y, const T *__restrict__ w,
                                                           const T *__restrict__ b, int width, float eps)
{
    __shared__ float red[33];
    const T *xp = x + (long long)blockIdx.x * width;
    T *yp = y + (long long)blockIdx.x * width;
    float s1 = 0.f, s2 = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) { float t = ld(xp + j); s1 += t; s2 = fmaf(t, t, s2); }
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    const float mean = s1 / (float)width;
    const float sv = sqrtf(__fadd_rn(__fadd_rn(__fdiv_rn(__fsub_rn(s2, __fmul_rn(__fmul_rn(2.f, s1), mean)), (float)width), __fmul_rn(mean, mean)), eps));
    for (int j = threadIdx.x; j < width; j += blockDim.x)
        st(yp + j, __fadd_rn(__fmul_rn(__fdiv_rn(__fsub_rn(ld(xp + j), mean), sv), ld(w + j)), ld(b + j)));
}
// Backward of the layer norm above (the reference has no backward; derived from its forward formula):
// xhat = (x - mean) / sv, g = w * dy;  dx = (g - mean_j(g) - xhat * mean_j(g * xhat)) / sv per row;
// dw[j] = sum_rows dy * xhat, db[j] = sum_rows dy.  Kernel 1: one CTA per row writes dx and the row's (mean, 1/sv);
// kernel 2: one thread per column adds over the rows in row order.
template <class T>
__global__ void __launch_bounds__(128) layernorm_bw_rows_kernel(const T *__restrict__ x, const T *__restrict__ w, const T *__restrict__ dy,
                                                                T *__restrict__ dx, float2 *__restrict__ stats, int width, float eps)
{
    __shared__ float red[33];
    const long long row = blockIdx.x;
    const T *xp = x + row * width, *gp = dy + row * width;
    float s1 = 0.f, s2 = 0.f;
    for (int j = threadIdx.x; j < width; j += blockDim.x) { float t = ld(xp + j); s1 += t; s2 = fmaf(t, t, s2); }
    s1 = block_sum(s1, red);
    s2 = block_sum(s2, red);
    const float mean = s1 / (float)width;
    const float sv = sqrtf(__fadd_rn(__fadd_rn(__fdiv_rn(__fsub_rn(s2, __fmul_rn(__fmul_rn(2.f, s1), mean)), (float)width), __fmul_rn(mean, mean)), eps));
    const float inv = 1.f / sv;
    float a = 0.f, b = 0.f;     // sum g, sum g * xhat
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float g = ld(w + j) * ld(gp + j), xh = (ld(xp + j) - mean) * inv;
        a += g; b = fmaf(g, xh, b);
    }
    a = block_sum(a, red);
    b = block_sum(b, red);
    const float ma = a / (float)width, mb = b / (float)width;
    for (int j = threadIdx.x; j < width; j += blockDim.x) {
        const float g = ld(w + j) * ld(gp + j), xh = (ld(xp + j) - mean) * inv;
        st(dx + row * width + j, (g - ma - xh * mb) * inv);
    }
    if (threadIdx.x == 0) stats[row] = make_float2(mean, inv);
}
template <class T>
__global__ void __launch_bounds__(128) layernorm_bw_cols_kernel(const T *__restrict__ x, const T *__restrict__ dy, const float2 *__restrict__ stats,
                                                                T *__restrict__ dw, T *__restrict__ db, int rows, int width)
{
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= width) return;
    float a = 0.f, b = 0.f;
    for (int r = 0; r < rows; r++) {
        const float2 st2 = stats[r];
        const float g = ld(dy + (long long)r * width + j);
        a = fmaf(g, (ld(x + (long long)r * width + j) - st2.x) * st2.y, a);
        b += g;
    }
    st(dw + j, a); st(db + j, b);
}
template <class T> void layernorm_bw(Scope &sc, const T *x, const T *w, const T *dy, T *dx, T *dw, T *db, int rows, int width, float eps)
{
    if (rows <= 0) return;
    float2 *stats = sc.scratch<float2>((size_t)rows);
    if (!stats) return;
    TL_LAUNCH((layernorm_bw_rows_kernel<T>), rows, 128, 0, x, w, dy, dx, stats, width, eps);
    TL_LAUNCH((layernorm_bw_cols_kernel<T>), ceil_div(width, 128), 128, 0, x, dy, stats, dw, db, rows, width);
}

template <class T> void layernorm_fw(const T *x, T *y, const T *w, const T *b, int rows, int width, float eps)
{
    if (rows <= 0) return;
    TL_LAUNCH((layernorm_fw_kernel<T>), rows, 128, 0, x, y, w, b, width, eps);
}

template <class T> __global__ void mean_std_kernel(const T *__restrict__ x, T *mean, T *var, T *stdev, int D, float eps)
{
    __shared__ float red[33];
    float s = 0.f, q = 0.f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) { float t = ld(x + d); s += t; q = fmaf(t, t, q); }
    s = block_sum(s, red);
    q = block_sum(q, red);
    if (threadIdx.x == 0) {
        const float inv = 1.f / (float)D;
        float m = s * inv, v = q * inv;
        v = __fsub_rn(v, __fmul_rn(m, m));
        v += eps;
        if (v < 0.f) v = eps;
        st(mean, m); st(var, v); st(stdev, sqrtf(v));
    }
}
template <class T> void mean_std(const T *x, T *mean, T *var, T *stdev, int D, float eps)
{
    TL_LAUNCH((mean_std_kernel<T>), 1, 256, 0, x, mean, var, stdev, D, eps);
}

// ------------------------------------------------------------------ losses
// MSE: loss = sum (1/dim) (t - y)^2; dy = (1/dim) * 2 * (y - t)   [ref: lib/sources/pulp_losses_fp32.c:214-275]
template <class T>
__global__ void __launch_bounds__(256) mse_fw_kernel(const T *__restrict__ y, const T *__restrict__ t, T *__restrict__ loss, int dim)
{
    __shared__ float red[33];
    const T *yp = y + (long long)blockIdx.x * dim, *tp = t + (long long)blockIdx.x * dim;
    const float meanval = 1.0f / (float)dim;
    float s = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) { float d = ld(tp + i) - ld(yp + i); s += meanval * d * d; }
    s = block_sum(s, red);
    if (threadIdx.x == 0) st(loss + blockIdx.x, s);
}
template <class T> __global__ void mse_bw_kernel(const T *__restrict__ y, const T *__restrict__ t, T *__restrict__ dy, int dim, long long total)
{
    const float meanval = 1.0f / (float)dim;
    GRID_STRIDE(i, total) st(dy + i, __fmul_rn(__fmul_rn(meanval, 2.0f), __fsub_rn(ld(y + i), ld(t + i))));
}
template <class T> void mse_fw(const T *y, const T *t, T *loss, int dim, int n) { if (n > 0) TL_LAUNCH((mse_fw_kernel<T>), n, 256, 0, y, t, loss, dim); }
template <class T> void mse_bw(const T *y, const T *t, T *dy, int dim, int n)
{
    long long total = (long long)dim * n;
    if (total > 0) TL_LAUNCH((mse_bw_kernel<T>), grid_for(total), 256, 0, y, t, dy, dim, total);
}

// CrossEntropy on raw logits with a probability-vector target: one thread per stream walks
// the class vector in the reference's order (log-sum-exp with max shift)
// [ref: lib/sources/pulp_losses_fp32.c:26-137].
template <class T>
__global__ void ce_kernel(const T *__restrict__ z, const T *__restrict__ t, T *__restrict__ loss, T *__restrict__ dz, int dim, int n)
{
    int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= n) return;
    const T *zp = z + (long long)s * dim, *tp = t + (long long)s * dim;
    float mx = ld(zp);
    for (int i = 1; i < dim; i++) mx = fmaxf(mx, ld(zp + i));
    float se = 0.f;
    for (int i = 0; i < dim; i++) se += expf(ld(zp + i) - mx);
    float dot = 0.f, sy = 0.f;
    for (int i = 0; i < dim; i++) { float yi = ld(tp + i); dot = __fadd_rn(dot, __fmul_rn(yi, ld(zp + i))); sy += yi; }
    if (sy == 0.f) sy = 1.f;
    if (loss) st(loss + s, -(dot - (logf(se) + mx) * sy));
    if (dz) {
        const float inv = 1.0f / se;
        for (int i = 0; i < dim; i++) st(dz + (long long)s * dim + i, expf(ld(zp + i) - mx) * inv * sy - ld(tp + i));
    }
}
template <class T> void ce_fw(const T *z, const T *t, T *loss, int dim, int n) { if (n > 0) TL_LAUNCH((ce_kernel<T>), ceil_div(n, 128), 128, 0, z, t, loss, (T *)nullptr, dim, n); }
template <class T> void ce_bw(const T *z, const T *t, T *dz, int dim, int n) { if (n > 0) TL_LAUNCH((ce_kernel<T>), ceil_div(n, 128), 128, 0, z, t, (T *)nullptr, dz, dim, n); }

// ------------------------------------------------------------------ SGD and vector ops
// w -= lr*g; with weight decay the gradient is first replaced by g + lambda*w, as the reference
// does in place [ref: lib/sources/pulp_optimizers_fp32.c:48-62].
template <class T> __global__ void sgd_kernel(T *__restrict__ w, T *__restrict__ g, long long n, float lr, float lambda)
{
    GRID_STRIDE(i, n) {
        float wv = ld(w + i), gv = ld(g + i);
        if (lambda != 0.f) { gv = __fadd_rn(gv, __fmul_rn(lambda, wv)); st(g + i, gv); }
        st(w + i, __fsub_rn(wv, __fmul_rn(lr, gv)));
    }
}
template <class T> void sgd(T *w, T *g, long long n, float lr, float lambda) { if (n > 0) TL_LAUNCH((sgd_kernel<T>), grid_for(n), 256, 0, w, g, n, lr, lambda); }

template <class T> __global__ void add_kernel(const T *a, const T *b, T *c, long long n) { GRID_STRIDE(i, n) st(c + i, __fadd_rn(ld(a + i), ld(b + i))); }
template <class T> void add(const T *a, const T *b, T *c, long long n) { if (n > 0) TL_LAUNCH((add_kernel<T>), grid_for(n), 256, 0, a, b, c, n); }
template <class T> __global__ void copy_kernel(const T *__restrict__ f, T *__restrict__ t, long long n) { GRID_STRIDE(i, n) t[i] = f[i]; }
template <class T> void copy_n(const T *from, T *to, long long n) { if (n > 0 && from != to) TL_LAUNCH((copy_kernel<T>), grid_for(n), 256, 0, from, to, n); }
template <class T> __global__ void fill_kernel(T *t, float v, long long n) { GRID_STRIDE(i, n) st(t + i, v); }
template <class T> void fill(T *to, float v, long long n) { if (n > 0) TL_LAUNCH((fill_kernel<T>), grid_for(n), 256, 0, to, v, n); }
template <class T> __global__ void scale_kernel(T *x, float s, long long n) { GRID_STRIDE(i, n) st(x + i, __fmul_rn(ld(x + i), s)); }
template <class T> void scale(T *x, float s, long long n) { if (n > 0) TL_LAUNCH((scale_kernel<T>), grid_for(n), 256, 0, x, s, n); }
// mat[H x W] += bias: per_row -> bias[row] [ref: lib/sources/pulp_train_utils_fp32.c:1286-1327], else bias[col]
template <class T> __global__ void bias_add_kernel(T *mat, const T *bias, int W, long long n, int per_row)
{
    GRID_STRIDE(i, n) st(mat + i, __fadd_rn(ld(mat + i), ld(bias + (per_row ? i / W : i % W))));
}
template <class T> void bias_add_rows(T *mat, const T *bias, int H, int W, int per_row)
{
    long long n = (long long)H * W;
    if (n > 0) TL_LAUNCH((bias_add_kernel<T>), grid_for(n), 256, 0, mat, bias, W, n, per_row);
}
__global__ void cast_h2f_kernel(const __half *s, float *d, long long n) { GRID_STRIDE(i, n) d[i] = __half2float(s[i]); }
__global__ void cast_f2h_kernel(const float *s, __half *d, long long n) { GRID_STRIDE(i, n) d[i] = __float2half_rn(s[i]); }
void cast_h2f(const __half *src, float *dst, long long n) { if (n > 0) TL_LAUNCH(cast_h2f_kernel, grid_for(n), 256, 0, src, dst, n); }
void cast_f2h(const float *src, __half *dst, long long n) { if (n > 0) TL_LAUNCH(cast_f2h_kernel, grid_for(n), 256, 0, src, dst, n); }

// ------------------------------------------------------------------ average pooling
// [ref: lib/sources/pulp_pooling_fp32.c:24-66 (FW), :69-115 (BW: every window adds dy/HWk to its pixels)]
template <class T>
__global__ void avgpool_fw_kernel(const T *__restrict__ x, T *__restrict__ y, long long total, int H, int W, int Ho, int Wo,
                                  int Hk, int Wk, int sh, int sw)
{
    GRID_STRIDE(e, total) {
        int wo = e % Wo, ho = (e / Wo) % Ho;
        long long plane = e / ((long long)Wo * Ho);
        const T *xp = x + plane * H * W;
        float s = 0.f;
        for (int hk = 0; hk < Hk; hk++)
            for (int wk = 0; wk < Wk; wk++) s += ld(xp + (hk + ho * sh) * W + wk + wo * sw);
        st(y + e, __fdiv_rn(s, (float)(Hk * Wk)));
    }
}
template <class T>
__global__ void avgpool_bw_kernel(const T *__restrict__ dy, T *__restrict__ dx, long long total, int H, int W, int Ho, int Wo,
                                  int Hk, int Wk, int sh, int sw)
{
    GRID_STRIDE(e, total) {
        int wi = e % W, hi = (e / W) % H;
        long long plane = e / ((long long)W * H);
        const T *gp = dy + plane * Ho * Wo;
        const float inv_cnt = (float)(Hk * Wk);
        float s = 0.f;
        // windows (ho, wo) covering this pixel, visited in the reference's (ho, wo) order
        for (int ho = 0; ho < Ho; ho++) {
            int hk = hi - ho * sh;
            if (hk < 0 || hk >= Hk) continue;
            for (int wo = 0; wo < Wo; wo++) {
                int wk = wi - wo * sw;
                if (wk < 0 || wk >= Wk) continue;
                s += __fdiv_rn(ld(gp + ho * Wo + wo), inv_cnt);
            }
        }
        st(dx + e, s);
    }
}
// Global pooling of fp32 planes (one window = the whole plane, a multiple of 4 elements): a thread per plane adds the plane
// in the reference's order from 16-byte loads; backward writes dy / count with 16-byte stores.
__global__ void __launch_bounds__(256) avgpool_global_fw_kernel(const float *__restrict__ x, float *__restrict__ y, long long planes, int hw4, float cnt)
{
    const long long pl = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (pl >= planes) return;
    const float4 *xp = reinterpret_cast<const float4 *>(x) + pl * hw4;
    float s = 0.f;
#pragma unroll 8
    for (int i = 0; i < hw4; i++) { const float4 v = xp[i]; s += v.x; s += v.y; s += v.z; s += v.w; }
    y[pl] = __fdiv_rn(s, cnt);
}
__global__ void __launch_bounds__(256) avgpool_global_bw_kernel(const float *__restrict__ dy, float4 *__restrict__ dx, long long total4, int hw4, float cnt)
{
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total4; e += (long long)gridDim.x * blockDim.x) {
        const float v = __fdiv_rn(dy[e / hw4], cnt);
        dx[e] = make_float4(v, v, v, v);
    }
}
static bool avgpool_global(const float *x, const float *y, int H, int W, int Ho, int Wo, int Hk, int Wk)
{
    return Ho == 1 && Wo == 1 && Hk == H && Wk == W && (H * W) % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)y)) & 15) == 0;
}
template <class T> static bool avgpool_global(const T *, const T *, int, int, int, int, int, int) { return false; }
static void avgpool_global_fw(const float *x, float *y, long long planes, int hw) { TL_LAUNCH(avgpool_global_fw_kernel, (unsigned)((planes + 255) / 256), 256, 0, x, y, planes, hw / 4, (float)hw); }
static void avgpool_global_bw(const float *dy, float *dx, long long planes, int hw)
{
    const long long total4 = planes * (hw / 4);
    TL_LAUNCH(avgpool_global_bw_kernel, grid_for(total4), 256, 0, dy, reinterpret_cast<float4 *>(dx), total4, hw / 4, (float)hw);
}
template <class T> static void avgpool_global_fw(const T *, T *, long long, int) {}
template <class T> static void avgpool_global_bw(const T *, T *, long long, int) {}
template <class T> void avgpool_fw(const T *x, T *y, int n, int C, int H, int W, int Ho, int Wo, int Hk, int Wk, int sh, int sw)
{
    if ((long long)n * C > 0 && avgpool_global(x, y, H, W, Ho, Wo, Hk, Wk)) { avgpool_global_fw(x, y, (long long)n * C, H * W); return; }
    long long total = (long long)n * C * Ho * Wo;
    if (total > 0) TL_LAUNCH((avgpool_fw_kernel<T>), grid_for(total), 256, 0, x, y, total, H, W, Ho, Wo, Hk, Wk, sh, sw);
}
template <class T> void avgpool_bw(const T *dy, T *dx, int n, int C, int H, int W, int Ho, int Wo, int Hk, int Wk, int sh, int sw)
{
    if ((long long)n * C > 0 && avgpool_global(dx, dx, H, W, Ho, Wo, Hk, Wk)) { avgpool_global_bw(dy, dx, (long long)n * C, H * W); return; }
    long long total = (long long)n * C * H * W;
    if (total > 0) TL_LAUNCH((avgpool_bw_kernel<T>), grid_for(total), 256, 0, dy, dx, total, H, W, Ho, Wo, Hk, Wk, sh, sw);
}

// ------------------------------------------------------------------ N-d transpose, broadcast add, pad
struct Shape8 { int n; int d[8]; long long s[8]; };   // extents and source strides, in output order

// out = in.transpose(axes): out extent i = dims[axes[i]]  [ref: lib/sources/pulp_train_utils_fp32.c:79-185]
template <class T> __global__ void transpose_kernel(const T *__restrict__ in, T *__restrict__ out, Shape8 sh, long long total)
{
    GRID_STRIDE(e, total) {
        long long rem = e, src = 0;
#pragma unroll
        for (int k = 7; k >= 0; k--) {
            if (k < sh.n) { src += (rem % sh.d[k]) * sh.s[k]; rem /= sh.d[k]; }
        }
        out[e] = in[src];
    }
}
// 2-D case: 32x32 tiles through shared memory so that both sides are coalesced.
template <class T> __global__ void transpose2d_kernel(const T *__restrict__ in, T *__restrict__ out, int R, int Ccols)
{
    __shared__ T tile[32][33];
    int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int r = threadIdx.y; r < 32; r += blockDim.y)
        if (r0 + r < R && c0 + threadIdx.x < Ccols) tile[r][threadIdx.x] = in[(long long)(r0 + r) * Ccols + c0 + threadIdx.x];
    __syncthreads();
    for (int c = threadIdx.y; c < 32; c += blockDim.y)
        if (c0 + c < Ccols && r0 + threadIdx.x < R) out[(long long)(c0 + c) * R + r0 + threadIdx.x] = tile[threadIdx.x][c];
}
template <class T> void transpose_nd(const T *in, T *out, const int *dims, const int *axes, int nd)
{
    if (nd < 1 || nd > 8) { set_error(TL_ERR_BAD_ARGS, "transpose: n_dim %d outside 1..8", nd); return; }
    long long total = 1;
    long long in_stride[8];
    for (int i = nd - 1; i >= 0; i--) { in_stride[i] = total; total *= dims[i]; }
    if (total <= 0) return;
    if (nd == 2 && axes[0] == 1 && axes[1] == 0) {
        dim3 grid(ceil_div(dims[1], 32), ceil_div(dims[0], 32));
        TL_LAUNCH((transpose2d_kernel<T>), grid, dim3(32, 8), 0, in, out, dims[0], dims[1]);
        return;
    }
    Shape8 sh; sh.n = nd;
    for (int i = 0; i < 8; i++) { sh.d[i] = 1; sh.s[i] = 0; }
    for (int i = 0; i < nd; i++) {
        int a = axes[i];
        if (a < 0 || a >= nd) { set_error(TL_ERR_BAD_ARGS, "transpose: axis %d out of range", a); return; }
        sh.d[i] = dims[a]; sh.s[i] = in_stride[a];
    }
    TL_LAUNCH((transpose_kernel<T>), grid_for(total), 256, 0, in, out, sh, total);
}

// dest = op_1 + op_2 with NumPy broadcasting (extents aligned from the last axis, 1 repeats)
// [ref: lib/sources/pulp_train_utils_fp32.c:225-806]
struct Bcast8 { int n; int d[8]; long long sa[8]; long long sb[8]; };
template <class T> __global__ void broadcast_add_kernel(const T *__restrict__ a, const T *__restrict__ b, T *__restrict__ c, Bcast8 bc, long long total)
{
    GRID_STRIDE(e, total) {
        long long rem = e, ia = 0, ib = 0;
#pragma unroll
        for (int k = 7; k >= 0; k--) {
            if (k < bc.n) { long long q = rem % bc.d[k]; ia += q * bc.sa[k]; ib += q * bc.sb[k]; rem /= bc.d[k]; }
        }
        st(c + e, __fadd_rn(ld(a + ia), ld(b + ib)));
    }
}
template <class T> void broadcast_add(const T *a, const T *b, T *c, const int *da, int na, const int *db, int nb)
{
    int n = na > nb ? na : nb;
    if (n < 1 || n > 8 || na < 1 || nb < 1) { set_error(TL_ERR_BAD_ARGS, "array_broadcast_sum: rank outside 1..8"); return; }
    if (na == nb) {
        bool same = true; long long tot = 1;
        for (int i = 0; i < n; i++) { same &= (da[i] == db[i]); tot *= da[i]; }
        if (same) { add<T>(a, b, c, tot); return; }
    }
    Bcast8 bc; bc.n = n;
    long long total = 1, stra = 1, strb = 1;
    for (int i = 0; i < 8; i++) { bc.d[i] = 1; bc.sa[i] = 0; bc.sb[i] = 0; }
    for (int k = 0; k < n; k++) {                         // k-th axis from the end
        int ea = k < na ? da[na - 1 - k] : 1, eb = k < nb ? db[nb - 1 - k] : 1;
        int e = ea > eb ? ea : eb;
        if ((ea != e && ea != 1) || (eb != e && eb != 1)) { set_error(TL_ERR_BAD_ARGS, "array_broadcast_sum: extents %d and %d do not broadcast", ea, eb); return; }
        bc.d[n - 1 - k] = e;
        bc.sa[n - 1 - k] = (ea == 1) ? 0 : stra;
        bc.sb[n - 1 - k] = (eb == 1) ? 0 : strb;
        stra *= ea; strb *= eb; total *= e;
    }
    if (total > 0) TL_LAUNCH((broadcast_add_kernel<T>), grid_for(total), 256, 0, a, b, c, bc, total);
}

// Zero padding of a C x H x W (or H x W x C) tensor [ref: lib/sources/pulp_train_utils_fp32.c:929-988]
template <class T>
__global__ void pad_kernel(const T *__restrict__ src, T *__restrict__ dst, int C, int H, int W, int padL, int padU, int Ho, int Wo, int hwc, long long total)
{
    GRID_STRIDE(e, total) {
        int c, ht, wt;
        if (!hwc) { wt = e % Wo; ht = (e / Wo) % Ho; c = e / ((long long)Wo * Ho); }
        else { c = e % C; wt = (e / C) % Wo; ht = e / ((long long)C * Wo); }
        int hs = ht - padU, ws = wt - padL;
        T v = src[0];
        bool inside = hs >= 0 && hs < H && ws >= 0 && ws < W;
        if (inside) v = hwc ? src[((long long)hs * W + ws) * C + c] : src[((long long)c * H + hs) * W + ws];
        if (inside) dst[e] = v; else st(dst + e, 0.f);
    }
}
template <class T> void pad2d(const T *src, T *dst, int C, int H, int W, int padL, int padR, int padU, int padD, int hwc)
{
    int Ho = H + padU + padD, Wo = W + padL + padR;
    long long total = (long long)C * Ho * Wo;
    if (total > 0) TL_LAUNCH((pad_kernel<T>), grid_for(total), 256, 0, src, dst, C, H, W, padL, padU, Ho, Wo, hwc, total);
}

#define INST(T)                                                                                                    \
    template void act_fw<T>(int, const T *, T *, long long, float);                                                \
    template void act_bw<T>(int, const T *, const T *, const T *, T *, long long, float);                          \
    template void softmax_fw<T>(const T *, T *, T *, T *, int, int, int);                                          \
    template void softmax_bw<T>(const T *, const T *, T *, T *, int, int, int);                                    \
    template void instnorm_fw<T>(const T *, T *, const T *, T *, T *, T *, int, int, int, bool, float);            \
    template void instnorm_bw_input<T>(const T *, const T *, T *, const T *, const T *, const T *, const T *, int, int, int); \
    template void instnorm_bw_param<T>(Scope &, const T *, const T *, T *, const T *, const T *, int, int, int);   \
    template void instnorm_bw_both<T>(Scope &, const T *, const T *, T *, T *, const T *, const T *, const T *, const T *, int, int, int); \
    template void column_sum<T>(Scope &, const T *, T *, int, int);                                                \
    template void instnorm_act_fw<T>(const T *, T *, const T *, const T *, T *, T *, T *, int, int, int, bool, float, bool);             \
    template void instnorm_relu_bw<T>(Scope &, const T *, const T *, T *, const T *, T *, T *, const T *, const T *, const T *, const T *, int, int, int); \
    template void batchnorm_fw<T>(const T *, T *, const T *, const T *, int, int, int, int, float);                \
    template void layernorm_fw<T>(const T *, T *, const T *, const T *, int, int, float);                          \
    template void layernorm_bw<T>(Scope &, const T *, const T *, const T *, T *, T *, T *, int, int, float);      \
    template void mse_fw<T>(const T *, const T *, T *, int, int);                                                  \
    template void mse_bw<T>(const T *, const T *, T *, int, int);                                                  \
    template void ce_fw<T>(const T *, const T *, T *, int, int);                                                   \
    template void ce_bw<T>(const T *, const T *, T *, int, int);                                                   \
    template void sgd<T>(T *, T *, long long, float, float);                                                       \
    template void add<T>(const T *, const T *, T *, long long);                                                    \
    template void copy_n<T>(const T *, T *, long long);                                                            \
    template void fill<T>(T *, float, long long);                                                                  \
    template void scale<T>(T *, float, long long);                                                                 \
    template void bias_add_rows<T>(T *, const T *, int, int, int);                                                 \
    template void avgpool_fw<T>(const T *, T *, int, int, int, int, int, int, int, int, int, int);                 \
    template void avgpool_bw<T>(const T *, T *, int, int, int, int, int, int, int, int, int, int);                 \
    template void transpose_nd<T>(const T *, T *, const int *, const int *, int);                                  \
    template void broadcast_add<T>(const T *, const T *, T *, const int *, int, const int *, int);                 \
    template void pad2d<T>(const T *, T *, int, int, int, int, int, int, int, int);                                \
    template void row_max<T>(const T *, T *, int, int);                                                            \
    template void exp_sum<T>(const T *, T *, const T *, T *, int, int);                                            \
    template void row_div<T>(T *, const T *, int, int);                                                            \
    template void mean_std<T>(const T *, T *, T *, T *, int, float);
INST(float)
INST(__half)

} // namespace tl
