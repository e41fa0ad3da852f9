// GEMM family on CUDA cores: register-tiled FFMA kernel with arbitrary operand strides
// (so that no transposed copy of an operand is ever materialised) and the three
// bandwidth-bound batch-1 Linear kernels.  Replaces the mm / mm_M / mm_unroll_* family
// [ref: lib/sources/pulp_matmul_fp32.c:190-3697, pulp_matmul_fp16.c:191-1908].
#include "tl_kernels.h"

namespace tl {

// ------------------------------------------------------------------ tiled FFMA GEMM
// CTA tile BM x BN, K step 16, each thread a TM x TN register tile, fp32 accumulate.
// Operand tiles are staged in shared memory as [k][row] so the inner product reads
// contiguous, conflict-free vectors.  k runs ascending inside a thread, i.e. the same
// summation order per output as the reference's single-accumulator loop
// [ref: lib/sources/pulp_matmul_fp32.c:247-259].
template <class T, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_ffma_kernel(GemmDesc<T> d)
{
    const int b = blockIdx.z;
    const T *A = d.A + (long long)b * d.a_bs;
    const T *B = d.B + (long long)b * d.b_bs;
    T *C = d.C + (long long)b * d.c_bs;

#include "tl_gemm_body.inc"
}

// The same tiles for up to three products of one shape whose operands are separate allocations: blockIdx.z picks the product
// (with selects: indexing a kernel parameter by a run-time value would move it to local memory).
template <class T, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_ffma_list_kernel(GemmDesc<T> d, GemmList<T> l)
{
    const int b = blockIdx.z;
    const T *A = b == 0 ? l.A[0] : b == 1 ? l.A[1] : l.A[2];
    const T *B = b == 0 ? l.B[0] : b == 1 ? l.B[1] : l.B[2];
    T *C = b == 0 ? l.C[0] : b == 1 ? l.C[1] : l.C[2];
    d.bias = b == 0 ? l.bias[0] : b == 1 ? l.bias[1] : l.bias[2];
    if (!d.bias) d.bias_mode = 0;
#include "tl_gemm_body.inc"
}

// Tensor-core path (tl_gemm_tc.cu); returns false when the shape/layout does not qualify.
template <class T> bool gemm_tensor_core(const GemmDesc<T> &d);
template <class T> bool gemm_tensor_core_tma(const GemmDesc<T> &d);

template <class T> void gemm(const GemmDesc<T> &d)
{
    if (d.N <= 0 || d.M <= 0 || d.batch <= 0) return;
    // 0 auto, 1 FFMA only, 2 staged tensor-core kernel forced, 3 TMA tensor-core kernel forced
    if (gemm_path() != 1 && gemm_path() != 2 && gemm_tensor_core_tma<T>(d)) return;
    if (gemm_path() != 1 && gemm_path() != 3 && gemm_tensor_core<T>(d)) return;
    long long tiles64 = (long long)ceil_div(d.N, 64) * ceil_div(d.M, 64) * d.batch;
    if (tiles64 >= sm_count() || (d.N > 32 && d.M > 32 && tiles64 * 4 >= 2 * sm_count())) {
        dim3 grid(ceil_div(d.M, 64), ceil_div(d.N, 64), d.batch);
        TL_LAUNCH((gemm_ffma_kernel<T, 64, 64, 4, 4>), grid, 256, 0, d);
    } else {
        dim3 grid(ceil_div(d.M, 32), ceil_div(d.N, 32), d.batch);
        // fewer 32 x 32 tiles than SMs: four times as many CTAs of a quarter of the work (fp32; the fp16 block of config 4
        // measured 2 % slower with them, config 3 4 % faster)
        if (sizeof(T) == 4 && (long long)grid.x * grid.y * grid.z < sm_count() && d.K >= 64) {
            dim3 g16(ceil_div(d.M, 16), ceil_div(d.N, 16), d.batch);
            TL_LAUNCH((gemm_ffma_kernel<T, 16, 16, 1, 1>), g16, 256, 0, d);
            return;
        }
        TL_LAUNCH((gemm_ffma_kernel<T, 32, 32, 2, 2>), grid, 256, 0, d);
    }
}

template <class T> void gemm_list(const GemmDesc<T> &shape, const GemmList<T> &l, int count)
{
    if (shape.N <= 0 || shape.M <= 0 || count <= 0) return;
    if (count > 3) { set_error(TL_ERR_BAD_ARGS, "gemm_list: %d products (3 at most)", count); return; }
    // products large enough for the tensor-core kernels, and forced paths, go one by one
    if (gemm_path() > 1 || (long long)shape.N * shape.M * shape.K >= (1ll << 26)) {
        for (int p = 0; p < count; p++) {
            GemmDesc<T> one = shape; one.batch = 1; one.A = l.A[p]; one.B = l.B[p]; one.C = l.C[p]; one.bias = l.bias[p];
            if (!one.bias) one.bias_mode = 0;
            gemm<T>(one);
        }
        return;
    }
    GemmDesc<T> d = shape;
    const long long tiles64 = (long long)ceil_div(d.N, 64) * ceil_div(d.M, 64) * count;
    if (tiles64 >= sm_count() || (d.N > 32 && d.M > 32 && tiles64 * 4 >= 2 * sm_count())) {
        dim3 grid(ceil_div(d.M, 64), ceil_div(d.N, 64), count);
        TL_LAUNCH((gemm_ffma_list_kernel<T, 64, 64, 4, 4>), grid, 256, 0, d, l);
    } else {
        dim3 grid(ceil_div(d.M, 32), ceil_div(d.N, 32), count);
        TL_LAUNCH((gemm_ffma_list_kernel<T, 32, 32, 2, 2>), grid, 256, 0, d, l);
    }
}

template <class T> void mm_contract(const T *A, const T *B, T *C, int N, int K, int M, int trans_B, bool accumulate)
{
    GemmDesc<T> d;
    d.A = A; d.B = B; d.C = C; d.N = N; d.M = M; d.K = K;
    d.a_rs = K; d.a_cs = 1;
    if (trans_B) { d.b_rs = 1; d.b_cs = K; } else { d.b_rs = M; d.b_cs = 1; }
    d.c_rs = M; d.c_cs = 1;
    d.accumulate = accumulate;
    gemm<T>(d);
}

// ------------------------------------------------------------------ batch-1 Linear (HBM-bound)
// y[o] = sum_i W[o][i] x[i] (+ b[o]).  One warp per output row: each lane streams 16-byte
// pieces of the row, partial sums meet in a shuffle tree.  Rows are `in` elements apart, so
// 16-byte loads need in % (16/sizeof(T)) == 0; otherwise the scalar tail loop does all of it.
template <class T, int VEC>
__device__ __forceinline__ float dot_row(const T *__restrict__ w, const T *__restrict__ x, int n, int lane);

template <> __device__ __forceinline__ float dot_row<float, 4>(const float *__restrict__ w, const float *__restrict__ x, int n, int lane)
{
    float s = 0.f;
    int n4 = ((((uintptr_t)w | (uintptr_t)x) & 15) == 0) ? n / 4 : 0;
    const float4 *w4 = (const float4 *)w, *x4 = (const float4 *)x;
    // four 16-byte loads in flight per lane, one accumulator each
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    int i = lane;
    for (; i + 96 < n4; i += 128) {
        const float4 a0 = __ldcs(w4 + i), a1 = __ldcs(w4 + i + 32), a2 = __ldcs(w4 + i + 64), a3 = __ldcs(w4 + i + 96);
        const float4 b0 = __ldg(x4 + i), b1 = __ldg(x4 + i + 32), b2 = __ldg(x4 + i + 64), b3 = __ldg(x4 + i + 96);
        s = fmaf(a0.x, b0.x, s); s = fmaf(a0.y, b0.y, s); s = fmaf(a0.z, b0.z, s); s = fmaf(a0.w, b0.w, s);
        s1 = fmaf(a1.x, b1.x, s1); s1 = fmaf(a1.y, b1.y, s1); s1 = fmaf(a1.z, b1.z, s1); s1 = fmaf(a1.w, b1.w, s1);
        s2 = fmaf(a2.x, b2.x, s2); s2 = fmaf(a2.y, b2.y, s2); s2 = fmaf(a2.z, b2.z, s2); s2 = fmaf(a2.w, b2.w, s2);
        s3 = fmaf(a3.x, b3.x, s3); s3 = fmaf(a3.y, b3.y, s3); s3 = fmaf(a3.z, b3.z, s3); s3 = fmaf(a3.w, b3.w, s3);
    }
    for (; i < n4; i += 32) {
        float4 a = __ldcs(w4 + i), b = __ldg(x4 + i);
        s = fmaf(a.x, b.x, s); s = fmaf(a.y, b.y, s); s = fmaf(a.z, b.z, s); s = fmaf(a.w, b.w, s);
    }
    s = (s + s1) + (s2 + s3);
    for (int t = n4 * 4 + lane; t < n; t += 32) s = fmaf(w[t], x[t], s);
    return s;
}
template <> __device__ __forceinline__ float dot_row<__half, 8>(const __half *__restrict__ w, const __half *__restrict__ x, int n, int lane)
{
    float s = 0.f;
    int n8 = ((((uintptr_t)w | (uintptr_t)x) & 15) == 0) ? n / 8 : 0;
    const uint4 *w8 = (const uint4 *)w, *x8 = (const uint4 *)x;
    for (int i = lane; i < n8; i += 32) {
        uint4 a = __ldcs(w8 + i), b = __ldg(x8 + i);
        const __half2 *ah = (const __half2 *)&a, *bh = (const __half2 *)&b;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            float2 af = __half22float2(ah[q]), bf = __half22float2(bh[q]);
            s = fmaf(af.x, bf.x, s); s = fmaf(af.y, bf.y, s);
        }
    }
    for (int i = n8 * 8 + lane; i < n; i += 32) s = fmaf(__half2float(w[i]), __half2float(x[i]), s);
    return s;
}

template <class T, int VEC>
__global__ void __launch_bounds__(256) linear_fw_kernel(const T *__restrict__ W, const T *__restrict__ x,
                                                        const T *__restrict__ bias, T *__restrict__ y, int out, int in, int parts)
{
    // a row is cut into `parts` segments (a multiple of 128 elements each), one warp per segment, so that layers with
    // few rows still put enough loads in flight; the segment sums of a row are added in segment order
    __shared__ float seg[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int rows_per_block = 8 / parts;
    const int r = warp / parts, p = warp % parts;
    int seg_len = ((in + parts - 1) / parts + 127) & ~127;
    const int i0 = p * seg_len, len = max(0, min(in - i0, seg_len));
    for (int ob = blockIdx.x * rows_per_block; ob < out; ob += gridDim.x * rows_per_block) {
        const int o = ob + r;
        float s = 0.f;
        if (o < out && len > 0) s = dot_row<T, VEC>(W + (long long)o * in + i0, x + i0, len, lane);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (parts == 1) {
            if (lane == 0 && o < out) st(y + o, bias ? s + ld(bias + o) : s);
        } else {
            if (lane == 0) seg[warp] = s;
            __syncthreads();
            if (lane == 0 && p == 0 && o < out) {
                float t = 0.f;
                for (int q = 0; q < parts; q++) t += seg[r * parts + q];
                st(y + o, bias ? t + ld(bias + o) : t);
            }
            __syncthreads();
        }
    }
}

template <class T> void linear_fw_gemv(const T *W, const T *x, const T *bias, T *y, int out, int in)
{
    // aim at >= 8 warps per SM: split rows while that leaves segments of at least 512 elements
    int parts = 1;
    while (parts < 8 && (long long)out * parts < (long long)sm_count() * 8 * 4 && in / (parts * 2) >= 512) parts *= 2;
    const int rows_per_block = 8 / parts;
    int blocks = ceil_div(out, rows_per_block);
    int cap = sm_count() * 8;
    if (blocks > cap) blocks = cap;
    TL_LAUNCH((linear_fw_kernel<T, sizeof(T) == 4 ? 4 : 8>), blocks, 256, 0, W, x, bias, y, out, in, parts);
}

// dW[o][i] = dy[o] * x[i]: a pure 16-byte-store stream over the out x in matrix.
template <class T>
__global__ void __launch_bounds__(256) linear_wg_kernel(const T *__restrict__ dy, const T *__restrict__ x,
                                                        T *__restrict__ dW, int out, int in)
{
    constexpr int V = 16 / sizeof(T);
    const long long total = (long long)out * in;
    const bool vec_ok = (in % V == 0) && (((uintptr_t)dW & 15) == 0) && (((uintptr_t)x & 15) == 0);
    if (vec_ok) {
        const long long nvec = total / V;
        const int row_vecs = in / V;
        for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < nvec; e += (long long)gridDim.x * blockDim.x) {
            int o = (int)(e / row_vecs), iv = (int)(e % row_vecs);
            float g = ld(dy + o);
            if (sizeof(T) == 4) {
                float4 xv = __ldg((const float4 *)x + iv);
                float4 r = make_float4(g * xv.x, g * xv.y, g * xv.z, g * xv.w);
                __stcs((float4 *)dW + e, r);
            } else {
                uint4 xv = __ldg((const uint4 *)x + iv);
                const __half2 *xh = (const __half2 *)&xv;
                uint4 r; __half2 *rh = (__half2 *)&r;
#pragma unroll
                for (int q = 0; q < 4; q++) { float2 f = __half22float2(xh[q]); rh[q] = __floats2half2_rn(g * f.x, g * f.y); }
                __stcs((uint4 *)dW + e, r);
            }
        }
    } else {
        for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
            int o = (int)(e / in), i = (int)(e % in);
            st(dW + e, ld(dy + o) * ld(x + i));
        }
    }
}

// Streams mode: dW[o][i] = sum over streams of dy[s][o] * x[s][i].  The contraction runs over the streams, so the
// streams are cut into blocks of 32: CTA b sums its block into partial b (thread = one dW element, x read
// coalesced, dy broadcast), a second launch adds the partials in block order (fixed order, no atomics).
template <class T>
__global__ void __launch_bounds__(256) linear_wg_streams_partial_kernel(const T *__restrict__ dy, const T *__restrict__ x, float *__restrict__ part,
                                                                        int n, int out, int in, int per)
{
    const int s0 = blockIdx.y * per, s1 = min(n, s0 + per);
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= out * in) return;
    const int o = e / in, i = e % in;
    float acc = 0.f;
    for (int s = s0; s < s1; s++) acc = fmaf(ld(dy + (long long)s * out + o), ld(x + (long long)s * in + i), acc);
    part[(long long)blockIdx.y * out * in + e] = acc;
}
template <class T>
__global__ void linear_wg_streams_reduce_kernel(const float *__restrict__ part, T *__restrict__ dW, int count, int blocks)
{
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= count) return;
    float acc = 0.f;
    for (int b = 0; b < blocks; b++) acc += part[(long long)b * count + e];
    st(dW + e, acc);
}
template <class T> bool linear_wg_streams(Scope &sc, const T *dy, const T *x, T *dW, int n, int out, int in)
{
    // worth it when the layer is small against the stream count; large layers keep the GEMM tiles
    if ((long long)out * in > 16384 || n < 64) return false;
    const int per = 32, blocks = ceil_div(n, per), count = out * in;
    float *part = sc.scratch<float>((size_t)blocks * count);
    if (!part) return false;
    dim3 grid(ceil_div(count, 256), blocks);
    TL_LAUNCH((linear_wg_streams_partial_kernel<T>), grid, 256, 0, dy, x, part, n, out, in, per);
    TL_LAUNCH((linear_wg_streams_reduce_kernel<T>), ceil_div(count, 256), 256, 0, part, dW, count, blocks);
    return true;
}

template <class T> void linear_wg_outer(const T *dy, const T *x, T *dW, int out, int in)
{
    long long work = ((long long)out * in) / (16 / sizeof(T)) + 1;
    int blocks = (int)((work + 255) / 256);
    int cap = sm_count() * 16;
    if (blocks > cap) blocks = cap;
    TL_LAUNCH((linear_wg_kernel<T>), blocks, 256, 0, dy, x, dW, out, in);
}

// dx[i] = sum_o W[o][i] dy[o].  The matrix is cut into row slabs; a CTA owns one slab and a
// 16-byte-wide column strip per thread, so every load is coalesced and W is read exactly once.
// Slab partials land in `part[slab][in]` and a second kernel adds them in slab order
// (deterministic; no atomics).
template <class T>
__global__ void __launch_bounds__(128) linear_ig_partial_kernel(const T *__restrict__ W, const T *__restrict__ dy,
                                                                float *__restrict__ part, int out, int in, int rows_per_slab)
{
    constexpr int V = 16 / sizeof(T);
    const int slab = blockIdx.y;
    const int o_begin = slab * rows_per_slab;
    const int o_end = min(out, o_begin + rows_per_slab);
    const int col0 = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (col0 >= in) return;
    float acc[V];
#pragma unroll
    for (int q = 0; q < V; q++) acc[q] = 0.f;
    const bool vec_ok = (in % V == 0) && (((uintptr_t)W & 15) == 0);
    if (vec_ok) {
#pragma unroll 8
        for (int o = o_begin; o < o_end; o++) {
            float g = ld(dy + o);
            if (sizeof(T) == 4) {
                float4 w = __ldcs((const float4 *)(W + (long long)o * in + col0));
                acc[0] = fmaf(w.x, g, acc[0]); acc[1] = fmaf(w.y, g, acc[1]);
                acc[2] = fmaf(w.z, g, acc[2]); acc[3] = fmaf(w.w, g, acc[3]);
            } else {
                uint4 w = __ldcs((const uint4 *)(W + (long long)o * in + col0));
                const __half2 *wh = (const __half2 *)&w;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    float2 f = __half22float2(wh[q]);
                    acc[2 * q] = fmaf(f.x, g, acc[2 * q]); acc[2 * q + 1] = fmaf(f.y, g, acc[2 * q + 1]);
                }
            }
        }
    } else {
        for (int o = o_begin; o < o_end; o++) {
            float g = ld(dy + o);
#pragma unroll
            for (int q = 0; q < V; q++)
                if (col0 + q < in) acc[q] = fmaf(ld(W + (long long)o * in + col0 + q), g, acc[q]);
        }
    }
#pragma unroll
    for (int q = 0; q < V; q++)
        if (col0 + q < in) part[(long long)slab * in + col0 + q] = acc[q];
}

// dx[i] = sum over slabs of part[slab][i], in a fixed order: 32 columns x 32 slices of the slabs per CTA
// (slice s adds slabs s, s+32, ...; one thread per column then adds the 32 slice sums in slice order).
template <class T>
__global__ void __launch_bounds__(1024) linear_ig_reduce_kernel(const float *__restrict__ part, T *__restrict__ dx, int in, int slabs)
{
    __shared__ float sm[32][33];
    const int cx = threadIdx.x & 31, sl = threadIdx.x >> 5;
    const int i = blockIdx.x * 32 + cx;
    float s = 0.f;
    if (i < in)
        for (int b = sl; b < slabs; b += 32) s += part[(long long)b * in + i];
    sm[sl][cx] = s;
    __syncthreads();
    if (sl == 0 && i < in) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 32; k++) t += sm[k][cx];
        st(dx + i, t);
    }
}

template <class T> void linear_ig_gemv(Scope &sc, const T *W, const T *dy, T *dx, int out, int in)
{
    constexpr int V = 16 / sizeof(T);
    int col_blocks = ceil_div(ceil_div(in, V), 128);
    // enough slabs to put ~4 CTAs on every SM, at least 8 rows each
    int slabs = ceil_div(4 * sm_count(), col_blocks);
    if (slabs > ceil_div(out, 8)) slabs = ceil_div(out, 8);
    if (slabs < 1) slabs = 1;
    int rows_per_slab = ceil_div(out, slabs);
    slabs = ceil_div(out, rows_per_slab);
    float *part = sc.scratch<float>((size_t)slabs * in);
    if (!part) return;
    TL_LAUNCH((linear_ig_partial_kernel<T>), dim3(col_blocks, slabs), 128, 0, W, dy, part, out, in, rows_per_slab);
    TL_LAUNCH((linear_ig_reduce_kernel<T>), ceil_div(in, 32), 1024, 0, part, dx, in, slabs);
}

// Both gradients of a batch-1 Linear layer in one launch [ref: lib/sources/pulp_linear_fp32.c:60-180, the two halves of
// pulp_linear_fp32_bw_cl].  A CTA owns 32 column strips of 16 bytes in one row slab; its four warps take every fourth
// row: for every row a thread loads its strip of W once, adds W * dy[o] to its dX partial and stores dy[o] * x[strip]
// to dW (a warp moves 512 contiguous bytes each way per row).  The four warps' partials are added in warp order, the
// slab's partial goes to `part`, and the CTA of a column block that finishes last (a ticket per column block) adds the
// slabs' partials, always in the same order, so the result does not depend on which CTA that is: one launch instead of
// three, W read once.
static __device__ unsigned tl_linear_tickets[8192];                 // one per column block; zero between launches
static constexpr int LBW_STRIPS = 32, LBW_LANES = 4;

template <class T>
__global__ void __launch_bounds__(LBW_STRIPS * LBW_LANES) linear_bw_fused_kernel(const T *__restrict__ W, const T *__restrict__ dy, const T *__restrict__ x,
                                                                                 T *__restrict__ dW, float *__restrict__ part, T *__restrict__ dx,
                                                                                 int out, int in, int rows_per_slab, int slabs)
{
    constexpr int V = 16 / sizeof(T);
    __shared__ float red[LBW_LANES][LBW_STRIPS][V + 1];
    __shared__ unsigned ticket_s;
    const int cx = threadIdx.x % LBW_STRIPS, ry = threadIdx.x / LBW_STRIPS, slab = blockIdx.y;
    const int o_end = min(out, (slab + 1) * rows_per_slab);
    const int col0 = (blockIdx.x * LBW_STRIPS + cx) * V;
    const bool live = col0 < in;                                    // in % V == 0 (host): a strip is inside or outside as a whole
    float acc[V], xv[V];
#pragma unroll
    for (int q = 0; q < V; q++) { acc[q] = 0.f; xv[q] = live ? ld(x + col0 + q) : 0.f; }
    if (live) {
#pragma unroll 8
        for (int o = slab * rows_per_slab + ry; o < o_end; o += LBW_LANES) {
            const float g = ld(dy + o);
            const long long e = (long long)o * in + col0;
            if (sizeof(T) == 4) {
                const float4 w = __ldcs((const float4 *)(W + e));
                acc[0] = fmaf(w.x, g, acc[0]); acc[1] = fmaf(w.y, g, acc[1]); acc[2] = fmaf(w.z, g, acc[2]); acc[3] = fmaf(w.w, g, acc[3]);
                __stcs((float4 *)(dW + e), make_float4(g * xv[0], g * xv[1], g * xv[2], g * xv[3]));
            } else {
                const uint4 w = __ldcs((const uint4 *)(W + e));
                const __half2 *wh = (const __half2 *)&w;
                uint4 r; __half2 *rh = (__half2 *)&r;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float2 f = __half22float2(wh[q]);
                    acc[2 * q] = fmaf(f.x, g, acc[2 * q]); acc[2 * q + 1] = fmaf(f.y, g, acc[2 * q + 1]);
                    rh[q] = __floats2half2_rn(g * xv[2 * q], g * xv[2 * q + 1]);
                }
                __stcs((uint4 *)(dW + e), r);
            }
        }
    }
#pragma unroll
    for (int q = 0; q < V; q++) red[ry][cx][q] = acc[q];
    __syncthreads();
    if (ry == 0 && live) {
#pragma unroll
        for (int q = 0; q < V; q++) __stcg(part + (long long)slab * in + col0 + q, ((red[0][cx][q] + red[1][cx][q]) + red[2][cx][q]) + red[3][cx][q]);
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket_s = atomicAdd(&tl_linear_tickets[blockIdx.x], 1u);
    __syncthreads();
    if (ticket_s != (unsigned)(slabs - 1)) return;
    __threadfence();                                                // the last CTA of this column block: every slab's partial is visible
    float t[V];
#pragma unroll
    for (int q = 0; q < V; q++) t[q] = 0.f;
    if (live)
        for (int b = ry; b < slabs; b += LBW_LANES)                 // lane r adds slabs r, r + 4, ...
#pragma unroll
            for (int q = 0; q < V; q += 4) {
                const float4 v = __ldcg((const float4 *)(part + (long long)b * in + col0 + q));
                t[q] += v.x; t[q + 1] += v.y; t[q + 2] += v.z; t[q + 3] += v.w;
            }
#pragma unroll
    for (int q = 0; q < V; q++) red[ry][cx][q] = t[q];
    __syncthreads();
    if (ry == 0 && live) {
#pragma unroll
        for (int q = 0; q < V; q++) st(dx + col0 + q, ((red[0][cx][q] + red[1][cx][q]) + red[2][cx][q]) + red[3][cx][q]);
    }
    if (threadIdx.x == 0) tl_linear_tickets[blockIdx.x] = 0;        // ready for the next launch on this device
}

// false: shape or alignment not covered (the caller issues the two separate kernels)
template <class T> bool linear_bw_fused(Scope &sc, const T *W, const T *dy, const T *x, T *dW, T *dx, int out, int in)
{
    constexpr int V = 16 / sizeof(T);
    if (in % V != 0 || ((((uintptr_t)W) | ((uintptr_t)dW) | ((uintptr_t)x) | ((uintptr_t)dx)) & 15) != 0) return false;
    const int col_blocks = ceil_div(in / V, LBW_STRIPS);
    if (col_blocks > 8192) return false;
    // about four CTAs per SM, at least 8 rows each
    int slabs = ceil_div(4 * sm_count(), col_blocks);
    if (slabs > ceil_div(out, 8)) slabs = ceil_div(out, 8);
    if (slabs < 1) slabs = 1;
    const int rows_per_slab = ceil_div(out, slabs);
    slabs = ceil_div(out, rows_per_slab);
    float *part = sc.scratch<float>((size_t)slabs * in);
    if (!part) return false;
    TL_LAUNCH((linear_bw_fused_kernel<T>), dim3(col_blocks, slabs), LBW_STRIPS * LBW_LANES, 0, W, dy, x, dW, part, dx, out, in, rows_per_slab, slabs);
    return true;
}
template bool linear_bw_fused<float>(Scope &, const float *, const float *, const float *, float *, float *, int, int);
template bool linear_bw_fused<__half>(Scope &, const __half *, const __half *, const __half *, __half *, __half *, int, int);

} // namespace tl

// ------------------------------------------------------------------ Linear input gradient without any allocation
// Some hosts cannot let a library allocate device memory: an application that has handed the whole device to its
// own memory pool (a cudaMalloc from here would fail or fragment it), a control loop whose memory budget is fixed
// at start-up, or a caller that cannot afford the implicit device-wide synchronisation an allocation may cause.
// For them the slab partials of the input-gradient kernel live in this fixed array instead of the staging arena.
// Every GPU that loads the library carries the 4 MiB until the process exits.
static constexpr size_t TL_NOALLOC_SCRATCH_FLOATS = (size_t)1 << 20;
static __device__ __align__(256) float tl_noalloc_scratch[TL_NOALLOC_SCRATCH_FLOATS];
static float *tl_noalloc_scratch_addr[64];          // per device: the array's device address (host code only has a stand-in symbol)

extern "C" __attribute__((visibility("default")))
int trainlib_linear_fp32_bw_input_grads_noalloc(const float *W, const float *dy, float *dx, int out, int in, void *cuda_stream)
{
    using namespace tl;
    if (!W || !dy || !dx || out < 1 || in < 1) { set_error(TL_ERR_BAD_ARGS, "linear input gradient (no-alloc): null pointer or empty layer"); return TL_ERR_BAD_ARGS; }
    if ((size_t)in > TL_NOALLOC_SCRATCH_FLOATS) {
        set_error(TL_ERR_TOO_LARGE, "linear input gradient (no-alloc): in = %d exceeds the fixed scratch of %zu floats", in, TL_NOALLOC_SCRATCH_FLOATS);
        return TL_ERR_TOO_LARGE;
    }
    int dev = 0;
    if (!TL_CUDA(cudaGetDevice(&dev))) return TL_ERR_CUDA;
    if (dev < 0 || dev >= 64) { set_error(TL_ERR_BAD_ARGS, "linear input gradient (no-alloc): device index %d", dev); return TL_ERR_BAD_ARGS; }
    if (!tl_noalloc_scratch_addr[dev]) {
        // once per device, with that device current: the symbol itself is not a device address
        float *ptr = nullptr;
        if (!TL_CUDA(cudaGetSymbolAddress((void **)&ptr, tl_noalloc_scratch))) return TL_ERR_CUDA;
        tl_noalloc_scratch_addr[dev] = ptr;
    }
    float *part = tl_noalloc_scratch_addr[dev];
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // same slab plan as the allocating entry point, capped by the scratch capacity
    const int col_blocks = ceil_div(ceil_div(in, 4), 128);
    int slabs = ceil_div(4 * sms, col_blocks);
    if (slabs > ceil_div(out, 8)) slabs = ceil_div(out, 8);
    const int cap = (int)(TL_NOALLOC_SCRATCH_FLOATS / (size_t)in);
    if (slabs > cap) slabs = cap;
    if (slabs < 1) slabs = 1;
    const int rows_per_slab = ceil_div(out, slabs);
    slabs = ceil_div(out, rows_per_slab);
    cudaStream_t st = (cudaStream_t)cuda_stream;
    // every partial that the second kernel reads is written by the first one of the same call: nothing needs clearing
    linear_ig_partial_kernel<float><<<dim3(col_blocks, slabs), 128, 0, st>>>(W, dy, part, out, in, rows_per_slab);
    count_launch();
    if (!TL_CUDA(cudaGetLastError())) return TL_ERR_CUDA;
    linear_ig_reduce_kernel<float><<<ceil_div(in, 32), 1024, 0, st>>>(part, dx, in, slabs);
    count_launch();
    if (!TL_CUDA(cudaGetLastError())) return TL_ERR_CUDA;
    return TL_OK;
}

namespace tl {

#define INST(T)                                                                                             \
    template void gemm<T>(const GemmDesc<T> &);                                                             \
    template void gemm_list<T>(const GemmDesc<T> &, const GemmList<T> &, int);                              \
    template void mm_contract<T>(const T *, const T *, T *, int, int, int, int, bool);                      \
    template void linear_fw_gemv<T>(const T *, const T *, const T *, T *, int, int);                        \
    template void linear_wg_outer<T>(const T *, const T *, T *, int, int);                                  \
    template bool linear_wg_streams<T>(Scope &, const T *, const T *, T *, int, int, int);                  \
    template void linear_ig_gemv<T>(Scope &, const T *, const T *, T *, int, int);
INST(float)
INST(__half)

} // namespace tl
