// Fused attention core of the multi-head self-attention layer.
//
// Forward: one kernel per (head, tile of queries) forms the scaled scores q^T k of its queries against all keys in
// shared memory, takes the row softmax there, writes the probabilities P once (the reference keeps them for the
// backward pass, so they are an output of the layer) and multiplies them with v before leaving: the scores never
// reach HBM and P is not read back  [ref: lib/sources/pulp_mhsa_fp32.c:348-560: per head a transpose, a matmul, a
// scalar multiply, a transpose, a softmax, a transpose and a matmul, each through memory].
//
// Backward: two kernels.  The query-tiled one recomputes nothing it can keep: dP = datt^T v for its queries is formed
// in shared memory (and written, because the reference exposes it as softmax_buffer.diff), turned into
// dS = (dP - sum_key dP P) P in place, and contracted with k into dq; it also leaves the row sums sum_key dP P behind.
// The key-tiled one rebuilds its columns of dS from P, dP and those row sums and contracts them with q and datt into
// dk and dv.  dS never reaches HBM  [ref: lib/sources/pulp_mhsa_fp32.c:842-1400].
//
// Layouts (reference convention): q, k, v, att and their gradients are F x L (token index fastest, head h owns rows
// h*H .. h*H+H-1); P and dP are heads x L x L indexed [head][query][key].  Every sum runs in a fixed order.
#include "tl_kernels.h"
#include "tl_reduce.cuh"

namespace tl {

static constexpr int ATT_THREADS = 256;
static constexpr int ATT_TQ = 4;                 // queries (or keys) per CTA = accumulators per thread (4 or 8).  Four: 256 CTAs for 4 heads x 256
                                                 // tokens, two per SM on most SMs; with eight (128 CTAs of 8 warps) the kernels ran at an eighth of the warp slots

// tile[t][j] = sum_d a_tile[d][t] * M[d][j]  for t < ATT_TQ, j < L: thread per column j, the H-long contraction in
// registers.  a_tile is [H][ATT_TQ] in shared memory (broadcast reads), M rows are read coalesced.
template <class T>
__device__ __forceinline__ void tile_from_rows(const float *a_tile, const T *__restrict__ M, float *tile, int Lp, int H, int L, float alpha)
{
    for (int j = threadIdx.x; j < L; j += ATT_THREADS) {
        float acc[ATT_TQ];
#pragma unroll
        for (int t = 0; t < ATT_TQ; t++) acc[t] = 0.f;
        for (int d = 0; d < H; d++) {
            const float m = ld(M + (size_t)d * L + j);
            const float4 a0 = *reinterpret_cast<const float4 *>(a_tile + d * ATT_TQ);
            acc[0] = fmaf(a0.x, m, acc[0]); acc[1] = fmaf(a0.y, m, acc[1]); acc[2] = fmaf(a0.z, m, acc[2]); acc[3] = fmaf(a0.w, m, acc[3]);
            if constexpr (ATT_TQ == 8) {
                const float4 a1 = *reinterpret_cast<const float4 *>(a_tile + d * ATT_TQ + 4);
                acc[4] = fmaf(a1.x, m, acc[4]); acc[5] = fmaf(a1.y, m, acc[5]); acc[6] = fmaf(a1.z, m, acc[6]); acc[7] = fmaf(a1.w, m, acc[7]);
            }
        }
#pragma unroll
        for (int t = 0; t < ATT_TQ; t++) tile[t * Lp + j] = __fmul_rn(acc[t], alpha);
    }
}

// out[d][t0 + t] = alpha * sum_j M[d][j] * tile[t][j]  for d < H, t < nt: a warp per row d, lanes over j (coalesced
// reads of M, conflict-free reads of the tile), butterfly reduction so that lane t holds the sum of column t.
template <class T>
__device__ __forceinline__ void rows_times_tile(const T *__restrict__ M, const float *tile, int Lp, int H, int L, T *__restrict__ out, int t0, int nt, float alpha)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int d = warp; d < H; d += ATT_THREADS / 32) {
        float acc[ATT_TQ];
#pragma unroll
        for (int t = 0; t < ATT_TQ; t++) acc[t] = 0.f;
        for (int j = lane; j < L; j += 32) {
            const float m = ld(M + (size_t)d * L + j);
#pragma unroll
            for (int t = 0; t < ATT_TQ; t++) acc[t] = fmaf(m, tile[t * Lp + j], acc[t]);
        }
        float mine = 0.f;
#pragma unroll
        for (int t = 0; t < ATT_TQ; t++) { const float s = warp_sum(acc[t]); if (lane == t) mine = s; }
        if (lane < nt) st(out + (size_t)d * L + t0 + lane, __fmul_rn(mine, alpha));
    }
}

// a_tile[d][t] = A[d][t0 + t] (zero beyond the last token)
template <class T>
__device__ __forceinline__ void load_a_tile(const T *__restrict__ A, float *a_tile, int H, int L, int t0)
{
    for (int i = threadIdx.x; i < H * ATT_TQ; i += ATT_THREADS) {
        const int d = i / ATT_TQ, t = i % ATT_TQ;
        a_tile[i] = (t0 + t < L) ? ld(A + (size_t)d * L + t0 + t) : 0.f;
    }
}

template <class T>
__global__ void __launch_bounds__(ATT_THREADS) attn_fw_kernel(const T *__restrict__ q, const T *__restrict__ k, const T *__restrict__ v,
                                                              T *__restrict__ P, T *__restrict__ att, int L, int H, float scaling)
{
    extern __shared__ __align__(16) float att_smem[];
    const int Lp = L + 1, head = blockIdx.y, t0 = blockIdx.x * ATT_TQ, nt = min(ATT_TQ, L - t0);
    float *a_tile = att_smem, *tile = att_smem + H * ATT_TQ;
    const size_t hoff = (size_t)head * H * L;
    load_a_tile(q + hoff, a_tile, H, L, t0);
    __syncthreads();
    tile_from_rows(a_tile, k + hoff, tile, Lp, H, L, scaling);
    __syncthreads();
    // row softmax, a warp per query: max, Schraudolph exp of (x - max), divide by the row sum  [ref: pulp_act_fp32.c:187-245]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp < nt) {
        float *row = tile + warp * Lp;
        float m = -FLT_MAX;
        for (int j = lane; j < L; j += 32) m = fmaxf(m, row[j]);
        m = warp_max(m);
        float s = 0.f;
        for (int j = lane; j < L; j += 32) { const float e = fastexp_gist_dev(__fsub_rn(row[j], m)); row[j] = e; s += e; }
        s = warp_sum(s);
        T *prow = P + ((size_t)head * L + t0 + warp) * L;
        for (int j = lane; j < L; j += 32) { const float p = __fdiv_rn(row[j], s); row[j] = p; st(prow + j, p); }
    } else if (warp < ATT_TQ) {
        float *row = tile + warp * Lp;
        for (int j = lane; j < L; j += 32) row[j] = 0.f;
    }
    __syncthreads();
    rows_times_tile(v + hoff, tile, Lp, H, L, att + hoff, t0, nt, 1.0f);
}

// Query-tiled half of the backward pass: dP (written), row sums of dP * P (written), dq (written).
template <class T>
__global__ void __launch_bounds__(ATT_THREADS) attn_bw_query_kernel(const T *__restrict__ datt, const T *__restrict__ v, const T *__restrict__ k,
                                                                    const T *__restrict__ P, T *__restrict__ dP, float *__restrict__ rowdot,
                                                                    T *__restrict__ dq, int L, int H, float scaling)
{
    extern __shared__ __align__(16) float att_smem[];
    const int Lp = L + 1, head = blockIdx.y, t0 = blockIdx.x * ATT_TQ, nt = min(ATT_TQ, L - t0);
    float *a_tile = att_smem, *tile = att_smem + H * ATT_TQ;
    const size_t hoff = (size_t)head * H * L;
    load_a_tile(datt + hoff, a_tile, H, L, t0);
    __syncthreads();
    tile_from_rows(a_tile, v + hoff, tile, Lp, H, L, 1.0f);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp < nt) {
        // dS = (dP - sum_key dP P) P   [ref: lib/sources/pulp_act_fp32.c:335-392]
        float *row = tile + warp * Lp;
        const size_t roff = ((size_t)head * L + t0 + warp) * L;
        float s = 0.f;
        for (int j = lane; j < L; j += 32) {
            float g = row[j];
            if (sizeof(T) == 2) g = __half2float(__float2half_rn(g));          // the value the caller sees in dP
            st(dP + roff + j, g);
            s = fmaf(g, ld(P + roff + j), s);
        }
        s = warp_sum(s);
        if (lane == 0) rowdot[(size_t)head * L + t0 + warp] = s;
        for (int j = lane; j < L; j += 32) {
            float g = row[j];
            if (sizeof(T) == 2) g = __half2float(__float2half_rn(g));
            row[j] = __fmul_rn(__fsub_rn(g, s), ld(P + roff + j));
        }
    } else if (warp < ATT_TQ) {
        float *row = tile + warp * Lp;
        for (int j = lane; j < L; j += 32) row[j] = 0.f;
    }
    __syncthreads();
    rows_times_tile(k + hoff, tile, Lp, H, L, dq + hoff, t0, nt, scaling);
}

// Key-tiled half: columns of P and of dS = (dP - rowdot) P for ATT_TQ keys against all queries, then
// dv[d][key] = sum_query datt[d][query] P[query][key] and dk[d][key] = scaling * sum_query q[d][query] dS[query][key].
template <class T>
__global__ void __launch_bounds__(ATT_THREADS) attn_bw_key_kernel(const T *__restrict__ datt, const T *__restrict__ q, const T *__restrict__ P,
                                                                  const T *__restrict__ dP, const float *__restrict__ rowdot,
                                                                  T *__restrict__ dk, T *__restrict__ dv, int L, int H, float scaling)
{
    extern __shared__ __align__(16) float att_smem[];
    const int Lp = L + 1, head = blockIdx.y, k0 = blockIdx.x * ATT_TQ, nk = min(ATT_TQ, L - k0);
    float *p_tile = att_smem, *ds_tile = att_smem + ATT_TQ * Lp;        // [key][query]
    const size_t hoff = (size_t)head * H * L;
    for (int i = threadIdx.x; i < L * ATT_TQ; i += ATT_THREADS) {
        const int query = i / ATT_TQ, kk = i % ATT_TQ;
        float p = 0.f, ds = 0.f;
        if (kk < nk) {
            const size_t off = ((size_t)head * L + query) * L + k0 + kk;
            p = ld(P + off);
            ds = __fmul_rn(__fsub_rn(ld(dP + off), rowdot[(size_t)head * L + query]), p);
        }
        p_tile[kk * Lp + query] = p; ds_tile[kk * Lp + query] = ds;
    }
    __syncthreads();
    rows_times_tile(datt + hoff, p_tile, Lp, H, L, dv + hoff, k0, nk, 1.0f);
    rows_times_tile(q + hoff, ds_tile, Lp, H, L, dk + hoff, k0, nk, scaling);
}

static size_t attn_smem_bytes(int L, int H, int tiles) { return ((size_t)H * ATT_TQ + (size_t)tiles * ATT_TQ * (L + 1)) * sizeof(float); }

// True when the fused kernels take this shape: the tiles of one CTA must fit in shared memory.
bool attn_fused_ok(int L, int H)
{
    return L >= 1 && H >= 1 && attn_smem_bytes(L, H, 2) <= 200 * 1024;
}

template <class T>
void attn_fw(const T *q, const T *k, const T *v, T *P, T *att, int L, int H, int heads, float scaling)
{
    const size_t smem = attn_smem_bytes(L, H, 1);
    if (smem > 48 * 1024) cudaFuncSetAttribute(attn_fw_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    TL_LAUNCH((attn_fw_kernel<T>), dim3(ceil_div(L, ATT_TQ), heads), ATT_THREADS, smem, q, k, v, P, att, L, H, scaling);
}

template <class T>
void attn_bw(const T *datt, const T *q, const T *k, const T *v, const T *P, T *dP, float *rowdot, T *dq, T *dk, T *dv,
             int L, int H, int heads, float scaling)
{
    const size_t smem1 = attn_smem_bytes(L, H, 1), smem2 = attn_smem_bytes(L, 0, 2);
    if (smem1 > 48 * 1024) cudaFuncSetAttribute(attn_bw_query_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1);
    if (smem2 > 48 * 1024) cudaFuncSetAttribute(attn_bw_key_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2);
    const dim3 grid(ceil_div(L, ATT_TQ), heads);
    TL_LAUNCH((attn_bw_query_kernel<T>), grid, ATT_THREADS, smem1, datt, v, k, P, dP, rowdot, dq, L, H, scaling);
    TL_LAUNCH((attn_bw_key_kernel<T>), grid, ATT_THREADS, smem2, datt, q, P, dP, rowdot, dk, dv, L, H, scaling);
}

#define INST(T)                                                                                                        \
    template void attn_fw<T>(const T *, const T *, const T *, T *, T *, int, int, int, float);                        \
    template void attn_bw<T>(const T *, const T *, const T *, const T *, const T *, T *, float *, T *, T *, T *, int, int, int, float);
INST(float)
INST(__half)

} // namespace tl
