// Tensor-core GEMM for the `mm` family (tcgen05.mma, accumulators in tensor memory):
//     C[N x M] = alpha * A[N x K] * B[K x M] (+ bias) (+ C),   arbitrary element strides, optional batch.
// Replaces the scalar products of the reference [ref: lib/sources/pulp_matmul_fp32.c:190-262 (mm), :264-340 (mm_M);
// lib/sources/pulp_matmul_fp16.c:191-262] for shapes large enough to fill 128 x BN tensor-core tiles.
//
// One CTA computes a 128 x BN tile of C.  Per K step of 8 sixteen-byte chunks (64 halves or 32 floats) all 256
// threads copy the A and B slices from global memory (any strides; 16-byte loads when K is the contiguous index,
// lane-coalesced scalar loads when the row index is) into shared memory in the tensor core's K-major
// "8 rows x 16 bytes" core-matrix layout, then one thread issues the MMAs of that stage and commits them to the
// stage's mbarrier; the copy of the next stage overlaps them (3 stages).
//   fp16: kind::f16, fp32 accumulation, BN = 128.
//   fp32: 3xTF32.  Every value is split into hi + lo while it is copied; B holds [hi rows | lo rows] so that
//         D'[:, 0:2BN] += A_hi [B_hi | B_lo]^T  and  D'[:, 0:BN] += A_lo B_hi^T  (BN = 64); the epilogue adds the
//         two halves.  The lo*lo term is below fp32 resolution.
// Every wait is bounded; a wait that gives up sets a status word the host reads (trainlib_tc_status()).
#include "tl_kernels.h"
#include "tl_tc.cuh"

namespace tl {

using namespace tc;

static constexpr int GT_THREADS = 256;
static constexpr int GT_BM = 128;          // rows of C per CTA = MMA M = TMEM lanes
static constexpr int GT_NCH = 8;           // 16-byte K chunks per stage
static constexpr int GT_STAGES = 3;

template <class T> struct GtCfg;
template <> struct GtCfg<__half> { static constexpr int KC = 8, BN = 128, B_ROWS = 128, A_PARTS = 1, DCOLS = 128; };
template <> struct GtCfg<float>  { static constexpr int KC = 4, BN = 64,  B_ROWS = 128, A_PARTS = 2, DCOLS = 128; };

struct GtParams {
    const void *A, *B; void *C; const void *bias;
    int N, M, K;
    long long a_rs, a_cs, b_rs, b_cs, c_rs, c_cs, a_bs, b_bs, c_bs;
    float alpha; int accumulate, bias_mode;
    int a_vec, b_vec;          // 1: K is the contiguous index and 16-byte loads are legal for this operand
    int *status;
};

// byte distance between K chunks of an operand block of `rows` rows: one extra 16 bytes so that the eight chunks
// of one row fall into different banks when a quarter warp stores them
__host__ __device__ constexpr uint32_t gt_lbo(int rows) { return (uint32_t)rows * 16u + 16u; }
__host__ __device__ constexpr uint32_t gt_block_bytes(int rows) { return gt_lbo(rows) * GT_NCH; }

__device__ __forceinline__ uint32_t pack_half2(__half a, __half b) { return (uint32_t)__half_as_ushort(a) | ((uint32_t)__half_as_ushort(b) << 16); }

// Copies rows [row0, row0+ROWS) x K range [k0, k0 + NCH*KC) of an operand (element (r, k) at base[r*rs + k*cs]) into
// shared memory; rows >= rows_valid and k >= K read as zero.  fp32: hi part to dst, lo part to dst_lo.
template <class T, int ROWS, int BLOCK_ROWS>
__device__ __forceinline__ void gt_stage(const T *__restrict__ base, long long rs, long long cs, int rows_valid, int K, int row0, int k0,
                                         uint32_t dst, uint32_t dst_lo, int vec)
{
    constexpr int KC = GtCfg<T>::KC;
    constexpr uint32_t LBO = gt_lbo(BLOCK_ROWS);     // the block may hold more rows than are copied here (fp32 B: hi | lo)
    const int tid = threadIdx.x;
    if (vec) {
        // 8 consecutive lanes read the 8 chunks (128 contiguous bytes) of one row
        for (int item = tid; item < ROWS * GT_NCH; item += GT_THREADS) {
            const int c = item % GT_NCH, r = item / GT_NCH;
            const int k = k0 + c * KC;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (row0 + r < rows_valid && k < K) {
                const T *p = base + (long long)(row0 + r) * rs + k;
                if (k + KC <= K) v = __ldg(reinterpret_cast<const uint4 *>(p));
                else {
                    __align__(16) T t[KC];
#pragma unroll
                    for (int j = 0; j < KC; j++) t[j] = (k + j < K) ? p[j] : T(0.f);
                    v = *reinterpret_cast<uint4 *>(t);
                }
            }
            const uint32_t off = (uint32_t)c * LBO + (uint32_t)(r >> 3) * 128u + (uint32_t)(r & 7) * 16u;
            if constexpr (sizeof(T) == 2) {
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + off), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
            } else {
                uint32_t h[4], l[4];
                split_tf32(__uint_as_float(v.x), h[0], l[0]); split_tf32(__uint_as_float(v.y), h[1], l[1]);
                split_tf32(__uint_as_float(v.z), h[2], l[2]); split_tf32(__uint_as_float(v.w), h[3], l[3]);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + off), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst_lo + off), "r"(l[0]), "r"(l[1]), "r"(l[2]), "r"(l[3]) : "memory");
            }
        }
    } else {
        // consecutive lanes take consecutive rows of one chunk: each of the KC scalar loads is coalesced when the
        // row index is the contiguous one, and the 16-byte shared stores of a quarter warp are contiguous
        for (int item = tid; item < ROWS * GT_NCH; item += GT_THREADS) {
            const int r = item % ROWS, c = item / ROWS;
            const int k = k0 + c * KC;
            float t[KC];
#pragma unroll
            for (int j = 0; j < KC; j++)
                t[j] = (row0 + r < rows_valid && k + j < K) ? ld(base + (long long)(row0 + r) * rs + (long long)(k + j) * cs) : 0.f;
            const uint32_t off = (uint32_t)c * LBO + (uint32_t)(r >> 3) * 128u + (uint32_t)(r & 7) * 16u;
            if constexpr (sizeof(T) == 2) {
                uint32_t w[4];
#pragma unroll
                for (int j = 0; j < 4; j++) w[j] = pack_half2(__float2half_rn(t[2 * j]), __float2half_rn(t[2 * j + 1]));
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + off), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
            } else {
                uint32_t h[4], l[4];
#pragma unroll
                for (int j = 0; j < 4; j++) split_tf32(t[j], h[j], l[j]);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst + off), "r"(h[0]), "r"(h[1]), "r"(h[2]), "r"(h[3]) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst_lo + off), "r"(l[0]), "r"(l[1]), "r"(l[2]), "r"(l[3]) : "memory");
            }
        }
    }
}

template <class T>
__global__ void __launch_bounds__(GT_THREADS) gemm_tc_kernel(GtParams p)
{
    typedef GtCfg<T> Cfg;
    constexpr int BN = Cfg::BN;
    constexpr uint32_t A_BYTES = gt_block_bytes(GT_BM), B_BYTES = gt_block_bytes(BN);
    // stage layout: A (hi) | A lo (fp32 only) | B hi rows | B lo rows (fp32 only, directly behind the hi rows of each chunk)
    constexpr uint32_t BBLK = (sizeof(T) == 4) ? gt_block_bytes(2 * BN) : B_BYTES;
    constexpr uint32_t STAGE_BYTES = Cfg::A_PARTS * A_BYTES + BBLK;
    extern __shared__ __align__(128) unsigned char gsm[];
    uint64_t *empty = reinterpret_cast<uint64_t *>(gsm + GT_STAGES * STAGE_BYTES);
    uint64_t *done = empty + GT_STAGES;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(done + 1);
    __shared__ int failed;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col0 = blockIdx.x * BN, row0 = blockIdx.y * GT_BM, b = blockIdx.z;
    const T *A = reinterpret_cast<const T *>(p.A) + (long long)b * p.a_bs;
    const T *B = reinterpret_cast<const T *>(p.B) + (long long)b * p.b_bs;
    T *C = reinterpret_cast<T *>(p.C) + (long long)b * p.c_bs;

    if (tid == 0) {
        for (int s = 0; s < GT_STAGES; s++) mbar_init(&empty[s], 1);
        mbar_init(done, 1);
        failed = 0;
        fence_barrier_init();
    }
    if (warp == 0) { tmem_alloc(tmem_slot, Cfg::DCOLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t d_tmem = *tmem_slot;
    const uint32_t sbase = smem_u32(gsm);

    const int ksteps = (p.K + GT_NCH * Cfg::KC - 1) / (GT_NCH * Cfg::KC);
    bool ok = true;
    for (int kt = 0; kt < ksteps; kt++) {
        const int s = kt % GT_STAGES, use = kt / GT_STAGES;
        if (use > 0 && ok) {
            // the MMAs that read this stage GT_STAGES steps ago must have finished
            if (!mbar_wait(&empty[s], (uint32_t)(use - 1) & 1u)) { ok = false; failed = 1; }
        }
        const uint32_t a_s = sbase + s * STAGE_BYTES, b_s = a_s + Cfg::A_PARTS * A_BYTES;
        const int k0 = kt * GT_NCH * Cfg::KC;
        if constexpr (sizeof(T) == 4) {
            gt_stage<T, GT_BM, GT_BM>(A, p.a_rs, p.a_cs, p.N, p.K, row0, k0, a_s, a_s + A_BYTES, p.a_vec);
            // B: row = column of C.  hi rows 0..BN-1 and lo rows BN..2BN-1 of a 2BN-row block
            gt_stage<T, BN, 2 * BN>(B, p.b_cs, p.b_rs, p.M, p.K, col0, k0, b_s, b_s + (uint32_t)(BN / 8) * 128u, p.b_vec);
        } else {
            gt_stage<T, GT_BM, GT_BM>(A, p.a_rs, p.a_cs, p.N, p.K, row0, k0, a_s, 0u, p.a_vec);
            gt_stage<T, BN, BN>(B, p.b_cs, p.b_rs, p.M, p.K, col0, k0, b_s, 0u, p.b_vec);
        }
        fence_proxy_async();
        __syncthreads();
        if (tid == 0 && ok && !failed) {
            tc_fence_after();
            if constexpr (sizeof(T) == 2) {
                constexpr uint32_t idesc = mma_idesc(FMT_F16, GT_BM, BN);
#pragma unroll
                for (int kk = 0; kk < GT_NCH / 2; kk++) {          // K = 16 halves = 2 chunks per MMA
                    const uint64_t ad = smem_desc_kmajor(a_s + kk * 2 * gt_lbo(GT_BM), gt_lbo(GT_BM), 128);
                    const uint64_t bd = smem_desc_kmajor(b_s + kk * 2 * gt_lbo(BN), gt_lbo(BN), 128);
                    mma_f16_ss(d_tmem, ad, bd, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
                }
            } else {
                constexpr uint32_t idesc_2n = mma_idesc(FMT_TF32, GT_BM, 2 * BN), idesc_n = mma_idesc(FMT_TF32, GT_BM, BN);
#pragma unroll
                for (int kk = 0; kk < GT_NCH / 2; kk++) {          // K = 8 floats = 2 chunks per MMA
                    const uint64_t ah = smem_desc_kmajor(a_s + kk * 2 * gt_lbo(GT_BM), gt_lbo(GT_BM), 128);
                    const uint64_t al = smem_desc_kmajor(a_s + A_BYTES + kk * 2 * gt_lbo(GT_BM), gt_lbo(GT_BM), 128);
                    const uint64_t bd = smem_desc_kmajor(b_s + kk * 2 * gt_lbo(2 * BN), gt_lbo(2 * BN), 128);
                    mma_tf32_ss(d_tmem, ah, bd, idesc_2n, (kt > 0 || kk > 0) ? 1u : 0u);
                    mma_tf32_ss(d_tmem, al, bd, idesc_n, 1u);
                }
            }
            mma_commit(&empty[s]);
            if (kt == ksteps - 1) mma_commit(done);
        }
        // no barrier here: the next iteration writes another stage, and re-use of this one waits on empty[s]
    }
    __syncthreads();
    if (failed) ok = false;
    if (ok && !mbar_wait(done, 0)) { ok = false; failed = 1; }
    tc_fence_after();
    if (ok) {
        // warp w reads TMEM lanes 32*(w%4).. (its quarter) and one half of the columns
        const int q = warp & 3, half = warp >> 2;
        const int row = row0 + q * 32 + lane;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        constexpr int CPW = BN / 2;                                // columns per warp
#pragma unroll 1
        for (int c0 = half * CPW; c0 < (half + 1) * CPW; c0 += 16) {
            uint32_t v[16];
            tmem_ld16(d_tmem + lane_addr + c0, v);
            if constexpr (sizeof(T) == 4) {
                uint32_t w[16];
                tmem_ld16(d_tmem + lane_addr + BN + c0, w);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
            } else {
                tmem_wait_ld();
            }
            if (row < p.N) {
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const int col = col0 + c0 + j;
                    if (col < p.M) {
                        float r = p.alpha * __uint_as_float(v[j]);
                        if (p.bias_mode == 1) r += ld(reinterpret_cast<const T *>(p.bias) + row);
                        else if (p.bias_mode == 2) r += ld(reinterpret_cast<const T *>(p.bias) + col);
                        T *dst = C + (long long)row * p.c_rs + (long long)col * p.c_cs;
                        if (p.accumulate) r += ld(dst);
                        st(dst, r);
                    }
                }
            }
        }
    }
    if (!ok && tid == 0) atomicCAS(p.status, 0, 7);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(d_tmem, Cfg::DCOLS);
}

int *tc_status_word();      // tl_conv_tc.cu

template <class T> bool gemm_tensor_core(const GemmDesc<T> &d)
{
    typedef GtCfg<T> Cfg;
    if (d.N < 1 || d.M < 1 || d.K < 1 || d.batch < 1) return false;
    if (gemm_path() != 2) {
        // tiles of 128 x BN: small or skinny products stay on the FFMA tiles.  Those also add in the reference's
        // order (k ascending, one accumulator), which keeps chains of small products such as the attention
        // backward at L = 256 inside 1e-5 of the reference; the tensor cores add in another order.
        if (d.N < 96 || d.M < 48 || d.K < 64) return false;
        if ((long long)d.N * d.M * d.K * d.batch < (1ll << 26)) return false;
    }
    int *status = tc_status_word();
    if (!status) return false;
    GtParams p;
    p.A = d.A; p.B = d.B; p.C = d.C; p.bias = d.bias;
    p.N = d.N; p.M = d.M; p.K = d.K;
    p.a_rs = d.a_rs; p.a_cs = d.a_cs; p.b_rs = d.b_rs; p.b_cs = d.b_cs; p.c_rs = d.c_rs; p.c_cs = d.c_cs;
    p.a_bs = d.a_bs; p.b_bs = d.b_bs; p.c_bs = d.c_bs;
    p.alpha = d.alpha; p.accumulate = d.accumulate ? 1 : 0; p.bias_mode = d.bias ? d.bias_mode : 0;
    const long long eb = 16 / (long long)sizeof(T);
    p.a_vec = (d.a_cs == 1 && d.a_rs % eb == 0 && d.a_bs % eb == 0 && ((uintptr_t)d.A & 15) == 0) ? 1 : 0;
    p.b_vec = (d.b_rs == 1 && d.b_cs % eb == 0 && d.b_bs % eb == 0 && ((uintptr_t)d.B & 15) == 0) ? 1 : 0;
    p.status = status;
    constexpr uint32_t BBLK = (sizeof(T) == 4) ? gt_block_bytes(2 * Cfg::BN) : gt_block_bytes(Cfg::BN);
    constexpr uint32_t STAGE_BYTES = Cfg::A_PARTS * gt_block_bytes(GT_BM) + BBLK;
    const size_t smem = (size_t)GT_STAGES * STAGE_BYTES + (GT_STAGES + 1) * 8 + 16;
    static bool attr_set = false;
    if (!attr_set) { cudaFuncSetAttribute(gemm_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr_set = true; }
    dim3 grid(ceil_div(d.M, Cfg::BN), ceil_div(d.N, GT_BM), d.batch);
    TL_LAUNCH((gemm_tc_kernel<T>), grid, GT_THREADS, smem, p);
    return true;
}
template bool gemm_tensor_core<float>(const GemmDesc<float> &);
template bool gemm_tensor_core<__half>(const GemmDesc<__half> &);

} // namespace tl
