// TMA-fed tensor-core GEMM for the large products of the `mm` family
// [ref: lib/sources/pulp_matmul_fp32.c:190-262, lib/sources/pulp_matmul_fp16.c:191-262]:
//     C[N x M] = alpha * A[N x K] * B[K x M] (+ bias) (+ C)
// Both operands are taken K-major ("A row-major, B as its transpose [M x K]").  An operand that is stored the other
// way round, or whose rows do not start on 16-byte boundaries, is first packed into K-major scratch by a tiled
// transpose; fp32 operands are packed anyway because 3xTF32 needs the (hi, lo) pair of every value.
//
// Kernel: one CTA per 128 x BN tile of C.  A producer thread issues cp.async.bulk.tensor (3-D: k, row, batch;
// 128-byte swizzle; out-of-range rows and k read as zero, so no tail code) into a ring of shared-memory stages;
// an issuer thread runs tcgen05.mma from shared-memory descriptors (K advances by 32 bytes inside the 128-byte
// swizzle atom) with the accumulator in tensor memory and releases each stage with tcgen05.commit; four warps
// read the accumulator with tcgen05.ld and write C (any strides).
//   fp16: kind::f16, BN = 256, 64 halves of K per stage, 4 stages of 48 KB.
//   fp32: kind::tf32 three times per K slice (hi*hi + hi*lo + lo*hi) into one accumulator, BN = 128, 32 floats of K
//         per stage, 3 stages of 64 KB (A_hi, A_lo, B_hi, B_lo).
// No multicast, one CTA per tile.  Every wait is bounded and reports through the library's status word.
#include "tl_kernels.h"
#include "tl_tc.cuh"

namespace tl {

using namespace tc;

int *tc_status_word();          // tl_conv_tc.cu
void *tc_encode_tiled_fn();     // tl_conv_tc.cu: cuTensorMapEncodeTiled through the runtime's driver entry point query

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static constexpr int TM_BM = 128;
static constexpr int TM_THREADS = 192;          // warps 0-3: epilogue, warp 4: TMA producer, warp 5: MMA issuer

template <class T> struct TmCfg;
template <> struct TmCfg<__half> { static constexpr int BN = 256, BK = 64, STAGES = 4, PARTS = 1, DCOLS = 256; };
template <> struct TmCfg<float>  { static constexpr int BN = 128, BK = 32, STAGES = 3, PARTS = 2, DCOLS = 128; };

struct TmParams {
    void *C; const void *bias;
    int N, M, K;
    long long c_rs, c_cs, c_bs;
    float alpha; int accumulate, bias_mode;
    int *status;
};

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *m, uint64_t *bar, int x, int y, int z)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ bool tm_wait(uint64_t *bar, uint32_t parity, volatile int *failed)
{
    for (uint32_t i = 0; i < 50000u; i++) {
        if (mbar_try_wait_hint(bar, parity, 20000u)) return true;
        if (*failed) return false;
    }
    *failed = 1;
    return false;
}

// maps: a0 = A (hi), a1 = A lo (fp32 only), b0 = B (hi), b1 = B lo
template <class T>
__global__ void __launch_bounds__(TM_THREADS) gemm_tma_kernel(const __grid_constant__ CUtensorMap a0, const __grid_constant__ CUtensorMap a1,
                                                              const __grid_constant__ CUtensorMap b0, const __grid_constant__ CUtensorMap b1, TmParams p)
{
    typedef TmCfg<T> Cfg;
    constexpr int BN = Cfg::BN, BK = Cfg::BK, ST = Cfg::STAGES;
    constexpr uint32_t A_BYTES = TM_BM * 128u, B_BYTES = BN * 128u;                // one 128-byte row per tile row
    constexpr uint32_t STAGE_BYTES = Cfg::PARTS * (A_BYTES + B_BYTES);
    extern __shared__ unsigned char tsm_raw[];
    const uint32_t sbase = (smem_u32(tsm_raw) + 1023u) & ~1023u;                    // swizzle atoms want 1024-byte alignment
    unsigned char *aligned = tsm_raw + (sbase - smem_u32(tsm_raw));
    uint64_t *full = reinterpret_cast<uint64_t *>(aligned + ST * STAGE_BYTES);
    uint64_t *empty = full + ST, *done = empty + ST;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(done + 1);
    volatile int *failed = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int col0 = blockIdx.x * BN, row0 = blockIdx.y * TM_BM, b = blockIdx.z;

    if (tid == 0) {
        for (int s = 0; s < ST; s++) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(done, 1);
        *failed = 0;
        fence_barrier_init();
        tma_prefetch_desc(&a0); tma_prefetch_desc(&b0);
        if (Cfg::PARTS == 2) { tma_prefetch_desc(&a1); tma_prefetch_desc(&b1); }
    }
    if (warp == 0) { tmem_alloc(tmem_slot, Cfg::DCOLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t d_tmem = *tmem_slot;
    const int ksteps = (p.K + BK - 1) / BK;

    if (warp == 4) {
        if (lane == 0) {
            for (int kt = 0; kt < ksteps; kt++) {
                const int s = kt % ST, use = kt / ST;
                if (use > 0 && !tm_wait(&empty[s], (uint32_t)(use - 1) & 1u, failed)) break;
                const uint32_t st = sbase + s * STAGE_BYTES;
                mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                tma_load_3d(st, &a0, &full[s], kt * BK, row0, b);
                if (Cfg::PARTS == 2) tma_load_3d(st + A_BYTES, &a1, &full[s], kt * BK, row0, b);
                tma_load_3d(st + Cfg::PARTS * A_BYTES, &b0, &full[s], kt * BK, col0, b);
                if (Cfg::PARTS == 2) tma_load_3d(st + 2 * A_BYTES + B_BYTES, &b1, &full[s], kt * BK, col0, b);
            }
        }
    } else if (warp == 5) {
        if (lane == 0) {
            constexpr uint32_t idesc = mma_idesc(sizeof(T) == 2 ? FMT_F16 : FMT_TF32, TM_BM, BN);
            bool ok = true;
            for (int kt = 0; kt < ksteps && ok; kt++) {
                const int s = kt % ST, use = kt / ST;
                if (!tm_wait(&full[s], (uint32_t)use & 1u, failed)) { ok = false; break; }
                tc_fence_after();
                const uint32_t st = sbase + s * STAGE_BYTES;
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {            // 4 MMAs of 32 bytes of K each per 128-byte row
                    const uint32_t acc = (kt > 0 || kk > 0) ? 1u : 0u;
                    if constexpr (sizeof(T) == 2) {
                        mma_f16_ss(d_tmem, smem_desc_kmajor_sw128(st + kk * 32, 1024), smem_desc_kmajor_sw128(st + A_BYTES + kk * 32, 1024), idesc, acc);
                    } else {
                        const uint64_t ah = smem_desc_kmajor_sw128(st + kk * 32, 1024), al = smem_desc_kmajor_sw128(st + A_BYTES + kk * 32, 1024);
                        const uint64_t bh = smem_desc_kmajor_sw128(st + 2 * A_BYTES + kk * 32, 1024), bl = smem_desc_kmajor_sw128(st + 2 * A_BYTES + B_BYTES + kk * 32, 1024);
                        mma_tf32_ss(d_tmem, ah, bh, idesc, acc);
                        mma_tf32_ss(d_tmem, ah, bl, idesc, 1u);
                        mma_tf32_ss(d_tmem, al, bh, idesc, 1u);
                    }
                }
                mma_commit(&empty[s]);
            }
            if (ok) mma_commit(done);
        }
    } else {
        // epilogue: warp w owns TMEM lanes 32w .. 32w+31 = rows row0 + 32w + lane
        bool ok = true;
        if (lane == 0) ok = tm_wait(done, 0, failed);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        tc_fence_after();
        if (ok) {
            const int row = row0 + warp * 32 + lane;
            const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
            T *crow = reinterpret_cast<T *>(p.C) + (long long)b * p.c_bs + (long long)row * p.c_rs;
            const T *bias = reinterpret_cast<const T *>(p.bias);
            const float brow = (p.bias_mode == 1 && row < p.N) ? ld(bias + row) : 0.f;
            const bool vec = p.c_cs == 1 && !p.accumulate && ((uintptr_t)crow & 15) == 0 && (col0 % 8) == 0;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 16) {
                uint32_t v[16];
                tmem_ld16(d_tmem + lane_addr + c0, v);
                tmem_wait_ld();
                if (row >= p.N || col0 + c0 >= p.M) continue;
                float r[16];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    r[j] = p.alpha * __uint_as_float(v[j]) + brow;
                    if (p.bias_mode == 2 && col0 + c0 + j < p.M) r[j] += ld(bias + col0 + c0 + j);
                }
                if (vec && col0 + c0 + 16 <= p.M) {
                    if constexpr (sizeof(T) == 2) {
                        uint32_t w[8];
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            __half2 h = __floats2half2_rn(r[2 * j], r[2 * j + 1]);
                            w[j] = *reinterpret_cast<uint32_t *>(&h);
                        }
                        uint4 *dst = reinterpret_cast<uint4 *>(crow + col0 + c0);
                        dst[0] = make_uint4(w[0], w[1], w[2], w[3]); dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
                    } else {
                        float4 *dst = reinterpret_cast<float4 *>(crow + col0 + c0);
#pragma unroll
                        for (int j = 0; j < 4; j++) dst[j] = make_float4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int col = col0 + c0 + j;
                        if (col < p.M) {
                            T *dst = crow + (long long)col * p.c_cs;
                            st(dst, p.accumulate ? r[j] + ld(dst) : r[j]);
                        }
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (*failed && tid == 0) atomicCAS(p.status, 0, 8);
    if (warp == 0) tmem_dealloc(d_tmem, Cfg::DCOLS);
}

// ---------------------------------------------------------------- operand packing
// dst[(b * rows + r) * Kp + k] = src[b*bs + r*rs + k*cs] for k < K (columns K..Kp-1 are never read: the tensor map
// ends at K).  fp32: hi part to dst, lo part to dst_lo.  32 x 32 tiles through shared memory so that both the
// global reads (along whichever index has the smaller stride) and the writes (along k) are coalesced.
template <class T>
__global__ void __launch_bounds__(256) pack_kmajor_kernel(const T *__restrict__ src, long long rs, long long cs, long long bs,
                                                          T *__restrict__ dst, T *__restrict__ dst_lo, int rows, int K, int Kp)
{
    __shared__ float tile[32][33];
    const int r0 = blockIdx.y * 32, k0 = blockIdx.x * 32, b = blockIdx.z;
    const T *s = src + (long long)b * bs;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const bool along_r = rs == 1 || (cs != 1 && llabs(rs) < llabs(cs));           // read with tx along the row index
    for (int i = ty; i < 32; i += 8) {
        const int r = along_r ? r0 + tx : r0 + i, k = along_r ? k0 + i : k0 + tx;
        float v = 0.f;
        if (r < rows && k < K) v = ld(s + (long long)r * rs + (long long)k * cs);
        tile[r - r0][k - k0] = v;
    }
    __syncthreads();
    for (int i = ty; i < 32; i += 8) {
        const int r = r0 + i, k = k0 + tx;
        if (r < rows && k < Kp) {
            const float v = tile[i][tx];
            const long long o = ((long long)b * rows + r) * Kp + k;
            if constexpr (sizeof(T) == 4) {
                uint32_t hi, lo;
                split_tf32(v, hi, lo);
                dst[o] = __uint_as_float(hi); dst_lo[o] = __uint_as_float(lo);
            } else {
                st(dst + o, v);
            }
        }
    }
}

template <class T> static bool make_map(EncodeTiledFn enc, CUtensorMap *m, const T *base, int K, int rows, int batch, long long rs, long long bs, int box_rows)
{
    constexpr int BK = TmCfg<T>::BK;
    cuuint64_t gdim[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t gstr[2] = {(cuuint64_t)rs * sizeof(T), (cuuint64_t)(batch > 1 ? bs : (long long)rows * rs) * sizeof(T)};
    cuuint32_t box[3] = {(cuuint32_t)BK, (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[3] = {1, 1, 1};
    return enc(m, sizeof(T) == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, (void *)base, gdim, gstr, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Returns false when the product should go to the other kernels (too small, or no tensor-map encoder).
template <class T> bool gemm_tensor_core_tma(const GemmDesc<T> &d)
{
    typedef TmCfg<T> Cfg;
    if (d.N < 1 || d.M < 1 || d.K < 1 || d.batch < 1) return false;
    if (gemm_path() != 3) {      // 3 = forced (tests): every shape, the tails come from the tensor maps' zero fill
        if (d.N < TM_BM || d.M < Cfg::BN / 2 || d.K < 2 * Cfg::BK) return false;
        if ((long long)d.N * d.M * d.K * d.batch < (1ll << 26)) return false;
    }
    EncodeTiledFn enc = (EncodeTiledFn)tc_encode_tiled_fn();
    int *status = tc_status_word();
    if (!enc || !status) return false;
    Scope sc;
    if (!sc.ok()) return false;
    constexpr long long EB = 16 / (long long)sizeof(T);
    const int Kp = (int)(((long long)d.K + EB - 1) / EB * EB);
    // operands as K-major [rows][K]: in place when fp16 is already laid out that way, packed otherwise
    struct Op { const T *hi, *lo; long long rs, bs; };
    auto prepare = [&](const T *src, long long rs, long long cs, long long bs, int rows, Op &o) -> bool {
        const bool in_place = sizeof(T) == 2 && cs == 1 && rs % EB == 0 && (d.batch == 1 || bs % EB == 0) && ((uintptr_t)src & 15) == 0;
        if (in_place) { o.hi = src; o.lo = nullptr; o.rs = rs; o.bs = bs; return true; }
        const size_t count = (size_t)d.batch * rows * Kp;
        T *hi = sc.scratch<T>(count), *lo = sizeof(T) == 4 ? sc.scratch<T>(count) : nullptr;
        if (!hi || (sizeof(T) == 4 && !lo)) return false;
        dim3 grid(ceil_div(Kp, 32), ceil_div(rows, 32), d.batch);
        TL_LAUNCH((pack_kmajor_kernel<T>), grid, 256, 0, src, rs, cs, bs, hi, lo, rows, d.K, Kp);
        o.hi = hi; o.lo = lo; o.rs = Kp; o.bs = (long long)rows * Kp;
        return true;
    };
    Op a, b;
    if (!prepare(d.A, d.a_rs, d.a_cs, d.a_bs, d.N, a)) return false;
    if (!prepare(d.B, d.b_cs, d.b_rs, d.b_bs, d.M, b)) return false;     // row of the B operand = column of C
    CUtensorMap ma0, ma1, mb0, mb1;
    if (!make_map<T>(enc, &ma0, a.hi, d.K, d.N, d.batch, a.rs, a.bs, TM_BM)) return false;
    if (!make_map<T>(enc, &mb0, b.hi, d.K, d.M, d.batch, b.rs, b.bs, Cfg::BN)) return false;
    ma1 = ma0; mb1 = mb0;
    if (sizeof(T) == 4) {
        if (!make_map<T>(enc, &ma1, a.lo, d.K, d.N, d.batch, a.rs, a.bs, TM_BM)) return false;
        if (!make_map<T>(enc, &mb1, b.lo, d.K, d.M, d.batch, b.rs, b.bs, Cfg::BN)) return false;
    }
    TmParams p;
    p.C = d.C; p.bias = d.bias; p.N = d.N; p.M = d.M; p.K = d.K;
    p.c_rs = d.c_rs; p.c_cs = d.c_cs; p.c_bs = d.c_bs;
    p.alpha = d.alpha; p.accumulate = d.accumulate ? 1 : 0; p.bias_mode = d.bias ? d.bias_mode : 0;
    p.status = status;
    constexpr uint32_t STAGE_BYTES = Cfg::PARTS * (TM_BM * 128u + Cfg::BN * 128u);
    const size_t smem = (size_t)Cfg::STAGES * STAGE_BYTES + (2 * Cfg::STAGES + 1) * 8 + 16 + 1024;
    static bool attr_set = false;
    if (!attr_set) { cudaFuncSetAttribute(gemm_tma_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); attr_set = true; }
    dim3 grid(ceil_div(d.M, Cfg::BN), ceil_div(d.N, TM_BM), d.batch);
    TL_LAUNCH((gemm_tma_kernel<T>), grid, TM_THREADS, smem, ma0, ma1, mb0, mb1, p);
    return true;
}
template bool gemm_tensor_core_tma<float>(const GemmDesc<float> &);
template bool gemm_tensor_core_tma<__half>(const GemmDesc<__half> &);

} // namespace tl
