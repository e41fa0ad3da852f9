// Width-preserving stride-1 convolution (forward, stride-1 input gradient, parity classes of a strided input
// gradient) as an implicit GEMM on the 5th-generation tensor cores, 3xTF32 split-precision fp32, with the input
// split into its TF32 parts ONCE per element.
//
//   D[pixel][(b, co)] = sum_{a, ci} X[ci][row(pixel) + a - padU][col(pixel)] * Wt[co][ci][a][b]
//   Y[co][pixel]      = sum_b D[pixel + (b - padL)][(b, co)]                     (b - padL stays inside the image row)
//
// i.e. the filter columns b are moved from the contraction index into the GEMM's N dimension, so the A operand
// never needs a copy of the input shifted by one float: for every filter row `a` and group of eight input channels
// it is the very block of image rows that TMA dropped into shared memory, read by the tensor core as an MN-major
// (pixel-contiguous) operand through a descriptor whose start address moves by whole rows.  The column shift is
// paid in the epilogue, where thread = pixel and a warp = whole image rows: one warp shuffle per filter column.
//
// Shared-memory "row slots": one slot = 8 channels x 32 pixels = 8 rows of 128 bytes, the unit of the only MN-major
// layout kind::tf32 accepts (128-byte swizzle with 32-byte atoms).  The 32 pixels are one image row of P = 32 / W
// streams side by side (W = 32 / 16 / 8 -> P = 1 / 2 / 4), which is what one row of a TMA box {W, P streams,
// 8 channels, rows} of the tensor map (x, stream, channel, row) produces (unswizzled: a swizzling TMA copy pads
// rows shorter than 128 bytes, so the converters apply the swizzle while they split).  A block of 128 output pixels (one MMA,
// "m-block") is 4 consecutive slots = 4 image rows of P streams; filter row `a` reads the slots `a` further down.
//
// Pipeline per CTA (persistent, one per SM): a TMA thread fills a ring of stages (one stage = all slots of one
// 8-channel group of one tile); four converter warps replace every raw value by its TF32 "big" part in place and
// write the "small" part to the stage's second array (one load, two stores per element); NI issuing threads, each
// owning one m-block of the tile and its private accumulator in tensor memory, issue per (channel group, filter row)
//     D[:, 0:2NB] (+)= A_hi * [B_hi | B_lo]^T      D[:, 0:NB] += A_lo * B_hi^T        (or three NB-wide MMAs when 2NB > 256)
// and hand the stage back with tcgen05.commit; 4 epilogue warps per issuer read D with tcgen05.ld, add the halves,
// shift-sum the filter columns and store the output.  Every accumulator has one issuing thread that adds in a fixed
// order, so results are bit-reproducible from run to run.
//
// Replaces the im2col + mm lowering [ref: lib/sources/pulp_conv2d_fp32.c:85-113, :504-549;
// lib/sources/pulp_im2col_fp32.c:157-232; lib/sources/pulp_matmul_fp32.c:190-262] and the naive kernels
// [ref: lib/sources/pulp_conv_naive_fp32.c:198-300, :410-516].
#include "tl_kernels.h"
#include "tl_tc.cuh"

namespace tl {

using namespace tc;

struct ConvMnParams {
    int n, Cout;                    // streams, channels of the output tensor
    int H, W;                       // plane of the computed grid (= the source plane)
    int Hk, Wk, padU, padL;         // window of source positions per output pixel
    int cigs;                       // 8-channel groups of the source
    int NT, NB, stack, DC;          // output channels per CTA, Wk*NT, [hi|lo] stacked in N, accumulator columns
    int NI, NBUF, VR, NSLOT;        // issuers (= m-blocks per tile), accumulators per issuer, image rows per tile (4 per m-block), slots per stage
    int P;                          // streams side by side in one slot (32 / W)
    int stage_bytes, nstage;
    int tiles_per_image, n_tiles;
    const float *w;                 // filters; see the operand builder for the three roles
    int Cout_w, Cin_w, flip, cls, kstep, kh_r, kh_m, kw_r, kw_m, w_Wk, w_taps;
    int oH, oW, osy, osx, oy0, ox0; // output pixel (y, x) of the grid lands at (y*osy + oy0, x*osx + ox0) of an oH x oW plane
    const float *bias;
    float *y;
    int *status;
};

#ifdef MN_DEBUG
__device__ float mn_dbg[4096];
#endif
static constexpr int MN_CONV_WARPS = 4;
static constexpr int MN_MAX_STAGE = 8;
static constexpr int MN_MAX_NI = 4;
static constexpr uint32_t MN_NAP = 64u;
static constexpr int MN_SLOT = 1024;            // bytes of one slot: 8 channels x 128 bytes
static constexpr int MN_RPB = 4;                // slots (image rows) per m-block

// status ids of this kernel's waits: 11 stage free (TMA), 12 accumulator free (issuer), 13 operand ready (issuer),
// 14 raw data landed (converter), 16 accumulator complete (epilogue)
__global__ void __launch_bounds__(32 * (5 * MN_MAX_NI + 1 + MN_CONV_WARPS), 1)
conv_mn_kernel(const __grid_constant__ CUtensorMap tmap, const ConvMnParams p)
{
    extern __shared__ unsigned char smem_dyn[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NI = p.NI;
    const int first_issuer = 4 * NI, tma_warp = 5 * NI, first_conv = 5 * NI + 1;
    const int nthreads = blockDim.x;

    // shared memory carve-up (stages first: swizzle atoms want 1024-byte alignment)
    const uint32_t base_u32 = smem_u32(smem_dyn);
    const uint32_t pad = ((base_u32 + 1023u) & ~1023u) - base_u32;
    unsigned char *stages = smem_dyn + pad;                                        // nstage x [raw/hi | lo]
    const uint32_t half_bytes = (uint32_t)p.stage_bytes;                           // bytes of one array of a stage
    float *Bs = reinterpret_cast<float *>(stages + (size_t)p.nstage * 2 * half_bytes);
    const uint32_t b_step_bytes = 64u * (uint32_t)p.NB;                            // [k4 = 2][2NB rows][4 floats]
    const size_t b_bytes = (size_t)p.cigs * p.Hk * b_step_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<unsigned char *>(Bs) + ((b_bytes + 127) & ~(size_t)127));
    uint64_t *raw_full = bars, *a_full = bars + MN_MAX_STAGE, *stage_empty = bars + 2 * MN_MAX_STAGE;
    uint64_t *d_full = bars + 3 * MN_MAX_STAGE, *d_empty = d_full + 2 * MN_MAX_NI;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(d_empty + 2 * MN_MAX_NI);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    if (threadIdx.x == 0) {
        for (int i = 0; i < p.nstage; i++) { mbar_init(&raw_full[i], 1); mbar_init(&a_full[i], MN_CONV_WARPS); mbar_init(&stage_empty[i], NI); }
        for (int i = 0; i < NI * p.NBUF; i++) { mbar_init(&d_full[i], 1); mbar_init(&d_empty[i], 4); }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap);
    }
    if (warp == tma_warp) { tmem_alloc(tmem_slot, 512u); tmem_relinquish(); }
    // B operand (weights of this CTA's output-channel slice), K-major core matrices of 8 rows x 16 bytes:
    // step (g, a) = channel group g, window row a; inside a step [k4 = 0..1][row r = 0..2NB-1][j = 0..3] with
    // row r = b*NT + c holding hi(w) and row NB + r holding lo(w) of output channel slice*NT + c, window column b,
    // source channel g*8 + k4*4 + j.
    {
        const int per_step = p.NB * 8;
        const int total = p.cigs * p.Hk * per_step;
        for (int e = threadIdx.x; e < total; e += nthreads) {
            const int j = e & 3, k4 = (e >> 2) & 1, r = (e >> 3) % p.NB, step = (e >> 3) / p.NB;
            const int a = step % p.Hk, g = step / p.Hk;
            const int b = r / p.NT, c = r % p.NT;
            const int n_out = blockIdx.y * p.NT + c, k_in = g * 8 + k4 * 4 + j;
            float v = 0.f;
            if (p.cls) {
                const int kh = p.kh_r + p.kstep * (p.kh_m - a), kw = p.kw_r + p.kstep * (p.kw_m - b);
                if (n_out < p.Cin_w && k_in < p.Cout_w) v = __ldg(p.w + ((long long)k_in * p.Cin_w + n_out) * p.w_taps + kh * p.w_Wk + kw);
            } else if (!p.flip) {
                if (n_out < p.Cout_w && k_in < p.Cin_w) v = __ldg(p.w + ((long long)n_out * p.Cin_w + k_in) * p.w_taps + a * p.Wk + b);
            } else {
                if (n_out < p.Cin_w && k_in < p.Cout_w) v = __ldg(p.w + ((long long)k_in * p.Cin_w + n_out) * p.w_taps + (p.w_taps - 1 - (a * p.Wk + b)));
            }
            uint32_t hi, lo;
            split_tf32(v, hi, lo);
            float *dst = Bs + (size_t)step * (b_step_bytes / 4) + (size_t)k4 * (2 * p.NB * 4) + j;
            dst[r * 4] = __uint_as_float(hi);
            dst[(p.NB + r) * 4] = __uint_as_float(lo);
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t stages_u32 = smem_u32(stages);
#ifdef MN_DEBUG
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x < 256) mn_dbg[threadIdx.x] = Bs[threadIdx.x];
    if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) { mn_dbg[4000] = (float)tmem_base; mn_dbg[4001] = (float)stages_u32; mn_dbg[4002] = (float)smem_u32(Bs); mn_dbg[4003] = (float)p.NI; mn_dbg[4004] = (float)p.DC; mn_dbg[4005] = (float)p.nstage; mn_dbg[4006]=(float)p.NB; mn_dbg[4007]=(float)p.stack; }
#endif

    if (warp == tma_warp) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t k = 0;                                     // chunk counter (tile, channel group)
            const uint32_t chunk_tx = (uint32_t)p.NSLOT * (uint32_t)MN_SLOT;
            bool ok = true;
            for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
                const int s0 = (t / p.tiles_per_image) * p.P, y0 = (t % p.tiles_per_image) * p.VR;
                for (int g = 0; g < p.cigs; g++, k++) {
                    const int st = k % p.nstage;
                    if (!wait_or_abort(&stage_empty[st], ((k / p.nstage) & 1) ^ 1, abort_flag, p.status, 11, 256u)) { ok = false; break; }
                    mbar_arrive_expect_tx(&raw_full[st], chunk_tx);
                    tma_load_4d(stages + (size_t)st * 2 * half_bytes, &tmap, &raw_full[st], 0, s0, g * 8, y0 - p.padU);
                }
            }
        }
    } else if (warp >= first_conv) {
        // ------------------------------------------------------------ converters: raw -> hi in place, lo beside it
        // TMA writes the slots unswizzled (row R of a slot = channel R, 128 bytes = the 32 pixels).  The tensor core reads
        // 32-byte pieces XOR-swizzled with R mod 4, so every 16-byte chunk i = R*8 + q of a slot moves to chunk
        // R*8 + (((q >> 1) ^ (R & 3)) << 1 | (q & 1)) of the same row while it is split.  One warp does one slot per pass:
        // lane l loads chunks l and l + 32, the warp synchronises (every source chunk has been read), then both parts are
        // stored - the big part in place of the raw data.
        const int cw = warp - first_conv;
        uint32_t k = 0;
        bool ok = true;
        const int R0 = lane >> 3, q = lane & 7;
        const int dst0 = R0 * 8 + ((((q >> 1) ^ (R0 & 3)) << 1) | (q & 1));        // rows 0..3 (chunk l); rows 4..7 have the same R & 3
        for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
            for (int g = 0; g < p.cigs; g++, k++) {
                const int st = k % p.nstage;
                if (!warp_wait_or_abort(&raw_full[st], (k / p.nstage) & 1, abort_flag, p.status, 14, MN_NAP, lane)) { ok = false; break; }
                float4 *hi4 = reinterpret_cast<float4 *>(stages + (size_t)st * 2 * half_bytes);
                float4 *lo4 = reinterpret_cast<float4 *>(stages + (size_t)st * 2 * half_bytes + half_bytes);
                for (int sl = cw; sl < p.NSLOT; sl += MN_CONV_WARPS) {
                    float4 *h = hi4 + sl * (MN_SLOT / 16), *l = lo4 + sl * (MN_SLOT / 16);
                    const float4 v0 = h[lane], v1 = h[lane + 32];
                    uint32_t a0, a1, a2, a3, b0, b1, b2, b3, c0, c1, c2, c3, d0, d1, d2, d3;
                    split_tf32_fast(v0.x, a0, b0); split_tf32_fast(v0.y, a1, b1); split_tf32_fast(v0.z, a2, b2); split_tf32_fast(v0.w, a3, b3);
                    split_tf32_fast(v1.x, c0, d0); split_tf32_fast(v1.y, c1, d1); split_tf32_fast(v1.z, c2, d2); split_tf32_fast(v1.w, c3, d3);
                    __syncwarp();
                    h[dst0] = make_float4(__uint_as_float(a0), __uint_as_float(a1), __uint_as_float(a2), __uint_as_float(a3));
                    l[dst0] = make_float4(__uint_as_float(b0), __uint_as_float(b1), __uint_as_float(b2), __uint_as_float(b3));
                    h[dst0 + 32] = make_float4(__uint_as_float(c0), __uint_as_float(c1), __uint_as_float(c2), __uint_as_float(c3));
                    l[dst0 + 32] = make_float4(__uint_as_float(d0), __uint_as_float(d1), __uint_as_float(d2), __uint_as_float(d3));
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(&a_full[st]);
            }
        }
    } else if (warp >= first_issuer) {
        // ------------------------------------------------------------ MMA issuers: issuer j owns m-block j of every tile
        if (lane == 0) {
            const int j = warp - first_issuer;
            const uint32_t n_wide = (uint32_t)(p.stack ? 2 * p.NB : p.NB);
            const uint32_t idesc_wide = mma_idesc(FMT_TF32, 128, n_wide) | IDESC_A_MN_MAJOR;
            const uint32_t idesc_nb = mma_idesc(FMT_TF32, 128, (uint32_t)p.NB) | IDESC_A_MN_MAJOR;
            const uint32_t b_u32 = smem_u32(Bs);
            const uint32_t b_lbo = (uint32_t)(2 * p.NB) * 16u, b_sbo = 128u, b_lo_rows = (uint32_t)p.NB * 16u;
            uint32_t k = 0, tseq = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, tseq++) {
                const int dbuf = (tseq % p.NBUF) * NI + j;
                const uint32_t use = tseq / p.NBUF;
                if (!wait_or_abort(&d_empty[dbuf], (use & 1) ^ 1, abort_flag, p.status, 12, MN_NAP)) break;
                tc_fence_after();
                const uint32_t d_addr = tmem_base + (uint32_t)(dbuf * p.DC);
                uint32_t acc = 0;
                for (int g = 0; g < p.cigs; g++, k++) {
                    const int st = k % p.nstage;
                    if (!wait_or_abort(&a_full[st], (k / p.nstage) & 1, abort_flag, p.status, 13, MN_NAP)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t hi_u32 = stages_u32 + (uint32_t)st * 2u * half_bytes, lo_u32 = hi_u32 + half_bytes;
                    for (int a = 0; a < p.Hk; a++) {
                        const uint32_t a_off = (uint32_t)(j * MN_RPB + a) * (uint32_t)MN_SLOT;
                        const uint64_t a_hi = smem_desc_mnmajor(hi_u32 + a_off, MN_SLOT, MN_SLOT / 2, LAYOUT_SW128_ATOM32);
                        const uint64_t a_lo = smem_desc_mnmajor(lo_u32 + a_off, MN_SLOT, MN_SLOT / 2, LAYOUT_SW128_ATOM32);
                        const uint32_t b_addr = b_u32 + (uint32_t)(g * p.Hk + a) * b_step_bytes;
                        const uint64_t b_hi = smem_desc_kmajor(b_addr, b_lbo, b_sbo);
                        if (p.stack) {
                            mma_tf32_ss(d_addr, a_hi, b_hi, idesc_wide, acc);
                            mma_tf32_ss(d_addr, a_lo, b_hi, idesc_nb, 1u);
                        } else {
                            const uint64_t b_lo = smem_desc_kmajor(b_addr + b_lo_rows, b_lbo, b_sbo);
                            mma_tf32_ss(d_addr, a_hi, b_hi, idesc_nb, acc);
                            mma_tf32_ss(d_addr, a_hi, b_lo, idesc_nb, 1u);
                            mma_tf32_ss(d_addr, a_lo, b_hi, idesc_nb, 1u);
                        }
                        acc = 1u;
                    }
                    mma_commit(&stage_empty[st]);
                }
                if (!ok) break;
                mma_commit(&d_full[dbuf]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: tensor memory -> shift-sum -> global
        const int j = warp >> 2, q = warp & 3;
        const int img = lane / p.W, x = lane % p.W;         // lane = pixel of the slot: stream `img` of the pack, column x
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const long long plane = (long long)p.oH * p.oW;
        const int co0 = blockIdx.y * p.NT;
        uint32_t tseq = 0;
        for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, tseq++) {
            const int dbuf = (tseq % p.NBUF) * NI + j;
            const uint32_t use = tseq / p.NBUF;
            const int s = (t / p.tiles_per_image) * p.P + img, y = (t % p.tiles_per_image) * p.VR + j * MN_RPB + q;
            const int oy = y * p.osy + p.oy0, ox = x * p.osx + p.ox0;
            const bool valid = (s < p.n) && (y < p.H) && (oy < p.oH) && (ox < p.oW);
            float *yp = p.y + ((long long)s * p.Cout + co0) * plane + (long long)oy * p.oW + ox;
            if (!warp_wait_or_abort(&d_full[dbuf], use & 1, abort_flag, p.status, 16, MN_NAP, lane)) break;
            tc_fence_after();
            const uint32_t d_addr = tmem_base + (uint32_t)(dbuf * p.DC) + lane_addr;
            for (int c0 = 0; c0 < p.NT; c0 += 8) {
                float acc[8];
#pragma unroll
                for (int i = 0; i < 8; i++) acc[i] = 0.f;
                for (int b = 0; b < p.Wk; b++) {
                    uint32_t h[8], l[8];
                    tmem_ld8(d_addr + (uint32_t)(b * p.NT + c0), h);
                    if (p.stack) tmem_ld8(d_addr + (uint32_t)(p.NB + b * p.NT + c0), l);
                    tmem_wait_ld();
#ifdef MN_DEBUG
                    if (blockIdx.x == 0 && blockIdx.y == 0 && tseq == 0 && warp == 0 && c0 == 0) { for (int i = 0; i < 8; i++) { mn_dbg[1280 + (b * 32 + lane) * 16 + i] = __uint_as_float(h[i]); mn_dbg[1280 + (b * 32 + lane) * 16 + 8 + i] = p.stack ? __uint_as_float(l[i]) : 0.f; } }
#endif
                    const int d = b - p.padL;
                    const int src = (lane + d) & 31;
                    const bool in_row = (unsigned)(x + d) < (unsigned)p.W;
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        float v = __uint_as_float(h[i]);
                        if (p.stack) v += __uint_as_float(l[i]);
                        v = __shfl_sync(0xffffffffu, v, src);
                        if (in_row) acc[i] += v;
                    }
                }
                if (c0 + 8 >= p.NT) {
                    // every value of this accumulator has been read: hand it back before the last stores go out
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&d_empty[dbuf]);
                }
                if (valid) {
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        const int co = co0 + c0 + i;
                        if (co < p.Cout) {
                            float v = acc[i];
                            if (p.bias) v += __ldg(p.bias + co);
                            yp[(long long)(c0 + i) * plane] = v;
                        }
                    }
                }
            }
        }
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == tma_warp) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, 512u); }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
void *tc_encode_tiled_fn();
int *tc_status_word();

// Same contract as conv_tc_run (tl_conv_tc.cu); false = the geometry is not one this kernel covers.
bool conv_mn_run(const float *src, const float *w, const float *bias, float *dst,
                 int n, int C_src, int H_src, int W_src, int C_dst, int H_dst, int W_dst,
                 int Hk, int Wk, int sh, int sw, int padU, int padL, int Cout_w, int Cin_w, bool flip, bool dry_run, const ConvTcClass *cls)
{
    EncodeTiledFn enc = (EncodeTiledFn)tc_encode_tiled_fn();
    if (!enc) return false;
    if (sh != 1 || sw != 1 || W_src != W_dst || H_src != H_dst) return false;
    const int W = W_dst, H = H_dst;
    if (W != 32 && W != 16 && W != 8) return false;
    if ((((uintptr_t)src) & 15) != 0 || n < 1) return false;
    if (Hk < 1 || Wk < 1 || Hk > 7 || Wk > 5 || padU < 0 || padL < 0 || padU > Hk - 1 || padL > Wk - 1) return false;

    ConvMnParams p;
    p.n = n; p.Cout = C_dst; p.H = H; p.W = W; p.Hk = Hk; p.Wk = Wk; p.padU = padU; p.padL = padL;
    p.cigs = ceil_div(C_src, 8);
    p.P = 32 / W;

    // Output-channel slice, issuers and stages: the widest slice whose weights leave room for at least three stages.
    const int cpad = ((C_dst + 15) / 16) * 16;
    bool found = false;
    size_t smem = 0;
    for (int NT = std::min(cpad, 64); NT >= 16 && !found; NT -= 16) {
        if (cpad % NT != 0 && NT != 16) continue;
        const int NB = Wk * NT;
        if (NB > 256) continue;
        const int stack = (2 * NB <= 256) ? 1 : 0;
        const int DC = stack ? 2 * NB : NB;
        int NI = 512 / DC;
        if (NI > MN_MAX_NI) NI = MN_MAX_NI;
        for (; NI >= 1 && !found; NI--) {
            if (NI == 3) continue;
            const int VR = NI * MN_RPB;
            if (H % VR != 0) continue;
            const int NSLOT = VR + Hk - 1;
            const int stage_bytes = NSLOT * MN_SLOT;
            const size_t b_bytes = ((size_t)p.cigs * Hk * 64 * NB + 127) & ~(size_t)127;
            const size_t fixed = 1024 + b_bytes + (3 * MN_MAX_STAGE + 4 * MN_MAX_NI) * 8 + 64;
            int nstage = (int)((220 * 1024 - (long long)fixed) / (2 * (long long)stage_bytes));
            if (nstage > MN_MAX_STAGE) nstage = MN_MAX_STAGE;
            if (nstage < 3 && !(nstage == 2 && NT == 16 && NI == 1)) continue;
            p.NT = NT; p.NB = NB; p.stack = stack; p.DC = DC; p.NI = NI;
            p.NBUF = (2 * NI * DC <= 512) ? 2 : 1;
            p.VR = VR; p.NSLOT = NSLOT; p.stage_bytes = stage_bytes; p.nstage = nstage;
            p.tiles_per_image = H / VR;
            p.n_tiles = ceil_div(n, p.P) * p.tiles_per_image;
            smem = fixed + (size_t)nstage * 2 * stage_bytes;
            found = true;
        }
    }
    if (!found || p.NSLOT > 256) return false;
    if (dry_run) return true;

    CUtensorMap tmap;
    // dimensions in the order (x, stream, channel, row): a box {W, P, 8, rows} lands as [row][channel][stream][x], i.e.
    // rows of 128 bytes holding one image row of P streams, 8 channels per slot
    cuuint64_t gdim[4] = {(cuuint64_t)W, (cuuint64_t)n, (cuuint64_t)C_src, (cuuint64_t)H};
    cuuint64_t gstr[3] = {(cuuint64_t)W * H * C_src * 4, (cuuint64_t)W * H * 4, (cuuint64_t)W * 4};
    cuuint32_t box[4] = {(cuuint32_t)W, (cuuint32_t)p.P, 8u, (cuuint32_t)p.NSLOT};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)src, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;

    int *status = tc_status_word();
    if (!status) return false;
    p.w = w; p.Cout_w = Cout_w; p.Cin_w = Cin_w; p.flip = flip ? 1 : 0;
    p.oH = H; p.oW = W; p.osy = p.osx = 1; p.oy0 = p.ox0 = 0;
    p.cls = 0; p.kstep = 1; p.kh_r = p.kh_m = p.kw_r = p.kw_m = 0; p.w_Wk = Wk; p.w_taps = Hk * Wk;
    if (cls) {
        p.cls = 1; p.kstep = cls->kstep; p.kh_r = cls->kh_r; p.kh_m = cls->kh_m; p.kw_r = cls->kw_r; p.kw_m = cls->kw_m;
        p.w_Wk = cls->w_Wk; p.w_taps = cls->w_Hk * cls->w_Wk;
        p.oH = cls->oH; p.oW = cls->oW; p.osy = cls->osy; p.osx = cls->osx; p.oy0 = cls->oy0; p.ox0 = cls->ox0;
    }
    p.bias = bias; p.y = dst; p.status = status;
    const int co_tiles = ceil_div(C_dst, p.NT);
    int ctas = sm_count() / co_tiles;
    if (ctas < 1) ctas = 1;
    if (ctas > p.n_tiles) ctas = p.n_tiles;
    dim3 grid(ctas, co_tiles);
    const int threads = 32 * (5 * p.NI + 1 + MN_CONV_WARPS);
    static bool attr_set = false;
    if (!attr_set) { cudaFuncSetAttribute(conv_mn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); attr_set = true; }
    TL_LAUNCH(conv_mn_kernel, grid, threads, smem, tmap, p);
    return true;
}

#ifdef MN_DEBUG
extern "C" __attribute__((visibility("default"))) int trainlib_mn_debug_read(float *out) { return (int)cudaMemcpyFromSymbol(out, mn_dbg, sizeof(float) * 4096); }
#endif
} // namespace tl
