// Weight gradient of a 3x3, stride-1, pad-1 convolution on the 5th-generation tensor cores (3xTF32 split-precision fp32):
//
//   dW[co][ci][a][b] = sum over streams s and pixels (y, x) of  dY[s][co][y][x] * X[s][ci][y + a - 1][x + b - 1]
//
// as a GEMM whose contraction index is the PIXEL.  Both operands are K-major straight from CHW memory (a row = one
// channel, consecutive K = consecutive pixels of an image row), which is what TMA delivers:
//
//   D[(a, ci)][(b, co)] += sum_x  X[ci][y + a - 1][x] * dY_b[co][y][x],      dY_b[x] = dY[x - b + 1] (0 outside the row)
//
// M = (a, ci): for output-gradient row y the three input rows y-1, y, y+1 of all channels are CONSECUTIVE 8-row groups
// of the shared-memory array [row][channel group][8 channels][32 pixels], so one descriptor covers them (rows beyond
// the 3*Cin real ones compute garbage in accumulator lanes nobody reads).  N = (b, co): the three filter columns are
// three copies of the dY row shifted by one pixel, written by the converter warps together with the hi/lo split -
// a shift along K cannot be had from a descriptor (16-byte start alignment).  K = 8 pixels per MMA, 4 MMAs per row.
// "32 pixels" = one image row of P = 32 / W streams side by side, so the sum over the pixels of a slot already sums
// over P streams.
//
// Per k-step and M-block:  D (+)= X_hi * [dYb_hi | dYb_lo]^T ;  D[:, hi part] += X_lo * dYb_hi^T   (three N-wide MMAs
// into one set of columns where 6*Cout > 256).  The accumulators stay in tensor memory for the CTA's whole run (all its
// streams); each accumulator has exactly one issuing thread, k-steps are dealt round-robin to KS issuers with their
// own accumulators, and the epilogue adds the sets in a fixed order and writes the CTA's partial result in the
// accumulators' own [row][column] layout (64 contiguous bytes per thread and store: scattering it to dW[co][ci][kh][kw]
// from every CTA cost more than the arithmetic of a small launch); wgt_reduce_kernel sums the partials over the CTAs
// (fixed order: bit-reproducible) and scatters once.
//
// Stride 2 (3x3, pad 1, input rows twice as long as dY rows): X[2y + a - 1][2x + b - 1].  The converters de-interleave
// every input row into its even and odd pixels (two slots E and O per row and channel group, same 32-position K layout
// as dY: P streams of W output pixels), so that b = 1 pairs E[x] with dY[x], b = 2 pairs O[x] with dY[x] and b = 0
// pairs O[x - 1] with dY[x], i.e. O[x] with the copy dY[x + 1].  M = (input row, parity, ci): the three input rows
// 2y - 1, 2y, 2y + 1 of an output row are consecutive in the array [input row][parity][channel group], and moving to
// the next output row moves the descriptor by TWO input rows.  N = two copies of dY (x, x + 1).  One of the four
// (parity, copy) blocks, E with dY[x + 1], is computed and not used.
//
// Replaces the im2col + mm lowering of the weight gradient [ref: lib/sources/pulp_conv2d_fp32.c:294-333] and the
// naive kernel [ref: lib/sources/pulp_conv_naive_fp32.c:302-408].
#include "tl_kernels.h"
#include "tl_tc.cuh"

namespace tl {

using namespace tc;

struct WgtParams {
    int n, Cin, Cout, H, W, P;      // H, W: rows and row length of dY; P = 32 / W streams side by side in a 32-pixel slot
    int cigs, cogs;                 // 8-channel groups of X and dY
    int s2;                         // 1: stride-2 convolution (see the note on strides in the header comment)
    int xg, ncopy;                  // 8-row groups of one X row in the operand array (cigs, or 2 * cigs for stride 2); shifted dY copies (3 or 2)
    int T;                          // dY rows per tile (X rows: T + 2, or 2T + 1 for stride 2)
    int MB, KS, stack;              // M-blocks (16 groups each), k-step split, [hi|lo] stacked in N
    int DC;                         // accumulator columns per (set, M-block)
    int NR, NC;                     // stages of the raw ring (TMA -> converters) and of the operand ring (converters -> MMAs)
    int tiles_per_image, n_tiles;
    uint32_t raw_bytes, xh_bytes, conv_bytes;   // one raw stage [X rows | dY rows]; the X hi (= X lo) array; one operand stage [X hi | X lo | dY copies]
    float *part;                    // [gridDim.x][Cout][Cin][3][3]
    int *status;
};

static constexpr int WGT_CONV_WARPS = 8, WGT_MAX_ISS = 4, WGT_MAX_NR = 8, WGT_MAX_NC = 4;
static constexpr int WGT_THREADS = 32 * (WGT_CONV_WARPS + WGT_MAX_ISS + 1);
static constexpr int WGT_SLOT = 1024;           // 8 channels x 32 pixels x 4 bytes

// Two rings: the kernel streams its operands once from HBM, so what bounds it is the number of bytes in flight per SM.
// The raw ring (small stages, many of them) keeps TMA copies of the coming tiles in flight while the operand ring (large
// stages: every dY row becomes six arrays) holds the tiles being converted and multiplied.
//
// status ids of this kernel's waits: 21 raw stage free (TMA), 22 raw landed, 25 operand stage free (converters),
// 23 operands ready (issuer), 24 all MMAs done (epilogue)
__global__ void __launch_bounds__(WGT_THREADS, 1)
conv_wgt_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_dy, const WgtParams p)
{
    extern __shared__ unsigned char smem_dyn[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NISS = p.MB * p.KS;
    constexpr int first_issuer = WGT_CONV_WARPS, tma_warp = WGT_CONV_WARPS + WGT_MAX_ISS;

    const uint32_t base_u32 = smem_u32(smem_dyn);
    const uint32_t pad = ((base_u32 + 1023u) & ~1023u) - base_u32;
    unsigned char *conv = smem_dyn + pad;                                   // NC x [X hi | X lo | dY copies]
    unsigned char *raws = conv + (size_t)p.NC * p.conv_bytes;               // NR x [X rows | dY rows] (also the slack the last M-block overruns into)
    uint64_t *bars = reinterpret_cast<uint64_t *>(raws + (size_t)p.NR * p.raw_bytes);
    uint64_t *raw_full = bars, *raw_empty = bars + WGT_MAX_NR, *conv_full = bars + 2 * WGT_MAX_NR, *conv_empty = conv_full + WGT_MAX_NC, *all_done = conv_empty + WGT_MAX_NC;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(all_done + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    if (threadIdx.x == 0) {
        for (int i = 0; i < p.NR; i++) { mbar_init(&raw_full[i], 1); mbar_init(&raw_empty[i], WGT_CONV_WARPS); }
        for (int i = 0; i < p.NC; i++) { mbar_init(&conv_full[i], WGT_CONV_WARPS); mbar_init(&conv_empty[i], NISS); }
        mbar_init(all_done, NISS);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tmap_x); tma_prefetch_desc(&tmap_dy);
    }
    if (warp == tma_warp) { tmem_alloc(tmem_slot, 512u); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const int XS = p.s2 ? 2 * p.T + 1 : p.T + 2;    // X rows per stage
    const uint32_t x_row_bytes = (uint32_t)p.xg * WGT_SLOT, dyc_row_bytes = 2u * p.ncopy * p.cogs * WGT_SLOT;
    const int rowstep = p.s2 ? 2 : 1;               // X rows per dY row
    const uint32_t xraw_bytes = (uint32_t)XS * x_row_bytes;

    if (warp == tma_warp) {
        // ------------------------------------------------------------ TMA producer: one copy of X rows, one of dY rows per tile
        if (lane == 0) {
            uint32_t k = 0;
            for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, k++) {
                const int rs = k % p.NR;
                if (!wait_or_abort(&raw_empty[rs], ((k / p.NR) & 1) ^ 1, abort_flag, p.status, 21, 128u)) break;
                const int s0 = (t / p.tiles_per_image) * p.P, y0 = (t % p.tiles_per_image) * p.T;
                unsigned char *rb = raws + (size_t)rs * p.raw_bytes;
                mbar_arrive_expect_tx(&raw_full[rs], p.raw_bytes);
                tma_load_4d(rb, &tmap_x, &raw_full[rs], 0, s0, 0, rowstep * y0 - 1);
                tma_load_4d(rb + xraw_bytes, &tmap_dy, &raw_full[rs], 0, s0, 0, y0);
            }
        }
    } else if (warp < WGT_CONV_WARPS) {
        // ------------------------------------------------------------ converters (and, at the end, the epilogue)
        // A slot = 8 rows (channels) of 128 bytes (32 pixels).  The tensor core reads it K-major with the 128-byte swizzle:
        // 16-byte chunk q of row R lives at chunk q ^ R.  X slots: split into the hi and lo arrays.  dY slots: three copies
        // shifted by -1 / 0 / +1 pixel inside each stream's part of the row (zero beyond it), each split into hi and lo.
        const int R0 = lane >> 3, q = lane & 7;                     // lane l holds chunks l (row R0) and l + 32 (row R0 + 4)
        const int d0 = R0 * 8 + (q ^ R0), d1 = (R0 + 4) * 8 + (q ^ (R0 + 4));
        const int cpw = p.W / 4;                                    // chunks per stream row
        const bool left_edge = (q % cpw) == 0, right_edge = (q % cpw) == cpw - 1;
        uint32_t k = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, k++) {
            const int rs = k % p.NR, cs = k % p.NC;
            if (!warp_wait_or_abort(&raw_full[rs], (k / p.NR) & 1, abort_flag, p.status, 22, 32u, lane)) { ok = false; break; }
            if (!warp_wait_or_abort(&conv_empty[cs], ((k / p.NC) & 1) ^ 1, abort_flag, p.status, 25, 32u, lane)) { ok = false; break; }
            const unsigned char *rb = raws + (size_t)rs * p.raw_bytes;
            unsigned char *cb = conv + (size_t)cs * p.conv_bytes;
            const int nx = XS * p.cigs, ndy = p.T * p.cogs;
            for (int sl = warp; sl < nx + ndy; sl += WGT_CONV_WARPS) {
                if (sl < nx && p.s2) {
                    // a raw row of a channel = P streams x 2W pixels = 64 floats; 8 channels = 2 KB.  Even pixels go to slot E,
                    // odd pixels to slot O of (row, channel group); each in hi and lo.
                    const int row = sl / p.cigs, cig = sl % p.cigs;
                    const float4 *r4 = reinterpret_cast<const float4 *>(rb + (size_t)sl * 2 * WGT_SLOT);
                    unsigned char *eb = cb + (size_t)((row * 2 + 0) * p.cigs + cig) * WGT_SLOT, *ob = cb + (size_t)((row * 2 + 1) * p.cigs + cig) * WGT_SLOT;
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const int R = R0 + 4 * half, dst = half ? d1 : d0;
                        const float4 v0 = r4[R * 16 + 2 * q], v1 = r4[R * 16 + 2 * q + 1];
                        uint32_t eh0, eh1, eh2, eh3, el0, el1, el2, el3, oh0, oh1, oh2, oh3, ol0, ol1, ol2, ol3;
                        split_tf32_fast(v0.x, eh0, el0); split_tf32_fast(v0.z, eh1, el1); split_tf32_fast(v1.x, eh2, el2); split_tf32_fast(v1.z, eh3, el3);
                        split_tf32_fast(v0.y, oh0, ol0); split_tf32_fast(v0.w, oh1, ol1); split_tf32_fast(v1.y, oh2, ol2); split_tf32_fast(v1.w, oh3, ol3);
                        reinterpret_cast<float4 *>(eb)[dst] = make_float4(__uint_as_float(eh0), __uint_as_float(eh1), __uint_as_float(eh2), __uint_as_float(eh3));
                        reinterpret_cast<float4 *>(eb + p.xh_bytes)[dst] = make_float4(__uint_as_float(el0), __uint_as_float(el1), __uint_as_float(el2), __uint_as_float(el3));
                        reinterpret_cast<float4 *>(ob)[dst] = make_float4(__uint_as_float(oh0), __uint_as_float(oh1), __uint_as_float(oh2), __uint_as_float(oh3));
                        reinterpret_cast<float4 *>(ob + p.xh_bytes)[dst] = make_float4(__uint_as_float(ol0), __uint_as_float(ol1), __uint_as_float(ol2), __uint_as_float(ol3));
                    }
                } else if (sl < nx) {
                    const float4 *r4 = reinterpret_cast<const float4 *>(rb + (size_t)sl * WGT_SLOT);
                    float4 *h = reinterpret_cast<float4 *>(cb + (size_t)sl * WGT_SLOT), *l = reinterpret_cast<float4 *>(cb + p.xh_bytes + (size_t)sl * WGT_SLOT);
                    const float4 v0 = r4[lane], v1 = r4[lane + 32];
                    uint32_t a0, a1, a2, a3, b0, b1, b2, b3, c0, c1, c2, c3, e0, e1, e2, e3;
                    split_tf32_fast(v0.x, a0, b0); split_tf32_fast(v0.y, a1, b1); split_tf32_fast(v0.z, a2, b2); split_tf32_fast(v0.w, a3, b3);
                    split_tf32_fast(v1.x, c0, e0); split_tf32_fast(v1.y, c1, e1); split_tf32_fast(v1.z, c2, e2); split_tf32_fast(v1.w, c3, e3);
                    h[d0] = make_float4(__uint_as_float(a0), __uint_as_float(a1), __uint_as_float(a2), __uint_as_float(a3));
                    l[d0] = make_float4(__uint_as_float(b0), __uint_as_float(b1), __uint_as_float(b2), __uint_as_float(b3));
                    h[d1] = make_float4(__uint_as_float(c0), __uint_as_float(c1), __uint_as_float(c2), __uint_as_float(c3));
                    l[d1] = make_float4(__uint_as_float(e0), __uint_as_float(e1), __uint_as_float(e2), __uint_as_float(e3));
                } else {
                    const int ds = sl - nx, row = ds / p.cogs, cog = ds % p.cogs;
                    const float4 *raw = reinterpret_cast<const float4 *>(rb + xraw_bytes + (size_t)ds * WGT_SLOT);
                    unsigned char *crow = cb + 2 * p.xh_bytes + (size_t)row * dyc_row_bytes;
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        const float4 v = raw[lane + 32 * half];
                        // neighbours along the row: the last pixel of the chunk to the left, the first of the chunk to the right
                        float lft = __shfl_up_sync(0xffffffffu, v.w, 1), rgt = __shfl_down_sync(0xffffffffu, v.x, 1);
                        if (left_edge) lft = 0.f;
                        if (right_edge) rgt = 0.f;
                        const float sh[3][4] = {{v.y, v.z, v.w, rgt}, {v.x, v.y, v.z, v.w}, {lft, v.x, v.y, v.z}};   // b = 0: dY[x + 1], b = 1: dY[x], b = 2: dY[x - 1]
                        const int dst = half ? d1 : d0;
#pragma unroll
                        for (int b = 0; b < 3; b++) {
                            if (b >= p.ncopy) break;                 // stride 2 needs dY[x + 1] and dY[x] only
                            uint32_t h0, h1, h2, h3, l0, l1, l2, l3;
                            split_tf32_fast(sh[b][0], h0, l0); split_tf32_fast(sh[b][1], h1, l1); split_tf32_fast(sh[b][2], h2, l2); split_tf32_fast(sh[b][3], h3, l3);
                            float4 *hh = reinterpret_cast<float4 *>(crow + (size_t)((0 * p.ncopy + b) * p.cogs + cog) * WGT_SLOT);
                            float4 *ll = reinterpret_cast<float4 *>(crow + (size_t)((1 * p.ncopy + b) * p.cogs + cog) * WGT_SLOT);
                            hh[dst] = make_float4(__uint_as_float(h0), __uint_as_float(h1), __uint_as_float(h2), __uint_as_float(h3));
                            ll[dst] = make_float4(__uint_as_float(l0), __uint_as_float(l1), __uint_as_float(l2), __uint_as_float(l3));
                        }
                    }
                }
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&conv_full[cs]); mbar_arrive(&raw_empty[rs]); }
        }
        // ------------------------------------------------------------ epilogue (warps 0-3): accumulators -> this CTA's partial dW
        if (warp < 4 && ok) {
            if (warp_wait_or_abort(all_done, 0, abort_flag, p.status, 24, 64u, lane)) {
                tc_fence_after();
                const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
                // The partial leaves in the accumulators' own layout, [M row][column] with 16 consecutive columns (64 bytes) per
                // thread and store; wgt_reduce_kernel maps rows and columns to dW[co][ci][kh][kw] once, after the sum.
                const int NBc = p.ncopy * p.Cout;                      // columns of one product block
                float *out = p.part + (long long)blockIdx.x * ((long long)p.MB * 128 * NBc);
                for (int m = 0; m < p.MB; m++) {
                    float *orow = out + (long long)(m * 128 + warp * 32 + lane) * NBc;
                    const bool valid = m * 16 + (warp * 32 + lane) / 8 < 3 * p.xg;     // rows past the last channel group are never read
                    for (int c0 = 0; c0 < NBc; c0 += 16) {
                        float acc[16];
#pragma unroll
                        for (int i = 0; i < 16; i++) acc[i] = 0.f;
                        for (int qs = 0; qs < p.KS; qs++) {
                            const uint32_t col = tmem_base + lane_addr + (uint32_t)((qs * p.MB + m) * p.DC + c0);
                            uint32_t v[16], w[16];
                            tmem_ld16w(col, v);
                            if (p.stack) tmem_ld16w(col + NBc, w);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 16; i++) acc[i] += __uint_as_float(v[i]) + (p.stack ? __uint_as_float(w[i]) : 0.f);
                        }
#pragma unroll
                        for (int i = 0; i < 16; i += 4) if (valid) *reinterpret_cast<float4 *>(orow + c0 + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
                    }
                }
            }
        }
    } else if (warp >= first_issuer && warp < tma_warp) {
        // ------------------------------------------------------------ MMA issuers: issuer (m, qs) owns M-block m and the k-steps = qs (mod KS)
        const int j = warp - first_issuer;
        if (lane == 0 && j < NISS) {
            const int m = j % p.MB, qs = j / p.MB;
            const uint32_t n_nb = (uint32_t)(p.ncopy * p.Cout), n_wide = p.stack ? 2u * n_nb : n_nb;
            const uint32_t idesc_wide = mma_idesc(FMT_TF32, 128, n_wide), idesc_nb = mma_idesc(FMT_TF32, 128, n_nb);
            const uint64_t tmpl = smem_desc_kmajor_sw128(0u, WGT_SLOT);            // K-major rows of 128 bytes (32 pixels), a k-step advances 32 bytes inside the row
            const uint32_t hiword = (uint32_t)(tmpl >> 32), loword = (uint32_t)tmpl;
            const uint32_t d_addr = tmem_base + (uint32_t)((qs * p.MB + m) * p.DC);
            const uint32_t conv_u32 = smem_u32(conv);
            uint32_t k = 0, kstep = 0, acc = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, k++) {
                const int cs = k % p.NC;
                if (!wait_or_abort(&conv_full[cs], (k / p.NC) & 1, abort_flag, p.status, 23, 0u)) { ok = false; break; }
                const uint32_t sb = conv_u32 + (uint32_t)cs * p.conv_bytes;
                for (int r = 0; r < p.T; r++) {
                    const uint32_t a16 = (sb + (uint32_t)(r * rowstep) * x_row_bytes + (uint32_t)m * 16u * WGT_SLOT) >> 4;   // three consecutive rows of X = input rows y-1, y, y+1 (2y-1, 2y, 2y+1)
                    const uint32_t b16 = (sb + 2 * p.xh_bytes + (uint32_t)r * dyc_row_bytes) >> 4;
                    for (int kk = 0; kk < 4; kk++, kstep++) {
                        if ((int)(kstep % (uint32_t)p.KS) != qs) continue;
                        const uint64_t a_hi = ((uint64_t)hiword << 32) | (loword + a16 + 2u * kk), a_lo = ((uint64_t)hiword << 32) | (loword + a16 + (p.xh_bytes >> 4) + 2u * kk);
                        const uint64_t b_hi = ((uint64_t)hiword << 32) | (loword + b16 + 2u * kk);
                        if (p.stack) {
                            mma_tf32_ss(d_addr, a_hi, b_hi, idesc_wide, acc);
                            mma_tf32_ss(d_addr, a_lo, b_hi, idesc_nb, 1u);
                        } else {
                            const uint64_t b_lo = ((uint64_t)hiword << 32) | (loword + b16 + (((uint32_t)p.ncopy * p.cogs * WGT_SLOT) >> 4) + 2u * kk);
                            mma_tf32_ss(d_addr, a_hi, b_hi, idesc_nb, acc);
                            mma_tf32_ss(d_addr, a_hi, b_lo, idesc_nb, 1u);
                            mma_tf32_ss(d_addr, a_lo, b_hi, idesc_nb, 1u);
                        }
                        acc = 1u;
                    }
                }
                mma_commit(&conv_empty[cs]);
            }
            if (ok) mma_commit(all_done);
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

// dW[co][ci][kh][kw] = sum over the CTAs' partials, which lie in the accumulators' layout: row = 8 channels x (filter row,
// pixel parity, channel group), column = (copy of the dY row, co).  512 consecutive elements per CTA (partial_sums_quad).
__global__ void __launch_bounds__(1024) wgt_reduce_kernel(const float *__restrict__ part, float *__restrict__ dw, int groups, int Cin, int Cout,
                                                          int s2, int xg, int cigs, int ncopy, int MB)
{
    __shared__ float4 sm[8][128];
    const int NBc = ncopy * Cout;
    const long long nn = (long long)MB * 128 * NBc, i = (long long)blockIdx.x * PSUM_ELEMS + (threadIdx.x & 127) * 4;
    const bool used = i < nn && (int)(i / NBc) / 8 < 3 * xg;            // a quad lies inside one row (NBc is a multiple of 16)
    float4 t;
    if (!partial_sums_quad(part, nn, groups, i, used, t, sm)) return;
    const float v[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
        const long long o = wgt_partial_index(i + e, Cin, Cout, s2, xg, cigs, ncopy);
        if (o >= 0) dw[o] = v[e];
    }
}
// the second half of conv_wgt_run: sums `groups` partials into dW
void conv_wgt_reduce(const float *part, float *dw, int groups, int Cin, int Cout, int stride, bool deferred)
{
    const int cigs = Cin / 8, s2 = stride == 2 ? 1 : 0, xg = s2 ? 2 * cigs : cigs, ncopy = s2 ? 2 : 3, MB = ceil_div(3 * xg, 16);
    const long long nn = (long long)MB * 128 * ncopy * Cout;
    if (deferred) { defer_wgt(part, dw, groups, nn, Cin, Cout, s2, xg, cigs, ncopy); return; }
    TL_LAUNCH(wgt_reduce_kernel, ceil_div(nn, PSUM_ELEMS), 1024, 0, part, dw, groups, Cin, Cout, s2, xg, cigs, ncopy, MB);
}

// Weight gradient on the tensor cores for 3x3 / pad 1 with stride 1 or 2 and channel counts that are multiples of 8
// (C_out a multiple of 16).  H x W is the size of the dY planes (rows of 32, 16 or 8 pixels; stride 2: 16 or 8), the X
// planes are stride times as large.  Writes `*groups_out` partial results of `*group_floats_out` floats each (the
// accumulators' layout) into `part` (capacity part_groups); conv_wgt_reduce sums them into dW.  false = geometry not
// covered (nothing launched).
bool conv_wgt_run(const float *x, const float *dy, float *part, int part_groups, int *groups_out, long long *group_floats_out, int n, int Cin, int Cout, int H,
                  int W, int stride, bool dry_run)
{
    EncodeTiledFn enc = (EncodeTiledFn)tc_encode_tiled_fn();
    if (!enc) return false;
    if (stride != 1 && stride != 2) return false;
    if (W != 32 && W != 16 && W != 8) return false;
    if (stride == 2 && W == 32) return false;                  // an input row of 64 pixels does not fit the 64-float raw row of the converter
    if (Cin % 8 != 0 || Cout % 16 != 0 || Cin > 64 || Cout > 64 || Cin < 8 || n < 1) return false;
    if ((((uintptr_t)x | (uintptr_t)dy) & 15) != 0) return false;
    WgtParams p;
    p.n = n; p.Cin = Cin; p.Cout = Cout; p.H = H; p.W = W; p.P = 32 / W;
    p.cigs = Cin / 8; p.cogs = Cout / 8;
    p.s2 = stride == 2 ? 1 : 0;
    p.xg = p.s2 ? 2 * p.cigs : p.cigs; p.ncopy = p.s2 ? 2 : 3;
    p.MB = ceil_div(3 * p.xg, 16);
    if (p.MB > WGT_MAX_ISS) return false;
    p.stack = (2 * p.ncopy * Cout <= 256) ? 1 : 0;
    p.DC = p.stack ? 2 * p.ncopy * Cout : p.ncopy * Cout;
    p.KS = 512 / (p.MB * p.DC);
    if (p.KS > WGT_MAX_ISS / p.MB) p.KS = WGT_MAX_ISS / p.MB;
    if (p.KS < 1) return false;
    // Rows per tile and ring depths within 224 KB: operand stages first (up to 3, leaving room for at least 2 raw
    // stages), the rest goes to raw stages.  Two rows per tile when that still leaves two operand stages, else one.
    bool found = false;
    size_t smem = 0;
    for (int T = 2; T >= 1 && !found; T--) {
        if (H % T != 0) continue;
        const uint32_t XS = p.s2 ? 2u * T + 1u : (uint32_t)T + 2u;
        const uint32_t raw = (XS * p.xg + (uint32_t)T * p.cogs) * WGT_SLOT;
        const uint32_t xh = XS * p.xg * WGT_SLOT, cv = 2 * xh + 2u * p.ncopy * T * p.cogs * WGT_SLOT;
        // two operand stages (converting and multiplying overlap) matter more than a deep raw ring: two raw stages
        // suffice (measured: 32 -> 32 with T = 2, two operand and two raw stages 0.19 ms against 0.25 ms with T = 1, three
        // and three); more rows per tile (T = 4, 8) gained nothing further
        const long long budget = 224 * 1024, min_raw = 2;
        int NC = 0;
        for (int c = 3; c >= 1; c--) if ((long long)c * cv + min_raw * raw <= budget) { NC = c; break; }
        if (NC == 0 || (NC < 2 && T > 1)) continue;
        int NR = (int)((budget - (long long)NC * cv) / raw);
        if (NR > WGT_MAX_NR) NR = WGT_MAX_NR;
        if (NR * (long long)raw < 16 * 1024) continue;          // the raw ring doubles as the slack behind the last operand stage
        p.T = T; p.NC = NC; p.NR = NR; p.raw_bytes = raw; p.xh_bytes = xh; p.conv_bytes = cv;
        smem = 1024 + (size_t)NC * cv + (size_t)NR * raw + 512;
        found = true;
    }
    if (!found) return false;
    p.tiles_per_image = H / p.T;
    p.n_tiles = ceil_div(n, p.P) * p.tiles_per_image;
    int ctas = sm_count();
    if (ctas > p.n_tiles) ctas = p.n_tiles;
    if (ctas > part_groups) return false;
    *group_floats_out = (long long)p.MB * 128 * p.ncopy * Cout;
    if (dry_run) { *groups_out = ctas; return true; }

    CUtensorMap tx, tdy;
    const int Wx = W * stride, Hx = H * stride;
    cuuint64_t gstr_x[3] = {(cuuint64_t)Wx * Hx * Cin * 4, (cuuint64_t)Wx * Hx * 4, (cuuint64_t)Wx * 4};
    cuuint64_t gdim_x[4] = {(cuuint64_t)Wx, (cuuint64_t)n, (cuuint64_t)Cin, (cuuint64_t)Hx};
    cuuint32_t box_x[4] = {(cuuint32_t)Wx, (cuuint32_t)p.P, (cuuint32_t)Cin, (cuuint32_t)(p.s2 ? 2 * p.T + 1 : p.T + 2)};
    cuuint64_t gstr_y[3] = {(cuuint64_t)W * H * Cout * 4, (cuuint64_t)W * H * 4, (cuuint64_t)W * 4};
    cuuint64_t gdim_y[4] = {(cuuint64_t)W, (cuuint64_t)n, (cuuint64_t)Cout, (cuuint64_t)H};
    cuuint32_t box_y[4] = {(cuuint32_t)W, (cuuint32_t)p.P, (cuuint32_t)Cout, (cuuint32_t)p.T};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)x, gdim_x, gstr_x, box_x, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    if (enc(&tdy, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)dy, gdim_y, gstr_y, box_y, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;
    p.part = part;
    p.status = tc_status_word();
    if (!p.status) return false;
    static bool attr_set = false;
    if (!attr_set) { cudaFuncSetAttribute(conv_wgt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); attr_set = true; }
    TL_LAUNCH(conv_wgt_kernel, ctas, WGT_THREADS, smem, tx, tdy, p);
    profile_add_flops(2.0 * n * Cout * Cin * 9.0 * H * W);          // H x W = the dY plane for either stride
    *groups_out = ctas;
    return true;
}

} // namespace tl
