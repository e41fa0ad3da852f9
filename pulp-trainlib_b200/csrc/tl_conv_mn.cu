// Width-preserving stride-1 convolution (forward, stride-1 input gradient, parity classes of a strided input
// gradient) as an implicit GEMM on the 5th-generation tensor cores, 3xTF32 split-precision fp32, with the input
// split into its TF32 parts ONCE per element.
//
//   D[pixel][(b, co)] = sum_{a, ci} X[ci][row(pixel) + a - padU][col(pixel)] * Wt[co][ci][a][b]
//   Y[co][pixel]      = sum_b D[pixel + (b - padL)][(b, co)]                     (b - padL stays inside the image row)
//
// i.e. the filter columns b are moved from the contraction index into the GEMM's N dimension, so the A operand
// never needs a copy of the input shifted by one float: for every filter row `a` and group of eight input channels
// it is the very block of image rows that TMA dropped into shared memory (after one in-place conversion pass), read
// through a descriptor whose start address moves by whole row slots.  The column shift is paid in the epilogue,
// where thread = pixel and a warp = whole image rows: one warp shuffle per shifted filter column.
//
// Shared-memory "row slots": one slot = 8 channels x 32 pixels = 1 KB.  The 32 pixels are one image row of
// P = 32 / W streams side by side (W = 32 / 16 / 8 -> P = 1 / 2 / 4), which is what one row of a TMA box {W, P streams,
// 8 channels, rows} of the tensor map (x, stream, channel, row) produces.  TMA writes a slot as [channel][pixel],
// unswizzled (a swizzling TMA copy pads rows shorter than 128 bytes, so narrow planes could not be packed); the
// converter warps transpose it to the K-major layout [pixel][8 channels] (32-byte rows, 32-byte swizzle) while they
// split.  A block of 128 output pixels (one MMA, "m-block") is 4 consecutive slots = 4 image rows of P streams; filter
// row `a` reads the slots `a` further down.
//
// Pipeline per CTA (persistent, one per SM): a TMA thread fills a ring of stages (one stage = all slots of one
// 8-channel group of one tile); three converter warps replace every raw value by its TF32 "big" part in place and
// write the "small" part to the stage's second array; NI issuing threads, each owning one m-block of the tile and its
// private accumulator in tensor memory, issue per (channel group, filter row)
//     D (+)= A_hi * B_hi^T;   D += A_hi * B_lo^T;   D += A_lo * B_hi^T          (the 3xTF32 products, fp32 accumulation)
// and hand the stage back with tcgen05.commit; epilogue warps read D with tcgen05.ld, shift-sum the filter columns
// and store the output.  Every accumulator has one issuing thread that adds in a fixed order, so results are
// bit-reproducible from run to run.
//
// A strided (3x3, pad 1, stride 2) input gradient runs as two launches, one per output-row parity, in the UP form of
// the kernel: the grid is the dY plane, accumulator column b holds filter column kw = b, and every grid pixel writes
// two neighbouring output pixels (see the template comment).  Other strides and filters go out as one launch per
// parity class, each a small dense stride-1 convolution written to every s-th pixel.
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
    int Hk, padU, padL;             // window rows, padding (the window width is the template parameter)
    int cigs;                       // 8-channel groups of the source
    int NT, NB;                     // output channels per CTA, accumulator columns = WK*NT
    int NI, NE, NBUF, VR, NSLOT;    // issuers (= m-blocks per tile), epilogue groups, accumulators per issuer, image rows per tile, slots per stage
    int P;                          // streams side by side in one slot (32 / W)
    int stage_bytes, nstage;
    int tiles_per_image, n_tiles;
    const float *w;                 // filters; see the operand builder for the three roles
    int Cout_w, Cin_w, flip, cls, up, kstep, kh_r, kh_m, kw_r, kw_m, w_Wk, w_taps;
    int oH, oW, osy, osx, oy0, ox0; // output pixel (y, x) of the grid lands at (y*osy + oy0, x*osx + ox0) of an oH x oW plane
    const float *bias;
    float *y;
    int *status;
};

static constexpr int MN_CONV_WARPS = 3;
static constexpr int MN_MAX_STAGE = 8;
static constexpr int MN_MAX_NI = 4;
static constexpr int MN_SLOT = 1024;            // bytes of one slot: 8 channels x 128 bytes
static constexpr int MN_RPB = 4;                // slots (image rows) per m-block
static constexpr int MN_MAX_NE = 2;             // epilogue groups of 4 warps (more bought nothing: the kernel is bound by shared-memory bandwidth)
static constexpr int MN_MAX_THREADS = 32 * (4 * MN_MAX_NE + MN_MAX_NI + 1 + MN_CONV_WARPS);   // 16 warps, 4 per scheduler: 128 registers each

// Every tcgen05 instruction (mma, commit, ld, fence) costs the thread that issues it about 130 cycles whatever its size
// (measured on B200), so the kernel counts instructions, not bytes: NI threads issue side by side, the epilogue reads an
// accumulator with the widest loads that fit the register file and the tensor-core fences sit only where tensor memory
// changes hands.
//
// status ids of this kernel's waits: 11 stage free (TMA), 12 accumulator free (issuer), 13 operand ready (issuer),
// 14 raw data landed (converter), 16 accumulator complete (epilogue)
// UP (stride-2 input gradient, 3x3, pad 1, one row parity per launch): the grid is the dY plane, accumulator column b
// holds filter column kw = b, and grid pixel j produces the TWO output pixels 2j (= T1[j]) and 2j + 1 (= T2[j] + T0[j + 1]),
// written as one 8-byte store: whole output rows are written contiguously instead of every second pixel per launch.
template <int WK, int PADL, bool UP = false>
__global__ void __launch_bounds__(MN_MAX_THREADS, 1)
conv_mn_kernel(const __grid_constant__ CUtensorMap tmap, const ConvMnParams p)
{
    extern __shared__ unsigned char smem_dyn[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NI = p.NI;
    const int first_issuer = 4 * p.NE, tma_warp = first_issuer + NI, first_conv = tma_warp + 1;
    const int nthreads = blockDim.x;
    constexpr uint32_t nap_conv = 32u, nap_epi = 20u, nap_iss = 0u;      // ns between failed polls (no measurable effect on the run time between 0 and 255)

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
    // step (g, a) = channel group g, window row a; inside a step [k4 = 0..1][row r = 0..2NB-1][j = 0..3].
    // Row r = chunk*(WK*16) + b*16 + c holds hi(w) and row NB + r lo(w) of output channel slice*NT + chunk*16 + c,
    // window column b, source channel g*8 + k4*4 + j: the WK columns of 16 output channels sit side by side,
    // so the epilogue fetches them with one wide load.
    {
        // one item = one row of one step: its 8 source channels are fetched, split and stored as two 16-byte chunks (hi) + two (lo).
        // Items are dealt so that the lanes of a warp read neighbouring addresses: the filter tap runs fastest (9 contiguous
        // floats of the stored filters in every role), then the index that is contiguous next: the channel group of a
        // forward filter (a whole row W[co][:][:][:] is contiguous), the output row otherwise (W[k][ci][:][:] for
        // neighbouring ci).  (Dealt by operand row, every one of the 8 loads of a lane fetched a sector of its own; the launch
        // times did not change with the dealing, the filters come from L1 / L2 either way.)
        const int taps = p.Hk * WK, items = taps * p.cigs * p.NT;
        const bool by_group = !p.cls && !p.flip;
        for (int it = threadIdx.x; it < items; it += nthreads) {
            const int tap = it % taps, rest = it / taps;
            const int a = tap / WK, b = tap % WK;
            const int g = by_group ? rest % p.cigs : rest / p.NT, c = by_group ? rest / p.cigs : rest % p.NT;
            const int chunk = c >> 4, r = chunk * (WK * 16) + b * 16 + (c & 15), step = g * p.Hk + a;
            const int n_out = blockIdx.y * p.NT + c;
            const float *src; long long kstride; int k_lim; bool row_ok;
            if (p.cls) {
                const int kh = p.kh_r + p.kstep * (p.kh_m - a), kw = UP ? b : p.kw_r + p.kstep * (p.kw_m - b);
                src = p.w + (long long)n_out * p.w_taps + kh * p.w_Wk + kw; kstride = (long long)p.Cin_w * p.w_taps; k_lim = p.Cout_w; row_ok = n_out < p.Cin_w;
            } else if (!p.flip) {
                src = p.w + (long long)n_out * p.Cin_w * p.w_taps + a * WK + b; kstride = p.w_taps; k_lim = p.Cin_w; row_ok = n_out < p.Cout_w;
            } else {
                src = p.w + (long long)n_out * p.w_taps + (p.w_taps - 1 - (a * WK + b)); kstride = (long long)p.Cin_w * p.w_taps; k_lim = p.Cout_w; row_ok = n_out < p.Cin_w;
            }
            uint32_t hi[8], lo[8];
#pragma unroll
            for (int k = 0; k < 8; k++) {
                const int k_in = g * 8 + k;
                const float v = (row_ok && k_in < k_lim) ? __ldg(src + (long long)k_in * kstride) : 0.f;
                split_tf32(v, hi[k], lo[k]);
            }
            float *dst = Bs + (size_t)step * (b_step_bytes / 4);
#pragma unroll
            for (int k4 = 0; k4 < 2; k4++) {
                float *d = dst + (size_t)k4 * (2 * p.NB * 4);
                *reinterpret_cast<float4 *>(d + r * 4) = make_float4(__uint_as_float(hi[4 * k4]), __uint_as_float(hi[4 * k4 + 1]), __uint_as_float(hi[4 * k4 + 2]), __uint_as_float(hi[4 * k4 + 3]));
                *reinterpret_cast<float4 *>(d + (p.NB + r) * 4) = make_float4(__uint_as_float(lo[4 * k4]), __uint_as_float(lo[4 * k4 + 1]), __uint_as_float(lo[4 * k4 + 2]), __uint_as_float(lo[4 * k4 + 3]));
            }
        }
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t stages_u32 = smem_u32(stages);
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
                    if (!wait_or_abort(&stage_empty[st], ((k / p.nstage) & 1) ^ 1, abort_flag, p.status, 11, 128u)) { ok = false; break; }
                    mbar_arrive_expect_tx(&raw_full[st], chunk_tx);
                    tma_load_4d(stages + (size_t)st * 2 * half_bytes, &tmap, &raw_full[st], 0, s0, g * 8, y0 - p.padU);
                }
            }
        }
    } else if (warp >= first_conv) {
        // ------------------------------------------------------------ converters: raw -> hi in place, lo beside it
        // TMA writes a slot as [channel 0..7][32 pixels].  The A operand is K-major (an MN-major tf32 operand, which would
        // need no transpose, accepts a single swizzle mode and was measured no faster: ~130 cycles of issue time per MMA
        // either way), so each slot is transposed while it is split: pixel p gets one 32-byte row holding its 8 channels, rows 32 bytes apart, the two 16-byte halves of a
        // row swapped when bit 2 of p is set (the 32-byte swizzle of the K-major layout).  One warp does one slot per
        // pass: lane = pixel reads its 8 channel values (conflict-free: lanes are consecutive floats), the warp
        // synchronises (the whole slot has been read), then hi goes back in place and lo to the second array.
        const int cw = warp - first_conv;
        uint32_t k = 0;
        bool ok = true;
        const int sw = (lane >> 2) & 1;
        for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
            for (int g = 0; g < p.cigs; g++, k++) {
                const int st = k % p.nstage;
                if (!warp_wait_or_abort(&raw_full[st], (k / p.nstage) & 1, abort_flag, p.status, 14, nap_conv, lane)) { ok = false; break; }
                float *hi_f = reinterpret_cast<float *>(stages + (size_t)st * 2 * half_bytes);
                float *lo_f = reinterpret_cast<float *>(stages + (size_t)st * 2 * half_bytes + half_bytes);
                for (int sl = cw; sl < p.NSLOT; sl += MN_CONV_WARPS) {
                    float *h = hi_f + sl * (MN_SLOT / 4), *l = lo_f + sl * (MN_SLOT / 4);
                    uint32_t hi[8], lo[8];
#pragma unroll
                    for (int c = 0; c < 8; c++) split_tf32_fast(h[c * 32 + lane], hi[c], lo[c]);
                    __syncwarp();
                    float4 *h4 = reinterpret_cast<float4 *>(h) + lane * 2, *l4 = reinterpret_cast<float4 *>(l) + lane * 2;
                    h4[sw] = make_float4(__uint_as_float(hi[0]), __uint_as_float(hi[1]), __uint_as_float(hi[2]), __uint_as_float(hi[3]));
                    h4[sw ^ 1] = make_float4(__uint_as_float(hi[4]), __uint_as_float(hi[5]), __uint_as_float(hi[6]), __uint_as_float(hi[7]));
                    l4[sw] = make_float4(__uint_as_float(lo[0]), __uint_as_float(lo[1]), __uint_as_float(lo[2]), __uint_as_float(lo[3]));
                    l4[sw ^ 1] = make_float4(__uint_as_float(lo[4]), __uint_as_float(lo[5]), __uint_as_float(lo[6]), __uint_as_float(lo[7]));
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
            const uint32_t idesc_nb = mma_idesc(FMT_TF32, 128, (uint32_t)p.NB);
            // Descriptors as (low word, high word): only the start-address field (low word, units of 16 bytes) moves between
            // MMAs, so the loop keeps running low words and adds constants (the issue loop is latency-bound on one thread).
            const uint64_t a_tmpl = smem_desc_swizzled(0u, 16u, 256u, LAYOUT_SW32);       // K-major, 32-byte swizzle: rows (pixels) 32 bytes apart, groups of 8 rows 256 bytes apart
            const uint64_t b_tmpl = smem_desc_kmajor(0u, (uint32_t)(2 * p.NB) * 16u, 128u);
            const uint32_t a_hiword = (uint32_t)(a_tmpl >> 32), a_loword = (uint32_t)a_tmpl;
            const uint32_t b_hiword = (uint32_t)(b_tmpl >> 32), b_loword = (uint32_t)b_tmpl;
            const uint32_t b_step16 = b_step_bytes >> 4, b_lo16 = ((uint32_t)p.NB * 16u) >> 4, half16 = half_bytes >> 4;
            const uint32_t b_base16 = smem_u32(Bs) >> 4, a_base16 = (stages_u32 + (uint32_t)(j * MN_RPB) * (uint32_t)MN_SLOT) >> 4;
            uint32_t k = 0, tseq = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, tseq++) {
                const int dbuf = (tseq % p.NBUF) * NI + j;
                const uint32_t use = tseq / p.NBUF;
                if (!wait_or_abort(&d_empty[dbuf], (use & 1) ^ 1, abort_flag, p.status, 12, nap_iss)) break;
                tc_fence_after();                               // the epilogue's tensor-memory loads of this accumulator come first
                const uint32_t d_addr = tmem_base + (uint32_t)(dbuf * p.NB);
                uint32_t acc = 0;
                uint32_t bw = b_loword + b_base16;              // low word of B_hi's descriptor for step (g, a), advanced as the loop goes
                for (int g = 0; g < p.cigs; g++, k++) {
                    const int st = k % p.nstage;
                    // (shared-memory operands: the converters' fence.proxy.async and the barrier order them, no tensor-core fence)
                    if (!wait_or_abort(&a_full[st], (k / p.nstage) & 1, abort_flag, p.status, 13, nap_iss)) { ok = false; break; }
                    uint32_t aw = a_loword + a_base16 + (uint32_t)st * 2u * half16;
                    for (int a = 0; a < p.Hk; a++, aw += MN_SLOT / 16, bw += b_step16) {
                        const uint64_t a_hi = ((uint64_t)a_hiword << 32) | aw, a_lo = ((uint64_t)a_hiword << 32) | (aw + half16);
                        const uint64_t b_hi = ((uint64_t)b_hiword << 32) | bw, b_lo = ((uint64_t)b_hiword << 32) | (bw + b_lo16);
                        mma_tf32_ss(d_addr, a_hi, b_hi, idesc_nb, acc);
                        mma_tf32_ss(d_addr, a_hi, b_lo, idesc_nb, 1u);
                        mma_tf32_ss(d_addr, a_lo, b_hi, idesc_nb, 1u);
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
        // Group e (4 warps = the 4 TMEM lane quarters = the 4 image rows of an m-block) serves the m-blocks e, e + NE, ...
        const int e = warp >> 2, q = warp & 3;
        const int img = lane / p.W, x = lane % p.W;         // lane = pixel of the slot: stream `img` of the pack, column x
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const long long plane = (long long)p.oH * p.oW;
        const int co0 = blockIdx.y * p.NT;
        const int ox = x * p.osx + p.ox0;
        int src[WK]; bool in_row[WK];
#pragma unroll
        for (int b = 0; b < WK; b++) { const int d = b - PADL; src[b] = (lane + d) & 31; in_row[b] = (unsigned)(x + d) < (unsigned)p.W; }
        uint32_t tseq = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x, tseq++) {
            const uint32_t use = tseq / p.NBUF;
            const int s = (t / p.tiles_per_image) * p.P + img;
            for (int j = e; j < NI; j += p.NE) {
                const int dbuf = (tseq % p.NBUF) * NI + j;
                const int y = (t % p.tiles_per_image) * p.VR + j * MN_RPB + q;
                const int oy = y * p.osy + p.oy0;
                const bool valid = (s < p.n) && (y < p.H) && (oy < p.oH) && (ox < p.oW);
                float *yp = p.y + ((long long)s * p.Cout + co0) * plane + (long long)oy * p.oW + ox;
                if (!warp_wait_or_abort(&d_full[dbuf], use & 1, abort_flag, p.status, 16, nap_epi, lane)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_addr = tmem_base + (uint32_t)(dbuf * p.NB) + lane_addr;
                for (int c0 = 0; c0 < p.NT; c0 += 16) {
                    uint32_t h[WK * 16];
                    const uint32_t col = d_addr + (uint32_t)((c0 >> 4) * (WK * 16));
                    if constexpr (WK == 1) { tmem_ld16w(col, h); }
                    else if constexpr (WK == 2) { tmem_ld32w(col, h); }
                    else { tmem_ld32w(col, h); tmem_ld16w(col + 32, h + 32); }
                    tmem_wait_ld();
                    if (c0 + 16 >= p.NT) {
                        // every value of this accumulator is in registers: hand it back before the arithmetic and the stores
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&d_empty[dbuf]);
                    }
                    if constexpr (UP) {
                        // even output pixel: the centre column; odd one: column 2 of this pixel + column 0 of the next pixel of the row
                        const bool next_in_row = x + 1 < p.W;
                        const int nco = min(16, p.Cout - co0 - c0);
                        float *yc = yp + (long long)c0 * plane;
#pragma unroll
                        for (int i = 0; i < 16; i++) {
                            const float v = __shfl_sync(0xffffffffu, __uint_as_float(h[i]), (lane + 1) & 31);
                            const float ev = __uint_as_float(h[16 + i]), od = __uint_as_float(h[32 + i]) + (next_in_row ? v : 0.f);
                            if (valid && i < nco) *reinterpret_cast<float2 *>(yc + (long long)i * plane) = make_float2(ev, od);
                        }
                    } else {
                    // out = centre column (no shift) + the other columns fetched from the neighbouring lanes; one shuffle per
                    // shifted column and channel (the SM does one warp shuffle per clock, they are the epilogue's main cost)
                    float acc[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) acc[i] = 0.f;
#pragma unroll
                    for (int b = 0; b < WK; b++) {
                        if (b == PADL) {
#pragma unroll
                            for (int i = 0; i < 16; i++) acc[i] += __uint_as_float(h[b * 16 + i]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; i++) {
                                const float v = __shfl_sync(0xffffffffu, __uint_as_float(h[b * 16 + i]), src[b]);
                                if (in_row[b]) acc[i] += v;
                            }
                        }
                    }
                    const int nco = min(16, p.Cout - co0 - c0);
                    if (valid && nco > 0) {
                        float *yc = yp + (long long)c0 * plane;
                        if (p.bias) {
                            for (int i = 0; i < 16; i++) if (i < nco) acc[i] += __ldg(p.bias + co0 + c0 + i);
                        }
                        if (nco == 16) {
#pragma unroll
                            for (int i = 0; i < 16; i++) yc[(long long)i * plane] = acc[i];
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; i++) if (i < nco) yc[(long long)i * plane] = acc[i];
                        }
                    }
                    }   // !UP
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
    if (Hk < 1 || Wk < 1 || Hk > 7 || Wk > 3 || padU < 0 || padL < 0 || padU > Hk - 1 || padL > Wk - 1) return false;
    if (Wk == 3 && padL != 1) return false;
    if (cls && cls->up && (Wk != 3 || cls->osx != 2 || cls->ox0 != 0 || cls->oW != 2 * W)) return false;

    ConvMnParams p;
    p.n = n; p.Cout = C_dst; p.H = H; p.W = W; p.Hk = Hk; p.padU = padU; p.padL = padL;
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
        int NI = 512 / NB;
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
            p.NT = NT; p.NB = NB; p.NI = NI;
            p.NE = NI < MN_MAX_NE ? NI : MN_MAX_NE;
            p.NBUF = (2 * NI * NB <= 512) ? 2 : 1;
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
    p.cls = 0; p.up = 0; p.kstep = 1; p.kh_r = p.kh_m = p.kw_r = p.kw_m = 0; p.w_Wk = Wk; p.w_taps = Hk * Wk;
    if (cls) {
        p.cls = 1; p.kstep = cls->kstep; p.kh_r = cls->kh_r; p.kh_m = cls->kh_m; p.kw_r = cls->kw_r; p.kw_m = cls->kw_m;
        p.w_Wk = cls->w_Wk; p.w_taps = cls->w_Hk * cls->w_Wk; p.up = cls->up;
        p.oH = cls->oH; p.oW = cls->oW; p.osy = cls->osy; p.osx = cls->osx; p.oy0 = cls->oy0; p.ox0 = cls->ox0;
    }
    p.bias = bias; p.y = dst; p.status = status;
    const int co_tiles = ceil_div(C_dst, p.NT);
    int ctas = sm_count() / co_tiles;
    if (ctas < 1) ctas = 1;
    if (ctas > p.n_tiles) ctas = p.n_tiles;
    dim3 grid(ctas, co_tiles);
    const int threads = 32 * (4 * p.NE + p.NI + 1 + MN_CONV_WARPS);
#define TL_MN_LAUNCH(WKV, PL, ...)                                                                                     \
    do {                                                                                                               \
        static bool attr_set = false;                                                                                  \
        if (!attr_set) { cudaFuncSetAttribute(conv_mn_kernel<WKV, PL, ##__VA_ARGS__>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); attr_set = true; } \
        TL_LAUNCH((conv_mn_kernel<WKV, PL, ##__VA_ARGS__>), grid, threads, smem, tmap, p);                             \
    } while (0)
    if (p.up) TL_MN_LAUNCH(3, 1, true);
    else if (Wk == 1) TL_MN_LAUNCH(1, 0); else if (Wk == 2 && padL == 0) TL_MN_LAUNCH(2, 0); else if (Wk == 2) TL_MN_LAUNCH(2, 1); else TL_MN_LAUNCH(3, 1);
#undef TL_MN_LAUNCH
    profile_add_flops(2.0 * n * C_dst * C_src * Hk * Wk * H_dst * W_dst);
    return true;
}

} // namespace tl
