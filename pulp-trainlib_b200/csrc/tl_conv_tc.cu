// Convolution on the 5th-generation tensor cores: implicit GEMM with 3xTF32 split-precision fp32.
//
//   D[pixel][co] = sum_{tap, ci} A[pixel][(tap,ci)] * B[co][(tap,ci)]
//
// One persistent CTA per SM walks tiles of 128 output pixels.  Per tile and 16-channel group a TMA
// tensor copy (cp.async.bulk.tensor, 4-D, out-of-bounds elements = the zero padding) drops the raw
// input patch into shared memory.  Converter warps read it once per filter tap, split every value into
// a TF32 "big" and "small" part (x ~= hi + lo) and store both straight into TENSOR MEMORY as the A
// operand (tcgen05.st): thread = pixel = TMEM lane, 16 columns of hi and 16 of lo per tap, so the im2col
// matrix never exists in shared or global memory.  One thread issues tcgen05.mma kind::tf32 with A from
// TMEM and B (the prepared weights [hi rows | lo rows]) from shared memory:
//     D'[:, 0:2N] += A_hi * [B_hi | B_lo]^T        D'[:, 0:N] += A_lo * B_hi^T
// i.e. the three products of 3xTF32 (the lo*lo term is below fp32 resolution) with fp32 accumulation in
// TMEM.  Epilogue warps read D' with tcgen05.ld, add the two halves and store the output.  The same
// kernel computes the stride-1 input gradient when it is handed the output gradient as "input" and the
// flipped, channel-swapped weights as "B".
//
// Replaces the im2col + mm lowering [ref: lib/sources/pulp_conv2d_fp32.c:85-113, :504-549;
// lib/sources/pulp_im2col_fp32.c:157-232; lib/sources/pulp_matmul_fp32.c:190-262].
#include "tl_kernels.h"
#include "tl_tc.cuh"
#include <cstdlib>

namespace tl {

using namespace tc;

struct ConvTcParams {
    int n, Cin, Cout, Hout, Wout;
    int Wk, taps, sh, sw;
    int TH, TW, S_T, tiles_w, tiles_h, n_tiles;
    int groups;                 // ceil(Cin / 16)
    int PH, PWB, xoff;          // patch rows, patch row pitch in floats, first used column
    int x_base, y_base;         // input coordinate of patch column 0 / row 0 for the tile at the origin
    int NT;                     // output channels per CTA (16, 32 or 64); blockIdx.y picks the slice
    int ring;                   // A buffers per converter group in use (2 or 3: 4*NT + 128*ring <= 512 TMEM columns)
    int nd, nd_log2;            // accumulator buffers in tensor memory (2 or 4: nd*2*NT + 128*ring <= 512 columns)
    const float *w;             // filters [Cout_w][Cin_w][taps]; every CTA builds its B operand from them in its prologue
    int Cout_w, Cin_w, flip;    // flip = input-gradient role: channels swap roles and the taps run backwards
    // Output placement: output pixel (ho, wo) of the tile grid lands at (ho*osy + oy0, wo*osx + ox0) of an oH x oW plane.
    int oH, oW, osy, osx, oy0, ox0;
    // Strided input gradient, one parity class of dX per launch (cls = 1): the "filter" walked by the kernel is the
    // window of dY positions that reach this class; window position (a, b) multiplies filter tap
    // kh = kh_r + kstep*(kh_m - a), kw = kw_r + kstep*(kw_m - b) of the full w_Hk x w_Wk filter (channels swapped as for flip).
    int cls, kstep, kh_r, kh_m, kw_r, kw_m, w_Wk, w_taps;
    const float *bias;
    float *y;
    int *status;                // 0 = ok; set to a wait id when a bounded wait gave up
};

// One thread can start a tcgen05.mma only every ~130 cycles whatever its size (measured on B200), while an
// MMA of this kernel (M 128 x N 32..128 x K 8) keeps the tensor pipe busy for 16..64 cycles.  Four warps
// therefore issue MMAs side by side.  The accumulators start from zero (the epilogue clears them), so the
// order in which the issuers' MMAs land does not matter.
//
// Work is dealt statically: the chunks (one filter tap of one 16-channel group) are numbered in the order
// tile, channel group, tap over the whole run of the CTA, and chunk c belongs to converter group c mod 4
// (4 warps, one per TMEM lane quarter), which converts it into its own ring of RING tensor-memory buffers;
// issuer j multiplies exactly the chunks of group j.  Numbering across tiles keeps the four groups level
// when the chunks of one tile (e.g. 9) do not divide by four.  Every mbarrier thus has one producer group and one consumer that both
// walk the same chunk sequence, so a waiter can never be more than one phase away from the barrier (the
// parity wait would alias otherwise).
static constexpr int GROUPS = 4;            // converter groups = MMA issuers
static constexpr int RING = 2;              // most A buffers per group (32 TMEM columns each: 16 hi + 16 lo); a third one bought nothing
// Warp roles, lightest first: the warp schedulers favour the oldest ready warp, and a converter warp is ready almost
// all the time.  With the epilogue warps last in the CTA (the first layout of this kernel) they were starved: the
// issuers spent a quarter of their time waiting for an accumulator buffer to be released.
static constexpr int FIRST_EPI = 0, FIRST_ISSUER = 4, FIRST_CONV = FIRST_ISSUER + GROUPS, TMA_WARP = FIRST_CONV + 4 * GROUPS;
static constexpr int TC_THREADS = (TMA_WARP + 1) * 32;
static_assert(FIRST_EPI == 0 && FIRST_ISSUER == 4, "the epilogue warps are the first four: warp w reads TMEM lanes 32 * (w % 4)");
static constexpr int PS = 3;                // raw patch ring
static constexpr int NA = GROUPS * RING;    // A buffers in tensor memory
static constexpr int MAX_ND = 4;            // accumulator buffers (2 when 4 would not fit the 512 columns)

// Polling costs issue slots that the converter warps need (half of the instructions this kernel executed were failed
// polls when every failed attempt slept 32 ns): the first attempt is bare, later ones sleep NAP_FAST / NAP_SLOW ns in
// between, and the abort flag is only looked at every 16th attempt.
static constexpr uint32_t NAP_FAST = 128u, NAP_SLOW = 512u;
__device__ __forceinline__ bool tc_wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int id)
{
    // ids 3..5 sit on the critical path and sleep least; about a second of attempts bounds the wait
    if (mbar_try_wait(bar, parity)) return true;
    const uint32_t nap = (id == 3 || id == 4 || id == 5) ? NAP_FAST : NAP_SLOW;
    for (uint32_t i = 0; i < 4000000u; i++) {
        __nanosleep(nap);
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 15u) == 15u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(status, 0, id);
    return false;
}

// Whole-warp variant for callers that go on to warp-collective tcgen05 instructions: every lane polls the same
// barrier in the same instruction, so the warp stays converged and all lanes get the same answer.
__device__ __forceinline__ bool tc_warp_wait_or_abort(uint64_t *bar, uint32_t parity, volatile int *abort_flag, int *status, int id, int lane)
{
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    const uint32_t nap = (id == 3 || id == 4 || id == 5) ? NAP_FAST : NAP_SLOW;
    for (uint32_t i = 0; i < 4000000u; i++) {
        __nanosleep(nap);
        if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
        if ((i & 15u) == 15u && __any_sync(0xffffffffu, *abort_flag != 0)) return false;
    }
    if (lane == 0) { *abort_flag = 1; atomicCAS(status, 0, id); }
    __syncwarp();
    return false;
}

// PLANE_B = bytes between two channels of the shared-memory patch when known at compile time (the 16 loads
// of a tap then carry immediate offsets), 0 = take it from the parameters.
template <int PLANE_B>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmap, const ConvTcParams p)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int NT = p.NT, N2 = 2 * NT;
    const int patch_floats = p.S_T * 16 * p.PH * p.PWB;
    const uint32_t patch_bytes = (uint32_t)patch_floats * 4u;

    // shared memory carve-up
    float *Bs = reinterpret_cast<float *>(smem_raw);                                   // chunks * 32 * NT floats
    const size_t b_floats = (size_t)p.groups * p.taps * 32 * NT;
    float *patch = Bs + ((b_floats + 31) & ~(size_t)31);                               // PS * patch_floats (128-byte aligned)
    const size_t patch_stride = ((size_t)patch_floats + 31) & ~(size_t)31;
    uint64_t *bars = reinterpret_cast<uint64_t *>(patch + PS * patch_stride);
    uint64_t *patch_full = bars, *patch_empty = bars + PS, *a_full = bars + 2 * PS, *a_empty = bars + 2 * PS + NA;
    uint64_t *d_full = bars + 2 * PS + 2 * NA, *d_empty = d_full + MAX_ND;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(d_empty + MAX_ND);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    uint32_t *tap_off = tmem_slot + 2;          // byte offset of every filter tap inside a patch plane (up to 25)

    const uint32_t tmem_cols = 512u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < PS; i++) { mbar_init(&patch_full[i], 1); mbar_init(&patch_empty[i], 4 * GROUPS); }
        for (int i = 0; i < NA; i++) { mbar_init(&a_full[i], 4); mbar_init(&a_empty[i], 1); }
        for (int i = 0; i < MAX_ND; i++) { mbar_init(&d_full[i], GROUPS); mbar_init(&d_empty[i], 4); }
        *abort_flag = 0;
        for (int t = 0; t < p.taps; t++) tap_off[t] = (uint32_t)((t / p.Wk) * p.PWB + (t % p.Wk)) * 4u;
        fence_barrier_init();
        tma_prefetch_desc(&tmap);
    }
    if (warp == TMA_WARP) { tmem_alloc(tmem_slot, tmem_cols); tmem_relinquish(); }
    // B operand of this CTA's output-channel slice, built from the filters straight into shared memory:
    // layout per (group g, tap): [k4 = 0..3][row r = 0..2NT-1][j = 0..3]; row r < NT holds hi(w), row r >= NT lo(w) of
    // output channel co = slice*NT + (r mod NT) and input channel ci = g*16 + k4*4 + j.
    {
        const int half = (int)(b_floats / 2);                  // one (hi, lo) pair per filter value
        const int nt_shift = 31 - __clz(NT);                   // NT is 16, 32 or 64
        for (int e = threadIdx.x; e < half; e += TC_THREADS) {
            const int j = e & 3, rn = (e >> 2) & (NT - 1), k4 = (e >> (2 + nt_shift)) & 3;
            const int rest = e >> (4 + nt_shift);
            const int tap = rest % p.taps, g = rest / p.taps;
            const int n_out = blockIdx.y * NT + rn, k_in = g * 16 + k4 * 4 + j;
            float v = 0.f;
            if (p.cls) {
                const int a = tap / p.Wk, b = tap % p.Wk;
                const int kh = p.kh_r + p.kstep * (p.kh_m - a), kw = p.kw_r + p.kstep * (p.kw_m - b);
                if (n_out < p.Cin_w && k_in < p.Cout_w) v = __ldg(p.w + ((long long)k_in * p.Cin_w + n_out) * p.w_taps + kh * p.w_Wk + kw);
            }
            else if (!p.flip) { if (n_out < p.Cout_w && k_in < p.Cin_w) v = __ldg(p.w + ((long long)n_out * p.Cin_w + k_in) * p.taps + tap); }
            else { if (n_out < p.Cin_w && k_in < p.Cout_w) v = __ldg(p.w + ((long long)k_in * p.Cin_w + n_out) * p.taps + (p.taps - 1 - tap)); }
            uint32_t hi, lo;
            split_tf32(v, hi, lo);
            const int base = ((rest * 4 + k4) * 2 * NT) * 4 + j;
            Bs[base + rn * 4] = __uint_as_float(hi);
            Bs[base + (NT + rn) * 4] = __uint_as_float(lo);
        }
        fence_proxy_async();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t d_col0 = tmem_base, a_col0 = tmem_base + p.nd * N2;      // nd accumulator buffers of 2 NT columns, then the A ring
    const int co0 = blockIdx.y * NT;
    const int tiles_per_stream_group = p.tiles_w * p.tiles_h;

    if (warp == TMA_WARP) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t pc = 0;
            for (int t = blockIdx.x; t < p.n_tiles && !*abort_flag; t += gridDim.x) {
                const int tw0 = (t % p.tiles_w) * p.TW, th0 = ((t / p.tiles_w) % p.tiles_h) * p.TH, s0 = (t / tiles_per_stream_group) * p.S_T;
                for (int g = 0; g < p.groups; g++, pc++) {
                    const int slot = pc % PS;
                    if (!tc_wait_or_abort(&patch_empty[slot], ((pc / PS) & 1) ^ 1, abort_flag, p.status, 1)) break;
                    mbar_arrive_expect_tx(&patch_full[slot], patch_bytes);
                    tma_load_4d(patch + slot * patch_stride, &tmap, &patch_full[slot], p.x_base + tw0 * p.sw, p.y_base + th0 * p.sh, g * 16, s0);
                }
            }
        }
    } else if (warp >= FIRST_ISSUER && warp < FIRST_CONV) {
        // ------------------------------------------------------------ MMA issuers
        if (lane == 0) {
            const int me = warp - FIRST_ISSUER;
            const uint32_t idesc_2n = mma_idesc(FMT_TF32, 128, N2), idesc_n = mma_idesc(FMT_TF32, 128, NT);
            const uint32_t bs_addr = smem_u32(Bs);
            const uint32_t lbo = N2 * 16, sbo = 128;
            const uint32_t tap_bytes = 32u * NT * 4u;
            const uint64_t bdesc0 = smem_desc_kmajor(bs_addr, lbo, sbo);
            uint32_t tcnt = 0;
            int rb = 0; uint32_t rph = 0;       // ring position and phase of this group's next chunk
            uint32_t cbase = 0;                 // chunks dealt so far (all groups), mod GROUPS
            bool ok = true;
            for (int t = blockIdx.x; t < p.n_tiles && ok && !*abort_flag; t += gridDim.x, tcnt++) {
                const int dbuf = tcnt & (p.nd - 1);
                if (!tc_wait_or_abort(&d_empty[dbuf], (tcnt >> p.nd_log2) & 1, abort_flag, p.status, 2)) break;
                tc_fence_after();
                const uint32_t d_addr = d_col0 + dbuf * N2;
                for (int g = 0; g < p.groups && ok; g++, cbase = (cbase + p.taps) & (GROUPS - 1)) {
                    for (int tap = (me - cbase) & (GROUPS - 1); tap < p.taps; tap += GROUPS) {
                        const int abuf = me * p.ring + rb;
                        if (!tc_wait_or_abort(&a_full[abuf], rph, abort_flag, p.status, 3)) { ok = false; break; }
                        if (++rb == p.ring) { rb = 0; rph ^= 1u; }
                        tc_fence_after();
                        const uint32_t a_addr = a_col0 + abuf * 32;
                        // descriptor of this tap's weights: the start-address field (bits 0..13, units of 16 bytes) moves, the rest stays
                        const uint64_t b_tap = bdesc0 + (uint64_t)(((uint32_t)(g * p.taps + tap) * tap_bytes) >> 4);
#pragma unroll
                        for (int kk = 0; kk < 2; kk++) {
                            const uint64_t bdesc = b_tap + (uint64_t)((kk * 2 * lbo) >> 4);
                            mma_tf32_ts(d_addr, a_addr + kk * 8, bdesc, idesc_2n, 1u);
                            mma_tf32_ts(d_addr, a_addr + 16 + kk * 8, bdesc, idesc_n, 1u);
                        }
                        mma_commit(&a_empty[abuf]);
                    }
                }
                if (!ok) break;
                mma_commit(&d_full[dbuf]);       // one arrival per issuer: the tile is complete when all have landed
            }
        }
    } else if (warp >= FIRST_CONV) {
        // ------------------------------------------------------------ converters: raw patch -> (hi, lo) -> tensor memory
        // Warp (q, j): q = TMEM lane quarter (32 pixels), j = 0..3 takes the taps j, j+4, j+8, ... of every
        // channel group, all 16 channels of the group per tap.
        const int cw = warp - FIRST_CONV;
        const int q = warp & 3;                 // TMEM lane quarter this warp may access
        const int j = cw >> 2;                  // converter group: taps j, j+4, j+8, ... of every channel group
        const int m = q * 32 + lane;            // pixel of the tile = TMEM lane
        const int tp = p.TH * p.TW;
        const int sl = m / tp, ph = (m % tp) / p.TW, pw = m % p.TW;
        // all addressing below is 32-bit shared-window arithmetic, set up once per thread
        const uint32_t plane_b = PLANE_B ? (uint32_t)PLANE_B : (uint32_t)(p.PH * p.PWB) * 4u;
        const uint32_t slot_b = (uint32_t)patch_stride * 4u;
        const uint32_t base_b = smem_u32(patch) + (uint32_t)(((sl * 16) * p.PH + ph * p.sh) * p.PWB + p.xoff + pw * p.sw) * 4u;
        uint32_t cbase = 0;                     // chunks dealt so far (all groups), mod GROUPS
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        uint32_t pc = 0;
        int rb = 0; uint32_t rph = 0;           // ring position and phase of this group's next chunk (the paired issuer counts the same)
        bool ok = true;
        for (int t = blockIdx.x; t < p.n_tiles && ok; t += gridDim.x) {
            for (int g = 0; g < p.groups && ok; g++, pc++, cbase = (cbase + p.taps) & (GROUPS - 1)) {
                const int slot = pc % PS;
                if (!tc_warp_wait_or_abort(&patch_full[slot], (pc / PS) & 1, abort_flag, p.status, 4, lane)) { ok = false; break; }
                const int first = (j - cbase) & (GROUPS - 1);
                // Software pipeline over the taps n = first, first+4, ... of this group: while the tensor-memory
                // stores of tap n drain, tap n+1 is split in registers and the raw values of tap n+2 are fetched
                // from shared memory; only then does the warp wait for the stores and hand buffer n to its issuer.
                const uint32_t slot_base = base_b + slot * slot_b;
                float raw[16];
                uint32_t hi[16], lo[16];
                if (first < p.taps) {
                    uint32_t tap_b = slot_base + tap_off[first];
#pragma unroll
                    for (int c = 0; c < 16; c++) raw[c] = ld_shared_f32(tap_b + c * plane_b);
#pragma unroll
                    for (int c = 0; c < 16; c++) split_tf32_fast(raw[c], hi[c], lo[c]);
                    if (first + GROUPS < p.taps) {
                        tap_b = slot_base + tap_off[first + GROUPS];
#pragma unroll
                        for (int c = 0; c < 16; c++) raw[c] = ld_shared_f32(tap_b + c * plane_b);
                    }
                }
                for (int tap = first; tap < p.taps; tap += GROUPS) {
                    const int abuf = j * p.ring + rb;
                    if (!tc_warp_wait_or_abort(&a_empty[abuf], rph ^ 1u, abort_flag, p.status, 5, lane)) { ok = false; break; }
                    if (++rb == p.ring) { rb = 0; rph ^= 1u; }
                    tc_fence_after();
                    const uint32_t a_addr = a_col0 + abuf * 32 + lane_addr;
                    tmem_st16(a_addr, hi);
                    tmem_st16(a_addr + 16, lo);
                    if (tap + GROUPS < p.taps) {
#pragma unroll
                        for (int c = 0; c < 16; c++) split_tf32_fast(raw[c], hi[c], lo[c]);
                        if (tap + 2 * GROUPS < p.taps) {
                            const uint32_t tap_b = slot_base + tap_off[tap + 2 * GROUPS];
#pragma unroll
                            for (int c = 0; c < 16; c++) raw[c] = ld_shared_f32(tap_b + c * plane_b);
                        }
                    }
                    tmem_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&a_full[abuf]);
                }
                __syncwarp();
                if (ok && lane == 0) mbar_arrive(&patch_empty[slot]);
            }
        }
    } else {
        // ------------------------------------------------------------ epilogue: tensor memory -> global
        const int q = warp & 3;
        const int m = q * 32 + lane;
        const int tp = p.TH * p.TW;
        const int sl = m / tp, ph = (m % tp) / p.TW, pw = m % p.TW;
        const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
        const long long plane = (long long)p.oH * p.oW;
        const uint32_t zero8[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const uint32_t zero16[16] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0};
        // all accumulator buffers start from zero; the first "d_empty" phase completes once that is done
        for (int c0 = 0; c0 < p.nd * N2; c0 += 8) tmem_st8(d_col0 + lane_addr + c0, zero8);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) for (int i = 0; i < p.nd; i++) mbar_arrive(&d_empty[i]);
        uint32_t tcnt = 0;
        for (int t = blockIdx.x; t < p.n_tiles; t += gridDim.x, tcnt++) {
            const int dbuf = tcnt & (p.nd - 1);
            const int tw0 = (t % p.tiles_w) * p.TW, th0 = ((t / p.tiles_w) % p.tiles_h) * p.TH, s0 = (t / tiles_per_stream_group) * p.S_T;
            if (!tc_warp_wait_or_abort(&d_full[dbuf], (tcnt >> p.nd_log2) & 1, abort_flag, p.status, 6, lane)) break;
            tc_fence_after();
            const int s = s0 + sl, ho = th0 + ph, wo = tw0 + pw;
            const int oy = ho * p.osy + p.oy0, ox = wo * p.osx + p.ox0;
            const bool valid = (s < p.n) && (ho < p.Hout) && (wo < p.Wout) && (oy < p.oH) && (ox < p.oW);
            float *yp = p.y + ((long long)s * p.Cout + co0) * plane + (long long)oy * p.oW + ox;
            const uint32_t d_addr = d_col0 + dbuf * N2 + lane_addr;
            // 16 output channels per step: both halves of the accumulator are read with one wait, the zeros that clear them
            // for the next tile are issued at once and drain while the results go to global memory
            for (int c0 = 0; c0 < NT; c0 += 16) {
                uint32_t a[16], b[16];
                tmem_ld16(d_addr + c0, a);                      // A_hi*B_hi + A_lo*B_hi
                tmem_ld16(d_addr + NT + c0, b);                 // A_hi*B_lo
                tmem_wait_ld();
                tmem_st16(d_addr + c0, zero16);
                tmem_st16(d_addr + NT + c0, zero16);
                if (valid) {
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const int co = co0 + c0 + j;
                        if (co < p.Cout) {
                            float v = __uint_as_float(a[j]) + __uint_as_float(b[j]);
                            if (p.bias) v += __ldg(p.bias + co);
                            yp[(long long)(c0 + j) * plane] = v;
                        }
                    }
                }
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&d_empty[dbuf]);
        }
    }
    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == TMA_WARP) { __syncwarp(); tc_fence_after(); tmem_dealloc(tmem_base, tmem_cols); }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                  const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess && qres == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)ptr;
        else
            cudaGetLastError();
    }
    return fn;
}

static int *g_status_dev = nullptr;
static int *status_word()
{
    if (!g_status_dev) { if (cudaMalloc(&g_status_dev, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return nullptr; } cudaMemset(g_status_dev, 0, sizeof(int)); }
    return g_status_dev;
}
// the word if a tensor-core kernel has ever been launched, else null (never allocates)
int *tc_status_word_if_any() { return g_status_dev; }
// shared with the tensor-core GEMM (tl_gemm_tc.cu): one status word for every bounded wait of the library
int *tc_status_word() { return status_word(); }
void *tc_encode_tiled_fn() { return (void *)encode_fn(); }

bool conv_mn_run(const float *src, const float *w, const float *bias, float *dst,
                 int n, int C_src, int H_src, int W_src, int C_dst, int H_dst, int W_dst,
                 int Hk, int Wk, int sh, int sw, int padU, int padL, int Cout_w, int Cin_w, bool flip, bool dry_run, const ConvTcClass *cls);

// Runs the tensor-core kernel when the geometry qualifies; returns false to let the caller use the FFMA path.
// src: [n][C_src][H_src][W_src], dst: [n][C_dst][H_dst][W_dst]; `flip` = input-gradient role (stride must be 1).
bool conv_tc_run(Scope &sc, const float *src, const float *w, const float *bias, float *dst,
                 int n, int C_src, int H_src, int W_src, int C_dst, int H_dst, int W_dst,
                 int Hk, int Wk, int sh, int sw, int padU, int padL, int Cout_w, int Cin_w, bool flip, bool dry_run, const ConvTcClass *cls)
{
    if (gemm_path() == 1) return false;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return false;
    if (W_src % 4 != 0 || (((uintptr_t)src) & 15) != 0 || sh != sw || (sh != 1 && sh != 2)) return false;
    if (Hk * Wk > 25 || n < 1) return false;
    int TW, TH, S_T;
    if (W_dst % 32 == 0) { TW = 32; TH = 4; S_T = 1; }
    else if (W_dst == 16) { TW = 16; TH = 8; S_T = 1; }
    else if (W_dst == 8 && H_dst == 8) { TW = 8; TH = 8; S_T = 2; }
    else return false;
    if (H_dst % TH != 0) return false;
    const long long work = (long long)n * H_dst * W_dst * C_dst * C_src * Hk * Wk;
    if (gemm_path() != 2 && work < (1ll << 21)) return false;  // below about 2 M multiply-adds the FFMA tiles finish before the tensor-core prologue does
    // width-preserving stride-1 geometries on 32 / 16 / 8-pixel rows: the kernel that splits every input element once
    if (gemm_path() != 4 && conv_mn_run(src, w, bias, dst, n, C_src, H_src, W_src, C_dst, H_dst, W_dst, Hk, Wk, sh, sw, padU, padL,
                                        Cout_w, Cin_w, flip, dry_run, cls))
        return true;
    if (cls && cls->up) return false;          // pixel-pair classes exist in the row-slot kernel only

    ConvTcParams p;
    p.n = n; p.Cin = C_src; p.Cout = C_dst; p.Hout = H_dst; p.Wout = W_dst;
    p.Wk = Wk; p.taps = Hk * Wk; p.sh = sh; p.sw = sw;
    p.TH = TH; p.TW = TW; p.S_T = S_T;
    p.tiles_w = W_dst / TW; p.tiles_h = H_dst / TH;
    const int tiles_s = ceil_div(n, S_T);
    p.n_tiles = p.tiles_w * p.tiles_h * tiles_s;
    p.groups = ceil_div(C_src, 16);
    // the TMA start column must be a multiple of 4 floats (16 bytes): round down and remember the offset
    const int first = -padL;
    const int aligned = (first >= 0) ? (first / 4) * 4 : -(((-first) + 3) / 4) * 4;
    p.xoff = first - aligned; p.x_base = aligned; p.y_base = -padU;
    p.PH = (TH - 1) * sh + Hk;
    p.PWB = ((p.xoff + (TW - 1) * sw + Wk) + 3) & ~3;
    if (p.PWB > 256 || p.PH > 256) return false;
    const size_t patch_floats = (((size_t)S_T * 16 * p.PH * p.PWB) + 31) & ~(size_t)31;
    // output-channel slice per CTA: the largest of 64/32/16 whose weights fit beside the patch ring
    const int cpad = ((C_dst + 15) / 16) * 16;
    int NT = cpad >= 64 ? 64 : (cpad >= 32 ? 32 : 16);
    size_t smem = 0;
    for (;; NT /= 2) {
        const size_t b_floats = (((size_t)p.groups * p.taps * 32 * NT) + 31) & ~(size_t)31;
        smem = (b_floats + PS * patch_floats) * 4 + (2 * PS + 2 * NA + 2 * MAX_ND) * 8 + 16 + 112 + 128;
        if (smem <= 220 * 1024 || NT == 16) break;
    }
    if (smem > 220 * 1024) return false;
    if (dry_run) return true;   // geometry qualifies; nothing launched
    p.NT = NT;
    p.ring = (4 * NT + 32 * GROUPS * RING <= 512) ? RING : 2;
    p.nd = (MAX_ND * 2 * NT + 32 * GROUPS * p.ring <= 512) ? MAX_ND : 2;
    p.nd_log2 = p.nd == 4 ? 2 : 1;
    const int co_tiles = ceil_div(C_dst, NT);

    CUtensorMap tmap;
    cuuint64_t gdim[4] = {(cuuint64_t)W_src, (cuuint64_t)H_src, (cuuint64_t)C_src, (cuuint64_t)n};
    cuuint64_t gstr[3] = {(cuuint64_t)W_src * 4, (cuuint64_t)W_src * H_src * 4, (cuuint64_t)W_src * H_src * C_src * 4};
    cuuint32_t box[4] = {(cuuint32_t)p.PWB, (cuuint32_t)p.PH, 16u, (cuuint32_t)S_T};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    if (enc(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, (void *)src, gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return false;

    int *status = status_word();
    if (!status) return false;
    p.w = w; p.Cout_w = Cout_w; p.Cin_w = Cin_w; p.flip = flip ? 1 : 0;
    p.oH = H_dst; p.oW = W_dst; p.osy = p.osx = 1; p.oy0 = p.ox0 = 0;
    p.cls = 0; p.kstep = 1; p.kh_r = p.kh_m = p.kw_r = p.kw_m = 0; p.w_Wk = Wk; p.w_taps = Hk * Wk;
    if (cls) {
        p.cls = 1; p.kstep = cls->kstep; p.kh_r = cls->kh_r; p.kh_m = cls->kh_m; p.kw_r = cls->kw_r; p.kw_m = cls->kw_m;
        p.w_Wk = cls->w_Wk; p.w_taps = cls->w_Hk * cls->w_Wk;
        p.oH = cls->oH; p.oW = cls->oW; p.osy = cls->osy; p.osx = cls->osx; p.oy0 = cls->oy0; p.ox0 = cls->ox0;
    }
    p.bias = bias; p.y = dst; p.status = status;
    int ctas = sm_count() / co_tiles;
    if (ctas < 1) ctas = 1;
    if (ctas > p.n_tiles) ctas = p.n_tiles;
    dim3 grid(ctas, co_tiles);
    const int plane_b = p.PH * p.PWB * 4;
#define TL_TC_LAUNCH(PB)                                                                                              \
    do {                                                                                                              \
        static bool attr_set = false;                                                                                 \
        if (!attr_set) { cudaFuncSetAttribute(conv_tc_kernel<PB>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024); attr_set = true; } \
        TL_LAUNCH(conv_tc_kernel<PB>, grid, TC_THREADS, smem, tmap, p);                                               \
    } while (0)
    switch (plane_b) {                       // the patch shapes of 32x32 / 16x16 / 8x8 images with 3x3 and 1x1 filters
    case 960: TL_TC_LAUNCH(960); break;      // 6 x 40 and 10 x 24 and 15 x 16 floats
    case 640: TL_TC_LAUNCH(640); break;      // 10 x 16
    case 2448: TL_TC_LAUNCH(2448); break;    // 17 x 36 (stride 2, 16 output columns)
    case 1360: TL_TC_LAUNCH(1360); break;    // 17 x 20 (stride 2, 8 output columns)
    case 1920: TL_TC_LAUNCH(1920); break;    // 15 x 32 (1x1 stride 2)
    case 512: TL_TC_LAUNCH(512); break;      // 4 x 32 and 8 x 16 (1x1 stride 1)
    case 720: TL_TC_LAUNCH(720); break;      // parity classes of a strided input gradient, 16 x 16 class grid: 9 x 20,
    case 576: TL_TC_LAUNCH(576); break;      //   9 x 16 (and 8 x 20 = 640, 8 x 16 = 512 above)
    case 432: TL_TC_LAUNCH(432); break;      // 8 x 8 class grid: 9 x 12,
    case 384: TL_TC_LAUNCH(384); break;      //   8 x 12,
    case 288: TL_TC_LAUNCH(288); break;      //   9 x 8,
    case 256: TL_TC_LAUNCH(256); break;      //   8 x 8
    default: TL_TC_LAUNCH(0); break;
    }
#undef TL_TC_LAUNCH
    profile_add_flops(2.0 * n * C_dst * C_src * Hk * Wk * H_dst * W_dst);
    return true;
}

// Non-zero after a kernel gave up on a bounded wait (which wait is encoded in the value).
int conv_tc_status()
{
    int *dev = g_status_dev;
    if (!dev) return 0;                     // no tensor-core kernel has run
    int h = 0;
    // on the library's stream: ordered behind the kernels that may still write the word
    if (cudaMemcpyAsync(&h, dev, sizeof(int), cudaMemcpyDeviceToHost, stream()) == cudaSuccess && cudaStreamSynchronize(stream()) == cudaSuccess) return h;
    cudaGetLastError();
    return -1;
}

} // namespace tl
