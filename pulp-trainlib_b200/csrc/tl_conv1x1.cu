// 1x1 convolutions with a stride and no padding (the projection shortcuts of a residual network), fp32, CUDA cores.
//
//   forward          Y[co][p]          = sum_ci W[co][ci] * X[ci][s*oy][s*ox]              p = (oy, ox)
//   input gradient   dX[ci][s*oy][s*ox] += sum_co W[co][ci] * dY[co][p]                    (the pixels in between: untouched)
//   weight gradient  dW[co][ci]        = sum over streams and p of dY[co][p] * X[ci][s*oy][s*ox]
//
// Two FLOP per byte moved: all three are bound by memory traffic, so they are built around the loads.  Every kernel is
// persistent (a few CTAs per SM) and walks (stream, 64-pixel tile) items through a three-stage ring of shared-memory tiles
// filled with cp.async: the sampled input pixels are gathered 4 bytes at a time, dY tiles 16 bytes at a time, and the loads
// of the next two items are in flight while the current one is multiplied.  The products are small (K = 16 ... 64) and run
// on the warp-level tensor-core instruction (mma.sync m16n8k8, TF32 operands split into high and low parts in registers,
// three products per term, fp32 accumulation): next to an FFMA register tile that takes the shared-memory load traffic
// from 32 bytes per 16 FMAs to 8 bytes per 768, which is what bounded the FFMA version of these kernels.  The
// weights live in registers as ready-made fragments for the life of the CTA (forward, input gradient).  The weight
// gradient has the pixels as contraction index: a warp multiplies its 8 pixels of every tile, adds the tile's result to
// fp32 accumulators it keeps for the whole launch, the warps' sums are added in warp order through shared memory at the
// end, and every CTA leaves one partial result for reduce_partials_kernel (fixed order, no atomics).
// Replaces the im2col + mm lowering and the naive kernels for these shapes
// [ref: lib/sources/pulp_conv2d_fp32.c:85-113, :294-333, :504-549; lib/sources/pulp_conv_naive_fp32.c:198-516].
#include "tl_kernels.h"

namespace tl {

static constexpr int C1_TP = 64;          // pixels per tile
// floats between the rows of a staged tile (16-byte alignment kept), chosen so that the fragment loads of a warp hit 32 banks:
static constexpr int C1_LDK = C1_TP + 8;  // tiles read down the rows (lane -> row t, column g): forward and input gradient
static constexpr int C1_LDM = C1_TP + 4;  // tiles read along the rows (lane -> row g, column t): weight gradient
static constexpr int C1_THREADS = 256;
static constexpr int C1_NST = 3;          // ring stages
static constexpr size_t C1_SMEM_MAX = 200 * 1024;

struct Conv1x1Params {
    int n, Cin, Cout, Hin, Win, Ho, Wo, sh, sw;
    int tiles;                            // pixel tiles per stream
    int items;                            // n * tiles
    int yvec;                             // dY / Y rows may be moved 16 bytes at a time (pixel count and base address allow it)
    int tshift, wshift;                   // log2 of tiles / Wo where they are powers of two, else -1 (plain division)
    int opix, plane;                      // Ho * Wo, Hin * Win
};

__device__ __forceinline__ void c1_cp4(uint32_t dst, const float *src) { asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void c1_cp16(uint32_t dst, const float *src) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory"); }
__device__ __forceinline__ void c1_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void c1_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void c1_st_zero(uint32_t dst) { asm volatile("st.shared.b32 [%0], %1;" ::"r"(dst), "r"(0u) : "memory"); }
// v = q * d + r; a shift where the host found d to be a power of two (the usual case: 8, 16, 32 pixels per row)
__device__ __forceinline__ void c1_divmod(unsigned v, unsigned d, int shift, unsigned &q, unsigned &r)
{
    if (shift >= 0) { q = v >> shift; r = v & (d - 1); }
    else { q = v / d; r = v - q * d; }
}
// offset of output pixel px's sample inside an input plane
__device__ __forceinline__ unsigned c1_sample(const Conv1x1Params &p, unsigned px)
{
    unsigned oy, ox;
    c1_divmod(px, (unsigned)p.Wo, p.wshift, oy, ox);
    return oy * (unsigned)(p.sh * p.Win) + ox * (unsigned)p.sw;
}

// tile[c][q] <- plane c of stream `xs` at the sampled position of pixel p0 + q (zero past the last pixel); asynchronous.
// `tile` is a shared-space byte address.
template <int LD> __device__ __forceinline__ void gather_tile_async(const Conv1x1Params &p, const float *__restrict__ xs, uint32_t tile, unsigned p0, int C)
{
    const unsigned q = threadIdx.x % C1_TP, c0 = threadIdx.x / C1_TP, px = p0 + q;
    uint32_t dst = tile + (c0 * LD + q) * 4;
    if (px < (unsigned)p.opix) {
        const float *src = xs + c1_sample(p, px) + (size_t)c0 * p.plane;
        const size_t step = (size_t)(C1_THREADS / C1_TP) * p.plane;
        for (int c = c0; c < C; c += C1_THREADS / C1_TP, src += step, dst += (C1_THREADS / C1_TP) * LD * 4) c1_cp4(dst, src);
    } else
        for (int c = c0; c < C; c += C1_THREADS / C1_TP, dst += (C1_THREADS / C1_TP) * LD * 4) c1_st_zero(dst);
}
// tile[c][q] <- ys[c][p0 + q] (zero past the last pixel); asynchronous
template <int LD> __device__ __forceinline__ void load_tile_async(const Conv1x1Params &p, const float *__restrict__ ys, uint32_t tile, unsigned p0, int C)
{
    if (p.yvec) {                                                   // opix % 4 == 0: a quad is inside or outside as a whole
        constexpr int ROWS = C1_THREADS / (C1_TP / 4);
        const unsigned q = (threadIdx.x % (C1_TP / 4)) * 4, c0 = threadIdx.x / (C1_TP / 4), px = p0 + q;
        uint32_t dst = tile + (c0 * LD + q) * 4;
        if (px < (unsigned)p.opix) {
            const float *src = ys + c0 * (unsigned)p.opix + px;
            for (int c = c0; c < C; c += ROWS, src += ROWS * p.opix, dst += ROWS * LD * 4) c1_cp16(dst, src);
        } else
            for (int c = c0; c < C; c += ROWS, dst += ROWS * LD * 4) { c1_st_zero(dst); c1_st_zero(dst + 4); c1_st_zero(dst + 8); c1_st_zero(dst + 12); }
    } else {
        constexpr int ROWS = C1_THREADS / C1_TP;
        const unsigned q = threadIdx.x % C1_TP, c0 = threadIdx.x / C1_TP, px = p0 + q;
        uint32_t dst = tile + (c0 * LD + q) * 4;
        if (px < (unsigned)p.opix) {
            const float *src = ys + c0 * (unsigned)p.opix + px;
            for (int c = c0; c < C; c += ROWS, src += ROWS * p.opix, dst += ROWS * LD * 4) c1_cp4(dst, src);
        } else
            for (int c = c0; c < C; c += ROWS, dst += ROWS * LD * 4) c1_st_zero(dst);
    }
}

// The ring: ISSUE(stream, first pixel, stage) starts the loads of an item, BODY(stream, first pixel, stage) consumes them.
// One commit group per step, empty when there is nothing left to load, so that "all but the newest C1_NST - 1 groups"
// always means "this item".
#define C1_ITEM(it, s_, p0_) unsigned s_, p0_; c1_divmod((unsigned)(it), (unsigned)p.tiles, p.tshift, s_, p0_); p0_ *= C1_TP
#define C1_RING(ISSUE, BODY)                                                                                          \
    do {                                                                                                              \
        const int step = gridDim.x;                                                                                   \
        for (int j = 0; j < C1_NST - 1; j++) {                                                                        \
            const int it = blockIdx.x + j * step;                                                                     \
            if (it < p.items) { C1_ITEM(it, s_, p0_); ISSUE(s_, p0_, j); }                                            \
            c1_commit();                                                                                              \
        }                                                                                                             \
        int stage = 0;                                                                                                \
        for (int it = blockIdx.x; it < p.items; it += step) {                                                         \
            const int nxt = it + (C1_NST - 1) * step, nst = stage == 0 ? C1_NST - 1 : stage - 1;                      \
            if (nxt < p.items) { C1_ITEM(nxt, s_, p0_); ISSUE(s_, p0_, nst); }   /* the stage consumed one step ago: the trailing barrier freed it */ \
            c1_commit();                                                                                              \
            c1_wait<C1_NST - 1>();                                                                                    \
            __syncthreads();                                                                                          \
            { C1_ITEM(it, s_, p0_); BODY(s_, p0_, stage); }                                                           \
            __syncthreads();                                                                                          \
            stage = stage == C1_NST - 1 ? 0 : stage + 1;                                                              \
        }                                                                                                             \
        c1_wait<0>();                                                                                                 \
    } while (0)

// x = hi + lo with both parts representable in TF32 (10-bit mantissa); hi * hi' + hi * lo' + lo * hi' carries 21+ bits
__device__ __forceinline__ void split_tf32(float x, uint32_t &hi, uint32_t &lo)
{
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hi) : "f"(x));
    const float r = x - __uint_as_float(hi);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lo) : "f"(r));
}
// D (16 x 8, fp32) += A (16 x 8, row) * B (8 x 8, col).  Lane = 4 g + t holds A[g][t], A[g+8][t], A[g][t+4], A[g+8][t+4];
// B[t][g], B[t+4][g]; D[g][2t], D[g][2t+1], D[g+8][2t], D[g+8][2t+1].
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1)
{
    asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// the three products of the split, small terms first
__device__ __forceinline__ void mma_3x(float (&d)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4], uint32_t bh0, uint32_t bh1, uint32_t bl0, uint32_t bl1)
{
    mma_tf32(d, al, bh0, bh1); mma_tf32(d, ah, bl0, bl1); mma_tf32(d, ah, bh0, bh1);
}


// Forward (IG = false): Y[co][px] = sum_ci W[co][ci] X[ci][px] (+ bias).  Input gradient (IG = true): dX[ci][px] += sum_co
// W[co][ci] dY[co][px], the old values of dX at the sampled positions riding the ring beside the dY tile.
// M = the output's channels (16 per instruction), N = pixels (8), K = KT * 8 contraction channels.  The 8 warps are
// m_groups x n_groups: a warp owns MTW 16-channel blocks, whose weight fragments it keeps in registers, and every
// n_groups-th 8-pixel column block of a tile.
template <int KT, int MTW, bool IG>
__global__ void __launch_bounds__(C1_THREADS, (KT * MTW <= 4) ? 4 : 2) conv1x1s_mma_kernel(Conv1x1Params p, const float *__restrict__ src, const float *__restrict__ w,
                                                                  const float *__restrict__ bias, float *__restrict__ dst)
{
    constexpr int LD = C1_LDK, K = KT * 8;
    extern __shared__ __align__(16) float c1_smem[];
    const uint32_t smem_s = (uint32_t)__cvta_generic_to_shared(c1_smem);
    const int M = IG ? p.Cin : p.Cout;
    const int tile_f = (IG ? (K + M) : K) * LD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m_groups = M / (16 * MTW), n_groups = 8 / m_groups, mg = warp % m_groups, ng = warp / m_groups;
    const size_t src_stream = IG ? (size_t)p.Cout * p.opix : (size_t)p.Cin * p.plane, dst_stream = IG ? (size_t)p.Cin * p.plane : (size_t)p.Cout * p.opix;
    uint32_t ah[MTW][KT][4], al[MTW][KT][4];
    int row_off[MTW][2];                                            // offset of the thread's result rows inside a stream of dst
    float row_bias[MTW][2];
#pragma unroll
    for (int mt = 0; mt < MTW; mt++) {
#pragma unroll
        for (int kt = 0; kt < KT; kt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int r = (mg * MTW + mt) * 16 + g + (e & 1) * 8, c = kt * 8 + t + (e >> 1) * 4;
                split_tf32(IG ? w[(size_t)c * p.Cin + r] : w[(size_t)r * p.Cin + c], ah[mt][kt][e], al[mt][kt][e]);
            }
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int r = (mg * MTW + mt) * 16 + g + h * 8;
            row_off[mt][h] = r * (IG ? p.plane : p.opix);
            row_bias[mt][h] = (!IG && bias) ? bias[r] : 0.f;
        }
    }
    auto issue = [&](unsigned s, unsigned p0, int st) {
        const uint32_t tile = smem_s + st * tile_f * 4;
        if (IG) {
            load_tile_async<LD>(p, src + s * src_stream, tile, p0, K);
            gather_tile_async<LD>(p, dst + s * dst_stream, tile + K * LD * 4, p0, M);
        } else
            gather_tile_async<LD>(p, src + s * src_stream, tile, p0, K);
    };
    auto body = [&](unsigned s, unsigned p0, int st) {
        const float *act = c1_smem + st * tile_f + t * LD + g, *old = c1_smem + st * tile_f + K * LD + 2 * t;
        float *out = dst + s * dst_stream;
        for (int j = 0; j < m_groups; j++) {
            const int n0 = (ng + j * n_groups) * 8;
            const unsigned px = p0 + n0 + 2 * t;
            if (p0 + n0 >= (unsigned)p.opix) break;                 // column blocks past the last pixel (the same for the whole warp)
            float d[MTW][4];
#pragma unroll
            for (int mt = 0; mt < MTW; mt++) { d[mt][0] = d[mt][1] = d[mt][2] = d[mt][3] = 0.f; }
#pragma unroll
            for (int kt = 0; kt < KT; kt++) {
                uint32_t bh0, bl0, bh1, bl1;
                split_tf32(act[kt * 8 * LD + n0], bh0, bl0);
                split_tf32(act[(kt * 8 + 4) * LD + n0], bh1, bl1);
#pragma unroll
                for (int mt = 0; mt < MTW; mt++) mma_3x(d[mt], ah[mt][kt], al[mt][kt], bh0, bh1, bl0, bl1);
            }
            if (IG) {
                const bool in0 = px < (unsigned)p.opix, in1 = px + 1 < (unsigned)p.opix;
                const unsigned o0 = in0 ? c1_sample(p, px) : 0, o1 = in1 ? c1_sample(p, px + 1) : 0;
#pragma unroll
                for (int mt = 0; mt < MTW; mt++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const float2 was = *reinterpret_cast<const float2 *>(old + ((mg * MTW + mt) * 16 + g + h * 8) * LD + n0);
                        float *o = out + row_off[mt][h];
                        if (in0) o[o0] = __fadd_rn(d[mt][2 * h], was.x);
                        if (in1) o[o1] = __fadd_rn(d[mt][2 * h + 1], was.y);
                    }
            } else {
#pragma unroll
                for (int mt = 0; mt < MTW; mt++)
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        float *o = out + row_off[mt][h] + px;
                        const float v0 = d[mt][2 * h] + row_bias[mt][h], v1 = d[mt][2 * h + 1] + row_bias[mt][h];
                        if (p.yvec) { if (px < (unsigned)p.opix) *reinterpret_cast<float2 *>(o) = make_float2(v0, v1); }
                        else { if (px < (unsigned)p.opix) o[0] = v0; if (px + 1 < (unsigned)p.opix) o[1] = v1; }
                    }
            }
        }
    };
    C1_RING(issue, body);
}

// Weight gradient: dW[co][ci] = sum over streams and pixels of dY[co][px] X[ci][px].  M = co (16 per instruction), N = ci
// (8), K = pixels (8).  The 8 warps are m_groups x k_groups: a warp owns MTW 16-row blocks of dW in all NT 8-column
// blocks and every k_groups-th 8-pixel slice of a tile.  Both operands change with every tile and are split on the way
// from shared memory to the instruction.
template <int MTW, int NT>
__global__ void __launch_bounds__(C1_THREADS, (MTW * NT <= 4) ? 4 : 2) conv1x1s_wg_kernel(Conv1x1Params p, const float *__restrict__ x, const float *__restrict__ dy, float *__restrict__ part)
{
    constexpr int LD = C1_LDM;
    extern __shared__ __align__(16) float c1_smem[];
    const uint32_t smem_s = (uint32_t)__cvta_generic_to_shared(c1_smem);
    const int tile_f = (p.Cin + p.Cout) * LD;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int m_groups = p.Cout / (16 * MTW), k_groups = 8 / m_groups, mg = warp % m_groups, kg = warp / m_groups;
    const size_t x_stream = (size_t)p.Cin * p.plane, y_stream = (size_t)p.Cout * p.opix;
    float run[MTW][NT][4];
#pragma unroll
    for (int mt = 0; mt < MTW; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++) { run[mt][nt][0] = run[mt][nt][1] = run[mt][nt][2] = run[mt][nt][3] = 0.f; }
    auto issue = [&](unsigned s, unsigned p0, int st) {
        const uint32_t tile = smem_s + st * tile_f * 4;
        gather_tile_async<LD>(p, x + s * x_stream, tile, p0, p.Cin);
        load_tile_async<LD>(p, dy + s * y_stream, tile + p.Cin * LD * 4, p0, p.Cout);
    };
    auto body = [&](unsigned, unsigned p0, int st) {
        const float *xa = c1_smem + st * tile_f + g * LD + t, *ya = c1_smem + st * tile_f + (p.Cin + mg * MTW * 16 + g) * LD + t;
        float d[MTW][NT][4];
#pragma unroll
        for (int mt = 0; mt < MTW; mt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++) { d[mt][nt][0] = d[mt][nt][1] = d[mt][nt][2] = d[mt][nt][3] = 0.f; }
        for (int j = 0; j < m_groups; j++) {
            const int k0 = (kg + j * k_groups) * 8;
            if (p0 + k0 >= (unsigned)p.opix) break;                 // pixel slices past the last pixel hold zeros
            uint32_t ah[MTW][4], al[MTW][4];
#pragma unroll
            for (int mt = 0; mt < MTW; mt++)
#pragma unroll
                for (int e = 0; e < 4; e++) split_tf32(ya[(mt * 16 + (e & 1) * 8) * LD + k0 + (e >> 1) * 4], ah[mt][e], al[mt][e]);
#pragma unroll
            for (int nt = 0; nt < NT; nt++) {
                uint32_t bh0, bl0, bh1, bl1;
                split_tf32(xa[nt * 8 * LD + k0], bh0, bl0);
                split_tf32(xa[nt * 8 * LD + k0 + 4], bh1, bl1);
#pragma unroll
                for (int mt = 0; mt < MTW; mt++) mma_3x(d[mt][nt], ah[mt], al[mt], bh0, bh1, bl0, bl1);
            }
        }
#pragma unroll
        for (int mt = 0; mt < MTW; mt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++) run[mt][nt][e] += d[mt][nt][e];
    };
    C1_RING(issue, body);
    // sum the k groups in group order: red[kg][co][ci]
    __syncthreads();
    float *red = c1_smem;
    const int nw = p.Cout * p.Cin;
#pragma unroll
    for (int mt = 0; mt < MTW; mt++)
#pragma unroll
        for (int nt = 0; nt < NT; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const int co = (mg * MTW + mt) * 16 + g + (e >> 1) * 8, ci = nt * 8 + 2 * t + (e & 1);
                red[kg * nw + co * p.Cin + ci] = run[mt][nt][e];
            }
    __syncthreads();
    for (int e = threadIdx.x; e < nw; e += C1_THREADS) {
        float v = 0.f;
        for (int k = 0; k < k_groups; k++) v += red[k * nw + e];
        part[(size_t)blockIdx.x * nw + e] = v;
    }
}

static int c1_log2(int v) { int s = 0; while ((1 << s) < v) s++; return (1 << s) == v ? s : -1; }
static bool c1_geometry(const ConvGeom &g, Conv1x1Params &p, const void *rows)
{
    if (!(g.Hk == 1 && g.Wk == 1 && g.padU == 0 && g.padL == 0 && !g.depthwise && !g.hwc && (g.sh > 1 || g.sw > 1))) return false;
    if (g.Cin % 16 != 0 || g.Cout % 16 != 0 || g.Cin > 128 || g.Cout > 128 || g.n < 1) return false;
    if ((long long)(g.Hout - 1) * g.sh >= g.Hin || (long long)(g.Wout - 1) * g.sw >= g.Win) return false;
    if ((long long)g.Hin * g.Win * 128 > 0x7fffffffLL || (long long)g.Hout * g.Wout * 128 > 0x7fffffffLL) return false;   // 32-bit offsets inside a stream
    p.n = g.n; p.Cin = g.Cin; p.Cout = g.Cout; p.Hin = g.Hin; p.Win = g.Win; p.Ho = g.Hout; p.Wo = g.Wout; p.sh = g.sh; p.sw = g.sw;
    p.opix = g.Hout * g.Wout; p.plane = g.Hin * g.Win;
    p.tiles = ceil_div(p.opix, C1_TP);
    if ((long long)g.n * p.tiles > 0x7fffffffLL / 4) return false;
    p.items = g.n * p.tiles;
    p.yvec = (p.opix % 4 == 0 && (((uintptr_t)rows) & 15) == 0) ? 1 : 0;
    p.tshift = c1_log2(p.tiles); p.wshift = c1_log2(p.Wo);
    return true;
}
static double c1_flops(const ConvGeom &g) { return 2.0 * g.n * g.Cout * g.Cin * g.Hout * g.Wout; }
// persistent grid: as many CTAs per SM as shared memory allows, at most 4
static int c1_grid(size_t smem, int items)
{
    int per_sm = (int)((220 * 1024) / (smem + 1024));
    per_sm = per_sm < 1 ? 1 : (per_sm > 4 ? 4 : per_sm);
    const long long ctas = (long long)sm_count() * per_sm;
    return (int)(ctas < items ? ctas : items);
}
// M = channels of the result (multiple of 16), K = contraction channels: the kernel variant that covers them, if any.
// MTW = 2 blocks per warp while the weight fragments fit the registers (K <= 32) and M has two blocks to give.
template <bool IG> static bool c1_launch(const Conv1x1Params &p, int M, int K, size_t smem, const float *src, const float *w, const float *bias, float *dst)
{
    const int mtw = (K <= 32 && M % 32 == 0) ? 2 : 1, m_groups = M / (16 * mtw);
    if (m_groups != 1 && m_groups != 2 && m_groups != 4 && m_groups != 8) return false;
#define C1_CASE(KTV, MTWV)                                                                                                     \
    if (K == KTV * 8 && mtw == MTWV) {                                                                                         \
        if (smem > 48 * 1024) cudaFuncSetAttribute(conv1x1s_mma_kernel<KTV, MTWV, IG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (IG) TL_LAUNCH((conv1x1s_mma_kernel<KTV, MTWV, true>), c1_grid(smem, p.items), C1_THREADS, smem, p, src, w, bias, dst); \
        else TL_LAUNCH((conv1x1s_mma_kernel<KTV, MTWV, false>), c1_grid(smem, p.items), C1_THREADS, smem, p, src, w, bias, dst); \
        return true;                                                                                                           \
    }
    C1_CASE(2, 1) C1_CASE(2, 2) C1_CASE(4, 1) C1_CASE(4, 2) C1_CASE(8, 1)
#undef C1_CASE
    return false;
}

bool conv1x1s_fw(const ConvGeom &g, const float *x, const float *w, const float *bias, float *y)
{
    Conv1x1Params p;
    if (!c1_geometry(g, p, y) || gemm_path() == 1 || gemm_path() == 2) return false;
    const size_t smem = (size_t)C1_NST * g.Cin * C1_LDK * sizeof(float);
    if (smem > C1_SMEM_MAX || !c1_launch<false>(p, g.Cout, g.Cin, smem, x, w, bias, y)) return false;
    profile_add_flops(c1_flops(g));
    return true;
}

// dX += the input gradient (the sampled positions only; the others keep their values)
bool conv1x1s_ig(const ConvGeom &g, const float *dy, const float *w, float *dx)
{
    Conv1x1Params p;
    if (!c1_geometry(g, p, dy) || gemm_path() == 1) return false;
    const size_t smem = (size_t)C1_NST * (g.Cin + g.Cout) * C1_LDK * sizeof(float);
    if (smem > C1_SMEM_MAX || !c1_launch<true>(p, g.Cin, g.Cout, smem, dy, w, nullptr, dx)) return false;
    profile_add_flops(c1_flops(g));
    return true;
}

// Partial results: `*groups_out` blocks of Cout*Cin floats in `part` (capacity part_groups); false = not covered, nothing launched.
bool conv1x1s_wg(const ConvGeom &g, const float *x, const float *dy, float *part, int part_groups, int *groups_out, bool dry_run)
{
    Conv1x1Params p;
    if (!c1_geometry(g, p, dy) || gemm_path() == 1) return false;
    const int NT = g.Cin / 8, mtw = (NT <= 4 && g.Cout % 32 == 0) ? 2 : 1, m_groups = g.Cout / (16 * mtw);
    if (m_groups != 1 && m_groups != 2 && m_groups != 4 && m_groups != 8) return false;
    if (NT != 2 && NT != 4 && NT != 8) return false;
    const size_t ring = (size_t)C1_NST * (g.Cin + g.Cout) * C1_LDM * sizeof(float), red = (size_t)(8 / m_groups) * g.Cout * g.Cin * sizeof(float);
    const size_t smem = ring > red ? ring : red;
    if (smem > C1_SMEM_MAX) return false;
    const int ctas = c1_grid(smem, p.items);
    if (ctas > part_groups) return false;
    *groups_out = ctas;
    if (dry_run) return true;
#define C1_CASE(MTWV, NTV)                                                                                                     \
    if (mtw == MTWV && NT == NTV) {                                                                                            \
        if (smem > 48 * 1024) cudaFuncSetAttribute(conv1x1s_wg_kernel<MTWV, NTV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        TL_LAUNCH((conv1x1s_wg_kernel<MTWV, NTV>), ctas, C1_THREADS, smem, p, x, dy, part);                                      \
        profile_add_flops(c1_flops(g));                                                                                        \
        return true;                                                                                                           \
    }
    C1_CASE(1, 2) C1_CASE(2, 2) C1_CASE(1, 4) C1_CASE(2, 4) C1_CASE(1, 8)
#undef C1_CASE
    return false;
}

} // namespace tl
