// Convolution kernels.  The reference lowers Conv2D to im2col + matmul
// [ref: lib/sources/pulp_conv2d_fp32.c:85-113 (FW), :294-333 (WG), :504-549 (IG)] or runs
// naive 7-deep loops [ref: lib/sources/pulp_conv_naive_fp32.c:198,302,410].  Here each step is
// one implicit-GEMM kernel: the receptive fields are gathered from a zero-filled input patch
// in shared memory, so no column buffer ever exists in global memory.  All kernels take
// `n` independent batch-1 streams ([n][C][H][W] activations, shared weights).
#include "tl_kernels.h"

namespace tl {

// multiply-adds of the operator's definition x 2 (borders counted as full windows)
static double conv_flops(const ConvGeom &g) { return 2.0 * g.n * g.Cout * (g.depthwise ? 1 : g.Cin) * g.Hk * g.Wk * g.Hout * g.Wout; }

static constexpr int CONV_THREADS = 256;
static constexpr int CO_T = 16;            // output channels per thread (register tile)

// ------------------------------------------------------------------ forward
// CTA = S_T streams x (TH x TW) output pixels x CO_T output channels; one thread per pixel.
// Loop over input-channel chunks: stage patch [S_T][cc][PH][PW] and weights [cc][Hk*Wk][CO_T].
template <class T>
__global__ void __launch_bounds__(CONV_THREADS)
conv_fw_kernel(ConvGeom g, const T *__restrict__ x, const T *__restrict__ w, const T *__restrict__ bias,
               T *__restrict__ y, int TH, int TW, int S_T, int CC, int tiles_w, int tiles_h)
{
    extern __shared__ __align__(16) float smem[];
    const int PH = (TH - 1) * g.sh + g.Hk, PW = (TW - 1) * g.sw + g.Wk;
    const int PWp = PW | 1;                                  // odd row pitch: fewer bank conflicts
    const int KK = g.Hk * g.Wk;
    float *patch = smem;                                     // [S_T][CC][PH][PWp]
    float *wsm = smem + (((size_t)S_T * CC * PH * PWp + 3) & ~(size_t)3);   // [CC][KK][CO_T], 16-byte aligned for float4 reads

    const int tid = threadIdx.x;
    const int tile = blockIdx.x;
    const int tw0 = (tile % tiles_w) * TW, th0 = ((tile / tiles_w) % tiles_h) * TH;
    const int s0 = (tile / (tiles_w * tiles_h)) * S_T;
    const int co0 = blockIdx.y * CO_T;

    const int pix = tid % (TH * TW), sl = tid / (TH * TW);   // local pixel / local stream
    const int ph = pix / TW, pw = pix % TW;
    const bool active = (sl < S_T) && (s0 + sl < g.n) && (th0 + ph < g.Hout) && (tw0 + pw < g.Wout);

    float acc[CO_T];
#pragma unroll
    for (int c = 0; c < CO_T; c++) acc[c] = 0.f;

    const int h_in0 = th0 * g.sh - g.padU, w_in0 = tw0 * g.sw - g.padL;
    const long long in_plane = (long long)g.Hin * g.Win;

    for (int ci0 = 0; ci0 < g.Cin; ci0 += CC) {
        const int cc = min(CC, g.Cin - ci0);
        // stage the input patch (zero outside the image = padding)
        const int patch_elems = S_T * cc * PH * PW;
        for (int e = tid; e < patch_elems; e += CONV_THREADS) {
            int c = e % PW, r = (e / PW) % PH, ci = (e / (PW * PH)) % cc, s = e / (PW * PH * cc);
            int hi = h_in0 + r, wi = w_in0 + c;
            float v = 0.f;
            if (s0 + s < g.n && hi >= 0 && hi < g.Hin && wi >= 0 && wi < g.Win)
                v = ld(x + ((long long)(s0 + s) * g.Cin + ci0 + ci) * in_plane + (long long)hi * g.Win + wi);
            patch[((s * CC + ci) * PH + r) * PWp + c] = v;
        }
        // stage weights as [ci][tap][co]
        const int w_elems = cc * KK * CO_T;
        for (int e = tid; e < w_elems; e += CONV_THREADS) {
            int co = e % CO_T, t = (e / CO_T) % KK, ci = e / (CO_T * KK);
            float v = 0.f;
            if (co0 + co < g.Cout) v = ld(w + ((long long)(co0 + co) * g.Cin + ci0 + ci) * KK + t);
            wsm[(ci * KK + t) * CO_T + co] = v;
        }
        __syncthreads();
        if (active) {
            const float *pbase = patch + ((sl * CC) * PH + ph * g.sh) * PWp + pw * g.sw;
            for (int ci = 0; ci < cc; ci++) {
                const float *prow = pbase + ci * PH * PWp;
                const float4 *wrow = (const float4 *)(wsm + ci * KK * CO_T);
                for (int kh = 0; kh < g.Hk; kh++) {
                    for (int kw = 0; kw < g.Wk; kw++) {
                        float xv = prow[kh * PWp + kw];
                        const float4 *w4 = wrow + (kh * g.Wk + kw) * (CO_T / 4);
#pragma unroll
                        for (int q = 0; q < CO_T / 4; q++) {
                            float4 wv = w4[q];
                            acc[4 * q + 0] = fmaf(xv, wv.x, acc[4 * q + 0]);
                            acc[4 * q + 1] = fmaf(xv, wv.y, acc[4 * q + 1]);
                            acc[4 * q + 2] = fmaf(xv, wv.z, acc[4 * q + 2]);
                            acc[4 * q + 3] = fmaf(xv, wv.w, acc[4 * q + 3]);
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
    if (active) {
        const long long out_plane = (long long)g.Hout * g.Wout;
        T *yp = y + ((long long)(s0 + sl) * g.Cout + co0) * out_plane + (long long)(th0 + ph) * g.Wout + tw0 + pw;
#pragma unroll
        for (int c = 0; c < CO_T; c++) {
            if (co0 + c < g.Cout) {
                float v = acc[c];
                if (bias) v += ld(bias + co0 + c);
                st(yp + c * out_plane, v);
            }
        }
    }
}

// Depthwise forward / weight grad / input grad: one filter per channel
// [ref: lib/sources/pulp_conv_naive_fp32.c:29,113,153].
template <class T>
__global__ void dw_fw_kernel(ConvGeom g, const T *__restrict__ x, const T *__restrict__ w, T *__restrict__ y)
{
    long long total = (long long)g.n * g.Cin * g.Hout * g.Wout;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        int wo = e % g.Wout, ho = (e / g.Wout) % g.Hout;
        long long sc = e / ((long long)g.Wout * g.Hout);        // stream*C + ch
        int ch = sc % g.Cin;
        const T *xp = x + sc * g.Hin * g.Win;
        const T *wp = w + (long long)ch * g.Hk * g.Wk;
        float acc = 0.f;
        for (int kh = 0; kh < g.Hk; kh++) {
            int hi = ho * g.sh + kh - g.padU;
            if (hi < 0 || hi >= g.Hin) continue;
            for (int kw = 0; kw < g.Wk; kw++) {
                int wi = wo * g.sw + kw - g.padL;
                if (wi < 0 || wi >= g.Win) continue;
                acc = fmaf(ld(wp + kh * g.Wk + kw), ld(xp + hi * g.Win + wi), acc);
            }
        }
        st(y + e, acc);
    }
}

template <class T>
__global__ void dw_ig_kernel(ConvGeom g, const T *__restrict__ dy, const T *__restrict__ w, T *__restrict__ dx)
{
    long long total = (long long)g.n * g.Cin * g.Hin * g.Win;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        int wi = e % g.Win, hi = (e / g.Win) % g.Hin;
        long long sc = e / ((long long)g.Win * g.Hin);
        int ch = sc % g.Cin;
        const T *dyp = dy + sc * g.Hout * g.Wout;
        const T *wp = w + (long long)ch * g.Hk * g.Wk;
        float acc = 0.f;
        for (int kh = 0; kh < g.Hk; kh++) {
            int t = hi + g.padU - kh;
            if (t < 0 || t % g.sh) continue;
            int ho = t / g.sh;
            if (ho >= g.Hout) continue;
            for (int kw = 0; kw < g.Wk; kw++) {
                int u = wi + g.padL - kw;
                if (u < 0 || u % g.sw) continue;
                int wo = u / g.sw;
                if (wo >= g.Wout) continue;
                acc = fmaf(ld(wp + kh * g.Wk + kw), ld(dyp + ho * g.Wout + wo), acc);
            }
        }
        st(dx + e, acc);
    }
}

// One CTA per (channel, tap): block-wide sum over streams and output pixels.
template <class T>
__global__ void __launch_bounds__(256) dw_wg_kernel(ConvGeom g, const T *__restrict__ x, const T *__restrict__ dy, T *__restrict__ dw)
{
    __shared__ float red[256];
    const int tap = blockIdx.x % (g.Hk * g.Wk), ch = blockIdx.x / (g.Hk * g.Wk);
    const int kh = tap / g.Wk, kw = tap % g.Wk;
    const long long per = (long long)g.Hout * g.Wout, total = per * g.n;
    float acc = 0.f;
    for (long long e = threadIdx.x; e < total; e += blockDim.x) {
        int s = e / per, p = e % per, ho = p / g.Wout, wo = p % g.Wout;
        int hi = ho * g.sh + kh - g.padU, wi = wo * g.sw + kw - g.padL;
        if (hi < 0 || hi >= g.Hin || wi < 0 || wi >= g.Win) continue;
        acc = fmaf(ld(x + (((long long)s * g.Cin + ch) * g.Hin + hi) * g.Win + wi),
                   ld(dy + ((long long)s * g.Cin + ch) * per + p), acc);
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o]; __syncthreads(); }
    if (threadIdx.x == 0) st(dw + blockIdx.x, red[0]);
}

static bool conv_fw_plan(const ConvGeom &g, int &TH, int &TW, int &S_T, int &CC, size_t &smem)
{
    TW = g.Wout >= 32 ? 32 : (g.Wout >= 16 ? 16 : (g.Wout >= 8 ? 8 : (g.Wout >= 4 ? 4 : (g.Wout >= 2 ? 2 : 1))));
    TH = CONV_THREADS / TW;
    while (TH / 2 >= g.Hout && TH > 1) TH /= 2;
    S_T = CONV_THREADS / (TH * TW);
    if (S_T > g.n) S_T = g.n;
    if (S_T < 1) S_T = 1;
    const int PH = (TH - 1) * g.sh + g.Hk, PW = ((TW - 1) * g.sw + g.Wk) | 1, KK = g.Hk * g.Wk;
    CC = g.Cin;
    for (;;) {
        smem = ((((size_t)S_T * CC * PH * PW + 3) & ~(size_t)3) + (size_t)CC * KK * CO_T) * sizeof(float);
        if (smem <= 40 * 1024 || CC == 1) break;
        CC = (CC + 1) / 2;
    }
    return smem <= 200 * 1024;
}

template <class T> static bool try_tc_fw(Scope &, const ConvGeom &, const T *, const T *, const T *, T *) { return false; }
template <> bool try_tc_fw<float>(Scope &sc, const ConvGeom &g, const float *x, const float *w, const float *bias, float *y)
{
    if (conv1x1s_fw(g, x, w, bias, y)) return true;          // strided 1x1: memory-bound, CUDA cores
    return conv_tc_run(sc, x, w, bias, y, g.n, g.Cin, g.Hin, g.Win, g.Cout, g.Hout, g.Wout, g.Hk, g.Wk, g.sh, g.sw, g.padU, g.padL, g.Cout, g.Cin, false);
}
// dY of a strided convolution spread onto the input grid: dil[s][co][h][w] = dY[s][co][h/sh][w/sw] where both
// divisions are exact and in range, 0 elsewhere.  One thread writes four consecutive columns (Win % 4 == 0).
__global__ void __launch_bounds__(256) conv_dilate_dy_kernel(const float *__restrict__ dy, float *__restrict__ dil, unsigned total4,
                                                            int Hout, int Wout, int Hin, int Win, int sh, int sw)
{
    // 32-bit index arithmetic throughout (the host checks the element count)
    const unsigned W4 = (unsigned)Win / 4u;
    for (unsigned e = blockIdx.x * blockDim.x + threadIdx.x; e < total4; e += gridDim.x * blockDim.x) {
        const unsigned w4 = e % W4, row = e / W4;       // row = plane * Hin + h
        const unsigned h = row % (unsigned)Hin, pl = row / (unsigned)Hin;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        const unsigned ho = h / (unsigned)sh;
        if (ho * (unsigned)sh == h && ho < (unsigned)Hout) {
            const float *src = dy + ((size_t)pl * Hout + ho) * Wout;
            if (sw == 2) {
                const unsigned wo = 2u * w4;            // columns 4*w4 and 4*w4 + 2 carry samples wo and wo + 1
                if (wo < (unsigned)Wout) v.x = __ldg(src + wo);
                if (wo + 1 < (unsigned)Wout) v.z = __ldg(src + wo + 1);
            } else {
                float t[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const unsigned w = 4u * w4 + j, wo = w / (unsigned)sw;
                    if (wo * (unsigned)sw == w && wo < (unsigned)Wout) t[j] = __ldg(src + wo);
                }
                v = make_float4(t[0], t[1], t[2], t[3]);
            }
        }
        *reinterpret_cast<float4 *>(dil + (size_t)e * 4) = v;
    }
}

// Input gradient of a 1x1 convolution with stride s and no padding: dX[ci][h*s][w*s] = sum_co W[co][ci] dY[co][h][w],
// zero at every other position.  One CTA per (stream, tile of dY pixels): the weights and the dY tile sit in shared
// memory, a thread owns one pixel and walks the input channels, four at a time.  dX is zeroed by a kernel of its own
// first; with ACC the samples are added to what dX holds instead (a gradient that another branch already wrote there),
// and the positions between the samples are not touched at all.
template <int PX, bool ACC>
__global__ void __launch_bounds__(PX) conv1x1_strided_ig_kernel(ConvGeom g, const float *__restrict__ dy, const float *__restrict__ w, float *__restrict__ dx)
{
    extern __shared__ __align__(16) float sm1[];
    float *ws = sm1;                                 // [Cout][Cin]
    float *dys = sm1 + g.Cout * g.Cin;               // [Cout][PX]
    const int opix = g.Hout * g.Wout, tiles = (opix + PX - 1) / PX;
    const int s = blockIdx.x / tiles, p0 = (blockIdx.x % tiles) * PX;
    for (int e = threadIdx.x; e < g.Cout * g.Cin; e += PX) ws[e] = w[e];
    const float *dyp = dy + (size_t)s * g.Cout * opix;
    for (int e = threadIdx.x; e < g.Cout * PX; e += PX) {
        const int co = e / PX, p = e % PX;
        dys[e] = (p0 + p < opix) ? dyp[(size_t)co * opix + p0 + p] : 0.f;
    }
    __syncthreads();
    const int p = p0 + threadIdx.x;
    const bool live = p < opix;
    const int ho = live ? p / g.Wout : 0, wo = live ? p % g.Wout : 0;
    float *dxs = dx + (size_t)s * g.Cin * g.Hin * g.Win;
    if ((g.Cin & 3) == 0 && ((g.Cout * g.Cin) & 3) == 0) {
        // four input channels per pass: one shared load of dY and one 16-byte broadcast load of weights per 4 FMAs
        for (int ci = 0; ci < g.Cin; ci += 4) {
            float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll 4
            for (int co = 0; co < g.Cout; co++) {
                const float d = dys[co * PX + threadIdx.x];
                const float4 wv = *reinterpret_cast<const float4 *>(ws + co * g.Cin + ci);
                a0 = fmaf(wv.x, d, a0); a1 = fmaf(wv.y, d, a1); a2 = fmaf(wv.z, d, a2); a3 = fmaf(wv.w, d, a3);
            }
            if (live) {
                float *o = dxs + ((size_t)ci * g.Hin + (size_t)ho * g.sh) * g.Win + (size_t)wo * g.sw;
                const size_t pl = (size_t)g.Hin * g.Win;
                if (ACC) { o[0] = __fadd_rn(a0, o[0]); o[pl] = __fadd_rn(a1, o[pl]); o[2 * pl] = __fadd_rn(a2, o[2 * pl]); o[3 * pl] = __fadd_rn(a3, o[3 * pl]); }
                else { o[0] = a0; o[pl] = a1; o[2 * pl] = a2; o[3 * pl] = a3; }
            }
        }
        return;
    }
    for (int ci = 0; ci < g.Cin; ci++) {
        float acc = 0.f;
        for (int co = 0; co < g.Cout; co++) acc = fmaf(ws[co * g.Cin + ci], dys[co * PX + threadIdx.x], acc);
        if (live) {
            float *o = dxs + ((size_t)ci * g.Hin + (size_t)ho * g.sh) * g.Win + (size_t)wo * g.sw;
            *o = ACC ? __fadd_rn(acc, *o) : acc;
        }
    }
}
// zero fill of dX before the scattered samples are written (16-byte stores)
__global__ void __launch_bounds__(256) zero_f4_kernel(float4 *__restrict__ p, size_t n4)
{
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n4; e += (size_t)gridDim.x * blockDim.x) p[e] = make_float4(0.f, 0.f, 0.f, 0.f);
}

// 1x1, strided, unpadded: a small per-pixel matrix product scattered onto a zeroed dX (or added into dX); bandwidth-bound,
// no tensor cores.  False when the geometry or the path selection rules it out.
static bool try_conv1x1_ig(const ConvGeom &g, const float *dy, const float *w, float *dx, bool acc)
{
    if (acc && conv1x1s_ig(g, dy, w, dx)) return true;    // added in place: nothing to zero first
    if (!(g.Hk == 1 && g.Wk == 1 && g.padU == 0 && g.padL == 0 && !g.depthwise && gemm_path() != 1 && (((uintptr_t)dx) & 15) == 0 && (g.Hin * g.Win) % 4 == 0 &&
          (g.sh > 1 || g.sw > 1) && (long long)(g.Hout - 1) * g.sh < g.Hin && (long long)(g.Wout - 1) * g.sw < g.Win))
        return false;
    const int opix = g.Hout * g.Wout, PX = opix >= 256 ? 256 : 64;
    const size_t smem = ((size_t)g.Cout * g.Cin + (size_t)g.Cout * PX) * sizeof(float);
    if (smem > 160 * 1024) return false;
    if (!acc) {
        const size_t n4 = (size_t)g.n * g.Cin * g.Hin * g.Win / 4;
        TL_LAUNCH(zero_f4_kernel, (unsigned)std::min<size_t>((n4 + 255) / 256, (size_t)sm_count() * 32), 256, 0, reinterpret_cast<float4 *>(dx), n4);
    }
    const unsigned grid = (unsigned)g.n * (unsigned)((opix + PX - 1) / PX);
#define TL_1X1(PXV, ACCV)                                                                                              \
    do {                                                                                                               \
        if (smem > 48 * 1024) cudaFuncSetAttribute(conv1x1_strided_ig_kernel<PXV, ACCV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        TL_LAUNCH((conv1x1_strided_ig_kernel<PXV, ACCV>), grid, PXV, smem, g, dy, w, dx);                               \
    } while (0)
    if (PX == 256) { if (acc) TL_1X1(256, true); else TL_1X1(256, false); }
    else { if (acc) TL_1X1(64, true); else TL_1X1(64, false); }
#undef TL_1X1
    profile_add_flops(conv_flops(g));
    return true;
}
template <class T> static bool try_conv1x1_ig(const ConvGeom &, const T *, const T *, T *, bool) { return false; }
template <class T> static bool try_tc_ig(Scope &, const ConvGeom &, const T *, const T *, T *) { return false; }
template <> bool try_tc_ig<float>(Scope &sc, const ConvGeom &g, const float *dy, const float *w, float *dx)
{
    // dX is a stride-1 convolution of dY with the rotated filters and padding k-1-pad
    if (g.Hk - 1 - g.padU < 0 || g.Wk - 1 - g.padL < 0) return false;
    if (g.sh == 1 && g.sw == 1)
        return conv_tc_run(sc, dy, w, (const float *)nullptr, dx, g.n, g.Cout, g.Hout, g.Wout, g.Cin, g.Hin, g.Win, g.Hk, g.Wk, 1, 1,
                           g.Hk - 1 - g.padU, g.Wk - 1 - g.padL, g.Cout, g.Cin, true);
    if (try_conv1x1_ig(g, dy, w, dx, false)) return true;
    // strided, general filter: one launch per parity class of dX.  Pixels (sh*i + ph, sw*j + pw) only see the filter taps
    // kh = r + sh*m with r = (ph + padU) mod sh, and those taps read dY rows i + q - m with q = (ph + padU) / sh: a dense
    // stride-1 convolution of dY with an (m_max+1)-row window, written to every sh-th row of dX.  No zeros are multiplied.
    if (g.sh == 2 && g.sw == 2 && g.Hk == 3 && g.Wk == 3 && g.padU == 1 && g.padL == 1 && g.Win == 2 * g.Wout && g.Hin == 2 * g.Hout && gemm_path() != 1) {
        // 3x3, pad 1, stride 2: one launch per ROW parity, both column parities together (pixel pairs, contiguous output rows)
        ConvTcClass cls[2];
        int Ah[2], pu[2];
        for (int ph = 0; ph < 2; ph++) {
            const int rh = (ph + 1) % 2, qh = (ph + 1) / 2, mh = (2 - rh) / 2;
            ConvTcClass &c = cls[ph];
            c.kstep = 2; c.kh_r = rh; c.kh_m = mh; c.kw_r = 0; c.kw_m = 0; c.w_Hk = 3; c.w_Wk = 3;
            c.oH = g.Hin; c.oW = g.Win; c.osy = 2; c.osx = 2; c.oy0 = ph; c.ox0 = 0; c.up = 1;
            Ah[ph] = mh + 1; pu[ph] = mh - qh;
        }
        bool ok = true;
        for (int ph = 0; ph < 2 && ok; ph++)
            ok = pu[ph] >= 0 && conv_tc_run(sc, dy, w, (const float *)nullptr, dx, g.n, g.Cout, g.Hout, g.Wout, g.Cin, g.Hout, g.Wout, Ah[ph], 3, 1, 1,
                                            pu[ph], 1, g.Cout, g.Cin, true, true, &cls[ph]);
        if (ok) {
            for (int ph = 0; ph < 2; ph++)
                if (!conv_tc_run(sc, dy, w, (const float *)nullptr, dx, g.n, g.Cout, g.Hout, g.Wout, g.Cin, g.Hout, g.Wout, Ah[ph], 3, 1, 1,
                                 pu[ph], 1, g.Cout, g.Cin, true, false, &cls[ph]))
                    return false;
            return true;
        }
    }
    if (g.sh == g.sw && g.sh >= 2 && g.sh <= 4 && gemm_path() != 1) {
        ConvTcClass cls[16];
        int Hc[16], Wc[16], Ah[16], Aw[16], pu[16], pl[16], ncls = 0;
        bool ok = true;
        for (int ph = 0; ph < g.sh && ok; ph++)
            for (int pw = 0; pw < g.sw && ok; pw++) {
                const int rh = (ph + g.padU) % g.sh, qh = (ph + g.padU) / g.sh, rw = (pw + g.padL) % g.sw, qw = (pw + g.padL) / g.sw;
                if (rh >= g.Hk || rw >= g.Wk || ph >= g.Hin || pw >= g.Win) { ok = false; break; }
                const int mh = (g.Hk - 1 - rh) / g.sh, mw = (g.Wk - 1 - rw) / g.sw;
                if (mh - qh < 0 || mw - qw < 0) { ok = false; break; }
                ConvTcClass &c = cls[ncls];
                c.kstep = g.sh; c.kh_r = rh; c.kh_m = mh; c.kw_r = rw; c.kw_m = mw; c.w_Hk = g.Hk; c.w_Wk = g.Wk;
                c.oH = g.Hin; c.oW = g.Win; c.osy = g.sh; c.osx = g.sw; c.oy0 = ph; c.ox0 = pw; c.up = 0;
                Hc[ncls] = (g.Hin - ph + g.sh - 1) / g.sh; Wc[ncls] = (g.Win - pw + g.sw - 1) / g.sw;
                Ah[ncls] = mh + 1; Aw[ncls] = mw + 1; pu[ncls] = mh - qh; pl[ncls] = mw - qw;
                ok = conv_tc_run(sc, dy, w, (const float *)nullptr, dx, g.n, g.Cout, g.Hout, g.Wout, g.Cin, Hc[ncls], Wc[ncls], Ah[ncls], Aw[ncls], 1, 1,
                                 pu[ncls], pl[ncls], g.Cout, g.Cin, true, true, &c);
                ncls++;
            }
        if (ok) {
            for (int i = 0; i < ncls; i++)
                if (!conv_tc_run(sc, dy, w, (const float *)nullptr, dx, g.n, g.Cout, g.Hout, g.Wout, g.Cin, Hc[i], Wc[i], Ah[i], Aw[i], 1, 1, pu[i], pl[i],
                                 g.Cout, g.Cin, true, false, &cls[i]))
                    return false;       // (cannot happen after the dry runs; the FFMA kernel then recomputes all of dX)
            return true;
        }
    }
    // otherwise: spread dY onto the input grid (zeros between the samples), then the same stride-1 convolution.
    // The tensor cores do sh*sw times the useful work, which still beats the FFMA kernel by a wide margin.
    if (g.Win % 4 != 0 || (long long)(g.Hout - 1) * g.sh >= g.Hin || (long long)(g.Wout - 1) * g.sw >= g.Win) return false;
    if (!conv_tc_run(sc, nullptr, w, (const float *)nullptr, dx, g.n, g.Cout, g.Hin, g.Win, g.Cin, g.Hin, g.Win, g.Hk, g.Wk, 1, 1,
                     g.Hk - 1 - g.padU, g.Wk - 1 - g.padL, g.Cout, g.Cin, true, true))
        return false;
    const long long planes = (long long)g.n * g.Cout;
    const long long total = planes * g.Hin * (g.Win / 4);
    if (total >= (1ll << 31)) return false;
    float *dil = sc.scratch<float>((size_t)planes * g.Hin * g.Win);
    if (!dil) return false;
    const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 32);
    TL_LAUNCH(conv_dilate_dy_kernel, blocks, 256, 0, dy, dil, (unsigned)total, g.Hout, g.Wout, g.Hin, g.Win, g.sh, g.sw);
    const bool ok = conv_tc_run(sc, dil, w, (const float *)nullptr, dx, g.n, g.Cout, g.Hin, g.Win, g.Cin, g.Hin, g.Win, g.Hk, g.Wk, 1, 1,
                                g.Hk - 1 - g.padU, g.Wk - 1 - g.padL, g.Cout, g.Cin, true);
    if (ok) profile_add_flops(conv_flops(g) - 2.0 * g.n * g.Cin * g.Cout * g.Hk * g.Wk * g.Hin * g.Win);   // the zeros between the samples are not work
    return ok;
}

template <class T> void conv_fw(Scope &sc, const ConvGeom &g, const T *x, const T *w, const T *bias, T *y)
{
    if (!g.depthwise && try_tc_fw<T>(sc, g, x, w, bias, y)) return;
    if (g.depthwise) {
        long long total = (long long)g.n * g.Cin * g.Hout * g.Wout;
        int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 16);
        TL_LAUNCH((dw_fw_kernel<T>), blocks, 256, 0, g, x, w, y);
        return;
    }
    int TH, TW, S_T, CC; size_t smem;
    if (!conv_fw_plan(g, TH, TW, S_T, CC, smem)) { set_error(TL_ERR_TOO_LARGE, "conv forward: kernel window too large for shared memory"); return; }
    if (smem > 48 * 1024) cudaFuncSetAttribute(conv_fw_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int tiles_w = ceil_div(g.Wout, TW), tiles_h = ceil_div(g.Hout, TH), tiles_s = ceil_div(g.n, S_T);
    dim3 grid(tiles_w * tiles_h * tiles_s, ceil_div(g.Cout, CO_T));
    TL_LAUNCH((conv_fw_kernel<T>), grid, CONV_THREADS, smem, g, x, w, bias, y, TH, TW, S_T, CC, tiles_w, tiles_h);
    profile_add_flops(conv_flops(g));
}

// ------------------------------------------------------------------ input gradient
// dX[ci][hi][wi] = sum_{co,kh,kw} W[co][ci][kh][kw] * dY[co][(hi+padU-kh)/sh][(wi+padL-kw)/sw]
// over the taps where both divisions are exact and in range.  Same tiling as the forward with
// the roles of the channel dimensions swapped; CI_T = 16 input channels per thread.
template <class T>
__global__ void __launch_bounds__(CONV_THREADS)
conv_ig_kernel(ConvGeom g, const T *__restrict__ dy, const T *__restrict__ w, T *__restrict__ dx,
               int TH, int TW, int S_T, int CC, int tiles_w, int tiles_h, int PH, int PW)
{
    extern __shared__ __align__(16) float smem[];
    const int PWp = PW | 1;
    const int KK = g.Hk * g.Wk;
    float *patch = smem;                                     // [S_T][CC][PH][PWp] of dY
    float *wsm = smem + (((size_t)S_T * CC * PH * PWp + 3) & ~(size_t)3);   // [CC(co)][KK][CO_T(ci)], 16-byte aligned

    const int tid = threadIdx.x;
    const int tile = blockIdx.x;
    const int tw0 = (tile % tiles_w) * TW, th0 = ((tile / tiles_w) % tiles_h) * TH;
    const int s0 = (tile / (tiles_w * tiles_h)) * S_T;
    const int ci0 = blockIdx.y * CO_T;

    const int pix = tid % (TH * TW), sl = tid / (TH * TW);
    const int ph = pix / TW, pw = pix % TW;
    const int hi = th0 + ph, wi = tw0 + pw;
    const bool active = (sl < S_T) && (s0 + sl < g.n) && (hi < g.Hin) && (wi < g.Win);

    // first output row/col that any pixel of the tile can touch (floor division, may be negative)
    const int t_lo = th0 + g.padU - (g.Hk - 1), u_lo = tw0 + g.padL - (g.Wk - 1);
    const int ho_base = (t_lo >= 0) ? t_lo / g.sh : -((-t_lo + g.sh - 1) / g.sh);
    const int wo_base = (u_lo >= 0) ? u_lo / g.sw : -((-u_lo + g.sw - 1) / g.sw);

    float acc[CO_T];
#pragma unroll
    for (int c = 0; c < CO_T; c++) acc[c] = 0.f;
    const long long out_plane = (long long)g.Hout * g.Wout;

    for (int co0 = 0; co0 < g.Cout; co0 += CC) {
        const int cc = min(CC, g.Cout - co0);
        const int patch_elems = S_T * cc * PH * PW;
        for (int e = tid; e < patch_elems; e += CONV_THREADS) {
            int c = e % PW, r = (e / PW) % PH, co = (e / (PW * PH)) % cc, s = e / (PW * PH * cc);
            int ho = ho_base + r, wo = wo_base + c;
            float v = 0.f;
            if (s0 + s < g.n && ho >= 0 && ho < g.Hout && wo >= 0 && wo < g.Wout)
                v = ld(dy + ((long long)(s0 + s) * g.Cout + co0 + co) * out_plane + (long long)ho * g.Wout + wo);
            patch[((s * CC + co) * PH + r) * PWp + c] = v;
        }
        const int w_elems = cc * KK * CO_T;
        for (int e = tid; e < w_elems; e += CONV_THREADS) {
            int ci = e % CO_T, t = (e / CO_T) % KK, co = e / (CO_T * KK);
            float v = 0.f;
            if (ci0 + ci < g.Cin) v = ld(w + ((long long)(co0 + co) * g.Cin + ci0 + ci) * KK + t);
            wsm[(co * KK + t) * CO_T + ci] = v;
        }
        __syncthreads();
        if (active) {
            for (int kh = 0; kh < g.Hk; kh++) {
                int t = hi + g.padU - kh;
                if (t < 0 || (t % g.sh) != 0) continue;
                int r = t / g.sh - ho_base;
                if (r < 0 || r >= PH) continue;
                for (int kw = 0; kw < g.Wk; kw++) {
                    int u = wi + g.padL - kw;
                    if (u < 0 || (u % g.sw) != 0) continue;
                    int c = u / g.sw - wo_base;
                    if (c < 0 || c >= PW) continue;
                    const float *pp = patch + ((sl * CC) * PH + r) * PWp + c;
                    const float4 *w4 = (const float4 *)(wsm + (kh * g.Wk + kw) * CO_T);
                    for (int co = 0; co < cc; co++) {
                        float dv = pp[co * PH * PWp];
                        const float4 *wq = w4 + co * KK * (CO_T / 4);
#pragma unroll
                        for (int q = 0; q < CO_T / 4; q++) {
                            float4 wv = wq[q];
                            acc[4 * q + 0] = fmaf(dv, wv.x, acc[4 * q + 0]);
                            acc[4 * q + 1] = fmaf(dv, wv.y, acc[4 * q + 1]);
                            acc[4 * q + 2] = fmaf(dv, wv.z, acc[4 * q + 2]);
                            acc[4 * q + 3] = fmaf(dv, wv.w, acc[4 * q + 3]);
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
    if (active) {
        const long long in_plane = (long long)g.Hin * g.Win;
        T *xp = dx + ((long long)(s0 + sl) * g.Cin + ci0) * in_plane + (long long)hi * g.Win + wi;
#pragma unroll
        for (int c = 0; c < CO_T; c++)
            if (ci0 + c < g.Cin) st(xp + c * in_plane, acc[c]);
    }
}

// dX += input gradient: in place where a kernel can add (1x1 strided), otherwise through scratch and one sum
template <class T> void conv_ig_accumulate(Scope &sc, const ConvGeom &g, const T *dy, const T *w, T *dx)
{
    if (try_conv1x1_ig(g, dy, w, dx, true)) return;
    const size_t nx = (size_t)g.n * g.Cin * g.Hin * g.Win;
    T *tmp = sc.scratch<T>(nx);
    if (!tmp) return;
    conv_ig<T>(sc, g, dy, w, tmp);
    add<T>(tmp, dx, dx, (long long)nx);
}
template <class T> void conv_ig(Scope &sc, const ConvGeom &g, const T *dy, const T *w, T *dx)
{
    if (!g.depthwise && try_tc_ig<T>(sc, g, dy, w, dx)) return;
    if (g.depthwise) {
        long long total = (long long)g.n * g.Cin * g.Hin * g.Win;
        int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 16);
        TL_LAUNCH((dw_ig_kernel<T>), blocks, 256, 0, g, dy, w, dx);
        return;
    }
    int TW = g.Win >= 32 ? 32 : (g.Win >= 16 ? 16 : (g.Win >= 8 ? 8 : (g.Win >= 4 ? 4 : (g.Win >= 2 ? 2 : 1))));
    int TH = CONV_THREADS / TW;
    while (TH / 2 >= g.Hin && TH > 1) TH /= 2;
    int S_T = CONV_THREADS / (TH * TW);
    if (S_T > g.n) S_T = g.n;
    if (S_T < 1) S_T = 1;
    const int PH = (TH - 1 + g.Hk - 1) / g.sh + 2, PW = (TW - 1 + g.Wk - 1) / g.sw + 2;
    const int KK = g.Hk * g.Wk;
    int CC = g.Cout; size_t smem;
    for (;;) {
        smem = ((((size_t)S_T * CC * PH * (PW | 1) + 3) & ~(size_t)3) + (size_t)CC * KK * CO_T) * sizeof(float);
        if (smem <= 40 * 1024 || CC == 1) break;
        CC = (CC + 1) / 2;
    }
    if (smem > 200 * 1024) { set_error(TL_ERR_TOO_LARGE, "conv input grad: kernel window too large for shared memory"); return; }
    if (smem > 48 * 1024) cudaFuncSetAttribute(conv_ig_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    int tiles_w = ceil_div(g.Win, TW), tiles_h = ceil_div(g.Hin, TH), tiles_s = ceil_div(g.n, S_T);
    dim3 grid(tiles_w * tiles_h * tiles_s, ceil_div(g.Cin, CO_T));
    TL_LAUNCH((conv_ig_kernel<T>), grid, CONV_THREADS, smem, g, dy, w, dx, TH, TW, S_T, CC, tiles_w, tiles_h, PH, PW);
    profile_add_flops(conv_flops(g));
}

// ------------------------------------------------------------------ weight gradient
// dW[co][ci][kh][kw] = sum over streams and output pixels of dY[co][ho][wo] * X[ci][ho*sh+kh-padU][wo*sw+kw-padL].
// The reduction dimension (streams x pixels) is split over `groups` CTAs per 16x16 (co,ci) tile.
// Thread (co,ci) keeps the Hk*Wk taps of its filter in registers while its CTA walks its share of
// (stream, pixel-tile) work items in ascending order; CTA partials go to scratch
// [group][Cout*Cin*KK] and a second kernel adds them in group order, so the result does not
// depend on scheduling (no atomics).
template <class T, int KH, int KW>
__global__ void __launch_bounds__(CONV_THREADS)
conv_wg_partial_kernel(ConvGeom g, const T *__restrict__ x, const T *__restrict__ dy, float *__restrict__ part,
                       int TH, int TW, int tiles_w, int tiles_h, int ci_tiles)
{
    extern __shared__ __align__(16) float smem[];
    const int PH = (TH - 1) * g.sh + g.Hk, PW = (TW - 1) * g.sw + g.Wk;
    const int PWp = PW | 1;
    const int PLANE = (PH * PWp) | 1;
    const int TP = TH * TW;
    float *xs = smem;                          // [16 ci][PLANE]
    float *dys = smem + 16 * PLANE;            // [16 co][TP + 1]
    constexpr int KK = KH * KW;

    const int tid = threadIdx.x;
    const int co_l = tid / 16, ci_l = tid % 16;
    const int ci0 = (blockIdx.x % ci_tiles) * 16, co0 = (blockIdx.x / ci_tiles) * 16;
    const int group = blockIdx.y, groups = gridDim.y;

    float acc[KK];
#pragma unroll
    for (int t = 0; t < KK; t++) acc[t] = 0.f;

    const long long in_plane = (long long)g.Hin * g.Win, out_plane = (long long)g.Hout * g.Wout;
    const long long items = (long long)g.n * tiles_h * tiles_w;
    // contiguous share of the work list, so partial sums follow stream order
    const long long per = (items + groups - 1) / groups;
    const long long it_begin = (long long)group * per, it_end = min(items, it_begin + per);

    for (long long it = it_begin; it < it_end; it++) {
        const int s = (int)(it / (tiles_h * tiles_w));
        const int trem = (int)(it % (tiles_h * tiles_w));
        const int th0 = (trem / tiles_w) * TH, tw0 = (trem % tiles_w) * TW;
        const int h_in0 = th0 * g.sh - g.padU, w_in0 = tw0 * g.sw - g.padL;
        for (int e = tid; e < 16 * PH * PW; e += CONV_THREADS) {
            int c = e % PW, r = (e / PW) % PH, ci = e / (PW * PH);
            int hi = h_in0 + r, wi = w_in0 + c;
            float v = 0.f;
            if (ci0 + ci < g.Cin && hi >= 0 && hi < g.Hin && wi >= 0 && wi < g.Win)
                v = ld(x + ((long long)s * g.Cin + ci0 + ci) * in_plane + (long long)hi * g.Win + wi);
            xs[ci * PLANE + r * PWp + c] = v;
        }
        for (int e = tid; e < 16 * TP; e += CONV_THREADS) {
            int p = e % TP, co = e / TP;
            int ho = th0 + p / TW, wo = tw0 + p % TW;
            float v = 0.f;
            if (co0 + co < g.Cout && ho < g.Hout && wo < g.Wout)
                v = ld(dy + ((long long)s * g.Cout + co0 + co) * out_plane + (long long)ho * g.Wout + wo);
            dys[co * (TP + 1) + p] = v;
        }
        __syncthreads();
        const float *xc = xs + ci_l * PLANE;
        const float *dc = dys + co_l * (TP + 1);
        for (int ph = 0; ph < TH; ph++) {
            for (int pw = 0; pw < TW; pw++) {
                float d = dc[ph * TW + pw];
                const float *xp = xc + (ph * g.sh) * PWp + pw * g.sw;
#pragma unroll
                for (int kh = 0; kh < KH; kh++)
#pragma unroll
                    for (int kw = 0; kw < KW; kw++) acc[kh * KW + kw] = fmaf(d, xp[kh * PWp + kw], acc[kh * KW + kw]);
            }
        }
        __syncthreads();
    }
    if (co0 + co_l < g.Cout && ci0 + ci_l < g.Cin) {
        float *pp = part + (long long)group * g.Cout * g.Cin * KK + ((long long)(co0 + co_l) * g.Cin + ci0 + ci_l) * KK;
#pragma unroll
        for (int t = 0; t < KK; t++) pp[t] = acc[t];
    }
}

// Weight gradient of a 3x3 filter with left padding 1 (K = 3) or a 1x1 filter without padding (K = 1), register-tiled.  One warp covers the whole 16 (co) x 16 (ci) channel tile:
// lane = (co block of 4) x (ci pair {b, b+8}), so a thread owns 4 x 2 x K*K accumulators (72 for 3x3).  The 8 warps of a CTA
// each take rows of the pixel tile, whose width TW is the whole output row.  Shared memory holds input rows as
// [4 zero columns][Win values][4 zero columns] (16-byte aligned, filled with 16-byte copies) and dY rows contiguously,
// so four output pixels cost 4 + 6 (stride 1) or 4 + 12 (stride 2) 16-byte shared loads for 288 FMAs.  The plane
// stride is 4 x odd floats: the 8 ci pairs of a quarter warp then touch all 32 banks exactly once per 16-byte load.
// At the end the warps add their accumulators into shared memory in warp order and the CTA writes one partial.
// TH (rows per item) and S_T (streams per item) are template parameters as well, so every shared-memory offset in
// the inner loop is an immediate.
template <int S, int TW, int K, int TH, int S_T> struct WgShape {
    static constexpr int WIN = S * TW;             // input row width (host guarantees g.Win == WIN)
    static constexpr int RW = WIN + 8;             // shared-memory row: input column w sits at 4 + w
    static constexpr int W4 = WIN / 4;
    static constexpr int KK = K * K, VOFF = (K == 1) ? 1 : 0;   // v[] starts one column left of the first input column
    static constexpr int PH = (TH - 1) * S + K;
    static constexpr int PLANE = 4 * ((PH * RW / 4) | 1);
    static constexpr int TP = TH * TW, DYP = S_T * TP + 4, TP4 = TP / 4;
    static constexpr int STAGE = S_T * 16 * PLANE + 16 * DYP;
};
// SMALL = at most 4 input channels (a network's first layer): the 8 lanes that would hold ci pairs hold 2 pairs x 4
// interleaved slices of the pixel row instead, and the four slice sums are added with shuffles before the cross-warp sum.
template <class T, int S, int TW, int K, int TH, int S_T, bool SMALL = false>
__global__ void __launch_bounds__(CONV_THREADS, 2)
conv_wg3x3_partial_kernel(ConvGeom g, const T *__restrict__ x, const T *__restrict__ dy, float *__restrict__ part,
                          int tiles_h, int ci_tiles, int vec, int nstage)
{
    extern __shared__ __align__(16) float smem[];
    typedef WgShape<S, TW, K, TH, S_T> WS;
    constexpr int WIN = WS::WIN, RW = WS::RW, W4 = WS::W4, KK = WS::KK, VOFF = WS::VOFF, PH = WS::PH, PLANE = WS::PLANE;
    constexpr int TP = WS::TP, DYP = WS::DYP, STAGE = WS::STAGE;
    // nstage stages of {input patch [S_T][16 ci][PLANE], dY tile [16 co][DYP]}: the next items are fetched with
    // 16-byte asynchronous copies while the current one is consumed
    float *accs = smem;                             // [16 co][16 ci][KK] cross-warp sum, reuses stage 0 after the loop

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cob = lane >> 3, cib = SMALL ? (lane & 1) : (lane & 7), kphase = SMALL ? ((lane >> 1) & 3) : 0;
    constexpr int CI_STEP = SMALL ? 2 : 8, K_STEP = SMALL ? 4 : 1;      // second channel of a lane; stride of its 4-pixel groups
    const int ci0 = (blockIdx.x % ci_tiles) * 16, co0 = (blockIdx.x / ci_tiles) * 16;
    const int group = blockIdx.y, groups = gridDim.y;

    float acc[4][2][KK];
#pragma unroll
    for (int c = 0; c < 4; c++)
#pragma unroll
        for (int i = 0; i < 2; i++)
#pragma unroll
            for (int t = 0; t < KK; t++) acc[c][i][t] = 0.f;

    // the zero columns on both sides of every row are written once; staging only touches columns 4 .. 4 + WIN
    for (int e = tid; e < nstage * STAGE; e += CONV_THREADS) smem[e] = 0.f;
    __syncthreads();

    const long long in_plane = (long long)g.Hin * g.Win, out_plane = (long long)g.Hout * g.Wout;
    const int s_tiles = (g.n + S_T - 1) / S_T;
    const long long items = (long long)s_tiles * tiles_h;
    const long long per = (items + groups - 1) / groups;
    const long long it_begin = (long long)group * per, it_end = min(items, it_begin + per);

    // warp-per-plane staging: a warp takes (stream, channel) planes, its lanes the 16-byte pieces of the plane
    auto stage_item = [&](long long it, float *xs, float *dys) {
        const int it32 = (int)it;                  // the host keeps the item count below 2^31
        const int s0 = (it32 / tiles_h) * S_T;
        const int th0 = (it32 % tiles_h) * TH;
        const int h_in0 = th0 * S - g.padU;
        if (vec) {
            if constexpr (sizeof(T) == 4) {
                // every 16-byte piece of the item is one asynchronous copy; thread tid takes the pieces tid, tid + 256, ...  The
                // piece -> (plane, row, column) split has compile-time divisors and 32-bit offsets from the item's base address.
                constexpr int NGX = S_T * 16 * PH * W4, NGD = 16 * S_T * WS::TP4;
                const float *xit = x + ((long long)s0 * g.Cin + ci0) * in_plane + (long long)h_in0 * WIN;
                const unsigned xdst = (unsigned)__cvta_generic_to_shared(xs) + 16u;
#pragma unroll
                for (int k = 0; k < (NGX + CONV_THREADS - 1) / CONV_THREADS; k++) {
                    const int e = tid + k * CONV_THREADS;
                    if (NGX % CONV_THREADS != 0 && e >= NGX) break;
                    const int c4 = e % W4, prow = e / W4, r = prow % PH, pl = prow / PH;
                    const int ci = pl & 15, sl = pl >> 4;
                    if (SMALL && ci >= 4) continue;          // never read; still zero from the initial fill
                    if (K == 1 && S > 1 && r % S != 0) continue;    // a strided 1x1 filter never reads the rows between its samples
                    const bool ok = s0 + sl < g.n && ci0 + ci < g.Cin && (unsigned)(h_in0 + r) < (unsigned)g.Hin;
                    const int goff = (sl * g.Cin + ci) * (int)in_plane + r * WIN + 4 * c4;
                    const float *sp = ok ? xit + goff : x;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(xdst + (unsigned)(pl * PLANE + r * RW + 4 * c4) * 4u), "l"(sp), "r"(ok ? 16 : 0) : "memory");
                }
                const float *dit = dy + ((long long)s0 * g.Cout + co0) * out_plane + (long long)th0 * TW;
                const unsigned ddst = (unsigned)__cvta_generic_to_shared(dys);
#pragma unroll
                for (int k = 0; k < (NGD + CONV_THREADS - 1) / CONV_THREADS; k++) {
                    const int e = tid + k * CONV_THREADS;
                    if (NGD % CONV_THREADS != 0 && e >= NGD) break;
                    const int q = e % WS::TP4, sl = (e / WS::TP4) % S_T, co = e / (WS::TP4 * S_T);
                    const bool ok = s0 + sl < g.n && co0 + co < g.Cout && th0 + (4 * q) / TW < g.Hout;
                    const int goff = (sl * g.Cout + co) * (int)out_plane + 4 * q;
                    const float *sp = ok ? dit + goff : dy;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(ddst + (unsigned)(co * DYP + sl * TP + 4 * q) * 4u), "l"(sp), "r"(ok ? 16 : 0) : "memory");
                }
            }
        } else {
            for (int rr = warp; rr < S_T * 16 * PH; rr += CONV_THREADS / 32) {
                const int r = rr % PH, ci = (rr / PH) & 15, sl = rr / (PH * 16);
                const int hi = h_in0 + r;
                const bool ok = s0 + sl < g.n && ci0 + ci < g.Cin && hi >= 0 && hi < g.Hin;
                const T *src = x + ((long long)(s0 + sl) * g.Cin + ci0 + ci) * in_plane + (long long)hi * WIN;
                float *dst = xs + (sl * 16 + ci) * PLANE + r * RW + 4;
                for (int c = lane; c < WIN; c += 32) dst[c] = ok ? ld(src + c) : 0.f;
            }
            for (int rr = warp; rr < 16 * S_T * TH; rr += CONV_THREADS / 32) {
                const int ph = rr % TH, sl = (rr / TH) % S_T, co = rr / (TH * S_T);
                const bool ok = s0 + sl < g.n && co0 + co < g.Cout && th0 + ph < g.Hout;
                const T *src = dy + ((long long)(s0 + sl) * g.Cout + co0 + co) * out_plane + (long long)(th0 + ph) * TW;
                float *dst = dys + co * DYP + sl * TP + ph * TW;
                for (int c = lane; c < TW; c += 32) dst[c] = ok ? ld(src + c) : 0.f;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // nstage = 2 or 3 shared-memory stages: items it+1 .. it+nstage-1 are in flight while item it is consumed.
    // One commit group per loop step, empty once the items run out, so the group count stays in step.
    auto stage_or_skip = [&](long long it, int stg) {
        if (it < it_end) stage_item(it, smem + stg * STAGE, smem + stg * STAGE + S_T * 16 * PLANE);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    };
    for (int a = 0; a < nstage - 1; a++) stage_or_skip(it_begin + a, a);
    int cur = 0;
    for (long long it = it_begin; it < it_end; it++, cur = (cur + 1 == nstage) ? 0 : cur + 1) {
        if (nstage == 3) asm volatile("cp.async.wait_group 1;" ::: "memory");
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();        // this item has landed for every thread, and every thread is done with the stage refilled next
        const float *xs = smem + cur * STAGE, *dys = xs + S_T * 16 * PLANE;
        stage_or_skip(it + nstage - 1, (cur + nstage - 1) % nstage);
#pragma unroll
        for (int rr = 0; rr < (S_T * TH + CONV_THREADS / 32 - 1) / (CONV_THREADS / 32); rr++) {
            const int row = warp + rr * (CONV_THREADS / 32);
            if (row >= S_T * TH) break;
            const int sl = row / TH, ph = row % TH;
            const float *xb = xs + (sl * 16 + cib) * PLANE + (ph * S) * RW;        // ci = cib (i = 0), + 8 planes for i = 1
            const float *dp = dys + (cob * 4) * DYP + sl * TP + ph * TW;
#pragma unroll
            for (int k0 = 0; k0 < TW / 4; k0 += K_STEP) {
                const int k = k0 + kphase;
                float4 d[4];
#pragma unroll
                for (int c = 0; c < 4; c++) d[c] = *reinterpret_cast<const float4 *>(dp + c * DYP + 4 * k);
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int kh = 0; kh < K; kh++) {
                        const float *rp = xb + i * CI_STEP * PLANE + kh * RW;
                        // v[m] = shared column 3 + 4*S*k + m: pixel j of this group reads v[S*j + kw]
                        float v[4 * S + 2];
                        v[0] = rp[4 * S * k + 3];
                        const float4 a = *reinterpret_cast<const float4 *>(rp + 4 * S * k + 4);
                        v[1] = a.x; v[2] = a.y; v[3] = a.z; v[4] = a.w;
                        if (S == 1) {
                            v[5] = rp[4 * k + 8];
                        } else {
                            const float4 b = *reinterpret_cast<const float4 *>(rp + 8 * k + 8);
                            v[5] = b.x; v[6] = b.y; v[7] = b.z; v[8] = b.w; v[9] = 0.f;
                        }
#pragma unroll
                        for (int j = 0; j < 4; j++)
#pragma unroll
                            for (int kw = 0; kw < K; kw++)
#pragma unroll
                                for (int c = 0; c < 4; c++) {
                                    const float dj = j == 0 ? d[c].x : (j == 1 ? d[c].y : (j == 2 ? d[c].z : d[c].w));
                                    acc[c][i][kh * K + kw] = fmaf(dj, v[S * j + kw + VOFF], acc[c][i][kh * K + kw]);
                                }
                    }
            }
        }
    }
    __syncthreads();
    if (SMALL) {
        // the four pixel slices of a (co block, ci pair) sit in lanes that differ in bits 1 and 2
#pragma unroll
        for (int c = 0; c < 4; c++)
#pragma unroll
            for (int i = 0; i < 2; i++)
#pragma unroll
                for (int t = 0; t < KK; t++) {
                    float v = acc[c][i][t];
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    acc[c][i][t] = v;
                }
    }
    // cross-warp sum in warp order (fixed order: same result on every run)
    for (int w = 0; w < CONV_THREADS / 32; w++) {
        if (warp == w && kphase == 0) {
#pragma unroll
            for (int c = 0; c < 4; c++)
#pragma unroll
                for (int i = 0; i < 2; i++)
#pragma unroll
                    for (int t = 0; t < KK; t++) {
                        float *a = accs + ((cob * 4 + c) * 16 + cib + CI_STEP * i) * KK + t;
                        *a = (w == 0) ? acc[c][i][t] : *a + acc[c][i][t];
                    }
        }
        __syncthreads();
    }
    float *pp = part + (long long)group * g.Cout * g.Cin * KK;
    for (int e = tid; e < 16 * 16 * KK; e += CONV_THREADS) {
        int t = e % KK, ci = (e / KK) % 16, co = e / (KK * 16);
        if (co0 + co < g.Cout && ci0 + ci < g.Cin) pp[((long long)(co0 + co) * g.Cin + ci0 + ci) * KK + t] = accs[e];
    }
}

// out[i] = sum over groups of part[g][i], always added in the same order: 32 consecutive weights x 32 slices of the
// groups per CTA (slice s adds groups s, s+32, ...; the slices are then added in slice order by one thread per weight).
template <class T>
__global__ void __launch_bounds__(1024) reduce_partials_kernel(const float *__restrict__ part, T *__restrict__ out, long long n, int groups)
{
    __shared__ float sm[32][33];
    const int wx = threadIdx.x & 31, sl = threadIdx.x >> 5;
    const long long i = (long long)blockIdx.x * 32 + wx;
    float s = 0.f;
    if (i < n)
        for (int gidx = sl; gidx < groups; gidx += 32) s += part[(long long)gidx * n + i];
    sm[sl][wx] = s;
    __syncthreads();
    if (sl == 0 && i < n) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 32; k++) t += sm[k][wx];
        st(out + i, t);
    }
}

// fp32 results: 512 consecutive weights per CTA, 16-byte loads (partial_sums_quad; the deferred mode uses the same function)
__global__ void __launch_bounds__(1024) reduce_partials_f32_kernel(const float *__restrict__ part, float *__restrict__ out, long long n, int groups)
{
    __shared__ float4 sm[8][128];
    const long long i = (long long)blockIdx.x * PSUM_ELEMS + (threadIdx.x & 127) * 4;
    float4 t;
    if (!partial_sums_quad(part, n, groups, i, true, t, sm)) return;
    out[i] = t.x;
    if (i + 1 < n) out[i + 1] = t.y;
    if (i + 2 < n) out[i + 2] = t.z;
    if (i + 3 < n) out[i + 3] = t.w;
}
// the sum of `groups` partial results into `out`: now, or noted for the batched launch of the deferred mode
template <class T> static void reduce_partials(const float *part, T *out, long long n, int groups, bool deferred)
{
    if constexpr (sizeof(T) == 4) {
        float *o = reinterpret_cast<float *>(out);
        if (deferred) defer_plain(part, o, n, groups);
        else TL_LAUNCH(reduce_partials_f32_kernel, ceil_div(n, PSUM_ELEMS), 1024, 0, part, o, n, groups);
    } else {
        TL_LAUNCH((reduce_partials_kernel<T>), ceil_div(n, 32), 1024, 0, part, out, n, groups);
    }
}

// Fallback for filter windows above 5x5: one CTA per weight, block-wide reduction.
template <class T>
__global__ void __launch_bounds__(256) conv_wg_direct_kernel(ConvGeom g, const T *__restrict__ x, const T *__restrict__ dy, T *__restrict__ dw)
{
    __shared__ float red[256];
    const int KK = g.Hk * g.Wk;
    const int tap = blockIdx.x % KK, ci = (blockIdx.x / KK) % g.Cin, co = blockIdx.x / (KK * g.Cin);
    const int kh = tap / g.Wk, kw = tap % g.Wk;
    const long long per = (long long)g.Hout * g.Wout, total = per * g.n;
    float acc = 0.f;
    for (long long e = threadIdx.x; e < total; e += blockDim.x) {
        int s = e / per, p = e % per, ho = p / g.Wout, wo = p % g.Wout;
        int hi = ho * g.sh + kh - g.padU, wi = wo * g.sw + kw - g.padL;
        if (hi < 0 || hi >= g.Hin || wi < 0 || wi >= g.Win) continue;
        acc = fmaf(ld(x + (((long long)s * g.Cin + ci) * g.Hin + hi) * g.Win + wi),
                   ld(dy + ((long long)s * g.Cout + co) * per + p), acc);
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o]; __syncthreads(); }
    if (threadIdx.x == 0) st(dw + blockIdx.x, red[0]);
}

// db[co] = sum over streams and pixels of dY[co]   [ref: lib/sources/pulp_conv_naive_fp32.c:354-361]
template <class T>
__global__ void __launch_bounds__(256) channel_sum_kernel(const T *__restrict__ dy, T *__restrict__ db, int n, int C, long long plane)
{
    __shared__ float red[256];
    const int c = blockIdx.x;
    float acc = 0.f;
    for (long long e = threadIdx.x; e < plane * n; e += blockDim.x) {
        long long s = e / plane, p = e % plane;
        acc += ld(dy + (s * C + c) * plane + p);
    }
    red[threadIdx.x] = acc;
    __syncthreads();
    for (int o = 128; o > 0; o >>= 1) { if (threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o]; __syncthreads(); }
    if (threadIdx.x == 0) st(db + c, red[0]);
}

// tensor-core weight gradient (tl_conv_wgt.cu) where its geometry applies and the work is large enough to fill the GPU
template <class T> static bool try_tc_wg(Scope &, const ConvGeom &, const T *, const T *, T *) { return false; }
template <> bool try_tc_wg<float>(Scope &sc, const ConvGeom &g, const float *x, const float *dy, float *dw)
{
    if (gemm_path() == 1 || g.depthwise) return false;
    if (!(g.Hk == 3 && g.Wk == 3 && g.padL == 1 && g.padU == 1 && g.sh == g.sw && (g.sh == 1 || g.sh == 2))) return false;
    if (g.Hin != g.Hout * g.sh || g.Win != g.Wout * g.sw) return false;
    const long long work = (long long)g.n * g.Hout * g.Wout * g.Cout * g.Cin * 9;
    // Measured at 4096 streams: 2.2x (32 channels) and 2.5x (64) faster than the register-tiled FFMA kernel, no gain at 16
    // channels with stride 1, where M = (kh, ci) fills 48 of the 128 rows of an MMA.  Stride 2 doubles the rows per
    // channel (even and odd pixels), so it pays from 16 channels on.
    if (gemm_path() != 2 && (work < (1ll << 28) || g.Cin < (g.sh == 2 ? 16 : 32))) return false;
    int groups = 0;
    long long group_floats = 0;
    if (!conv_wgt_run(x, dy, nullptr, sm_count(), &groups, &group_floats, g.n, g.Cin, g.Cout, g.Hout, g.Wout, g.sh, true)) return false;
    bool deferred;
    float *part = partials_alloc<float>(sc, (size_t)groups * (size_t)group_floats, deferred);
    if (!part) return false;
    if (!conv_wgt_run(x, dy, part, groups, &groups, &group_floats, g.n, g.Cin, g.Cout, g.Hout, g.Wout, g.sh, false)) return false;
    conv_wgt_reduce(part, dw, groups, g.Cin, g.Cout, g.sh, deferred);
    return true;
}

// strided 1x1 weight gradient: per-CTA partials + the fixed-order reduction
template <class T> static bool try_1x1_wg(Scope &, const ConvGeom &, const T *, const T *, T *) { return false; }
template <> bool try_1x1_wg<float>(Scope &sc, const ConvGeom &g, const float *x, const float *dy, float *dw)
{
    int groups = 0;
    if (!conv1x1s_wg(g, x, dy, nullptr, 8 * sm_count(), &groups, true)) return false;
    const long long nw = (long long)g.Cout * g.Cin;
    bool deferred;
    float *part = partials_alloc<float>(sc, (size_t)groups * nw, deferred);
    if (!part) return false;
    if (!conv1x1s_wg(g, x, dy, part, groups, &groups, false)) return false;
    reduce_partials<float>(part, dw, nw, groups, deferred);
    return true;
}

template <class T> void conv_wg(Scope &sc, const ConvGeom &g, const T *x, const T *dy, T *dw, T *dbias)
{
    if (dbias) TL_LAUNCH((channel_sum_kernel<T>), g.Cout, 256, 0, dy, dbias, g.n, g.Cout, (long long)g.Hout * g.Wout);
    const int KK = g.Hk * g.Wk;
    if (g.depthwise) {
        TL_LAUNCH((dw_wg_kernel<T>), g.Cin * KK, 256, 0, g, x, dy, dw);
        return;
    }
    const long long nw = (long long)g.Cout * g.Cin * KK;
    const int ci_tiles = ceil_div(g.Cin, 16), co_tiles = ceil_div(g.Cout, 16);
    const bool k3 = g.Hk == 3 && g.Wk == 3 && g.padL == 1, k1 = g.Hk == 1 && g.Wk == 1 && g.padL == 0 && g.padU == 0;
    if (try_tc_wg<T>(sc, g, x, dy, dw)) return;
    if (try_1x1_wg<T>(sc, g, x, dy, dw)) return;
    if ((k3 || k1) && g.sh == g.sw && (g.sh == 1 || g.sh == 2) && g.Win == g.sw * g.Wout && (g.Wout == 8 || g.Wout == 16 || g.Wout == 32)) {
        // about 256 (stride 1) or 128 (stride 2) pixels per item: whole output rows, two streams for 8-pixel rows.
        // The item shape is part of the kernel type: (TW, TH, S_T) = (32, 8, 1), (16, 16, 1), (8, 8, 2) for stride 1
        // and (16, 8, 1), (8, 8, 2) for stride 2; images with fewer rows use the generic kernel below.
        const int S = g.sh, TW = g.Wout, K = g.Hk;
        const int TH = TW == 8 ? 8 : (S == 1 ? 256 : 128) / TW, S_T = TW == 8 ? 2 : 1;
        if (g.Hout >= TH && !(S == 2 && TW == 32)) {     // (64-wide inputs with stride 2 take the generic kernel)
            const int PH = (TH - 1) * S + K, RW = g.Win + 8, PLANE = 4 * ((PH * RW / 4) | 1);
            const size_t stage = (size_t)S_T * 16 * PLANE + (size_t)16 * (S_T * TH * TW + 4);
            const int nstage = (3 * stage * sizeof(float) <= 110 * 1024) ? 3 : 2;
            const size_t smem = std::max<size_t>(nstage * stage, (size_t)16 * 16 * KK) * sizeof(float);
            const int tiles_h = ceil_div(g.Hout, TH);
            const long long items = (long long)ceil_div(g.n, S_T) * tiles_h;
            // one wave: two CTAs fit an SM, and a grid that needs a few CTAs more than the slots runs twice as long
            int groups = (2 * sm_count()) / (ci_tiles * co_tiles);
            if (groups > items) groups = (int)items;
            if (groups < 1) groups = 1;
            bool deferred;
            float *part = partials_alloc<T>(sc, (size_t)groups * nw, deferred);
            if (!part) return;
            const int vec = sizeof(T) == 4 && (((uintptr_t)x | (uintptr_t)dy) & 15) == 0;
            dim3 grid(ci_tiles * co_tiles, groups);
#define TL_WG3_LAUNCH2(S_, TW_, K_, TH_, ST_)                                                                         \
    do {                                                                                                              \
        cudaFuncSetAttribute(conv_wg3x3_partial_kernel<T, S_, TW_, K_, TH_, ST_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        TL_LAUNCH((conv_wg3x3_partial_kernel<T, S_, TW_, K_, TH_, ST_>), grid, CONV_THREADS, smem, g, x, dy, part, tiles_h, ci_tiles, vec, nstage); \
    } while (0)
#define TL_WG3_LAUNCH(S_, TW_, TH_, ST_) do { if (K == 3) TL_WG3_LAUNCH2(S_, TW_, 3, TH_, ST_); else TL_WG3_LAUNCH2(S_, TW_, 1, TH_, ST_); } while (0)
            if (S == 1 && TW == 32 && K == 3 && g.Cin <= 4) {
                // first layer of a network: 3 or 4 input channels
                cudaFuncSetAttribute(conv_wg3x3_partial_kernel<T, 1, 32, 3, 8, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                TL_LAUNCH((conv_wg3x3_partial_kernel<T, 1, 32, 3, 8, 1, true>), grid, CONV_THREADS, smem, g, x, dy, part, tiles_h, ci_tiles, vec, nstage);
            }
            else if (S == 1) { if (TW == 32) TL_WG3_LAUNCH(1, 32, 8, 1); else if (TW == 16) TL_WG3_LAUNCH(1, 16, 16, 1); else TL_WG3_LAUNCH(1, 8, 8, 2); }
            else        { if (TW == 16) TL_WG3_LAUNCH(2, 16, 8, 1); else TL_WG3_LAUNCH(2, 8, 8, 2); }
#undef TL_WG3_LAUNCH
#undef TL_WG3_LAUNCH2
            profile_add_flops(conv_flops(g));
            reduce_partials<T>(part, dw, nw, groups, deferred);
            return;
        }
    }
    // pixel tile: whole rows, about 256 pixels
    int TW = g.Wout < 64 ? g.Wout : 64;
    int TH = 256 / TW; if (TH < 1) TH = 1; if (TH > g.Hout) TH = g.Hout;
    const int PH = (TH - 1) * g.sh + g.Hk, PW = ((TW - 1) * g.sw + g.Wk) | 1;
    size_t smem = ((size_t)16 * ((PH * PW) | 1) + (size_t)16 * (TH * TW + 1)) * sizeof(float);
    const bool tiled = (g.Hk == g.Wk) && (g.Hk == 1 || g.Hk == 3 || g.Hk == 5) && smem <= 200 * 1024;
    if (!tiled) {
        TL_LAUNCH((conv_wg_direct_kernel<T>), g.Cout * g.Cin * KK, 256, 0, g, x, dy, dw);
        profile_add_flops(conv_flops(g));
        return;
    }
    int tiles_w = ceil_div(g.Wout, TW), tiles_h = ceil_div(g.Hout, TH);
    long long items = (long long)g.n * tiles_w * tiles_h;
    int groups = ceil_div(4 * sm_count(), ci_tiles * co_tiles);
    if (groups > items) groups = (int)items;
    if (groups < 1) groups = 1;
    bool deferred;
    float *part = partials_alloc<T>(sc, (size_t)groups * nw, deferred);
    if (!part) return;
    dim3 grid(ci_tiles * co_tiles, groups);
#define TL_WG_LAUNCH(KH_, KW_)                                                                                        \
    do {                                                                                                              \
        if (smem > 48 * 1024)                                                                                         \
            cudaFuncSetAttribute(conv_wg_partial_kernel<T, KH_, KW_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        TL_LAUNCH((conv_wg_partial_kernel<T, KH_, KW_>), grid, CONV_THREADS, smem, g, x, dy, part, TH, TW, tiles_w, tiles_h, ci_tiles); \
    } while (0)
    if (g.Hk == 1) TL_WG_LAUNCH(1, 1);
    else if (g.Hk == 3) TL_WG_LAUNCH(3, 3);
    else TL_WG_LAUNCH(5, 5);
#undef TL_WG_LAUNCH
    profile_add_flops(conv_flops(g));
    reduce_partials<T>(part, dw, nw, groups, deferred);
}

// ------------------------------------------------------------------ explicit im2row / im2col / blocktranspose
// Kept for API completeness (the conv entry points never call them); index arithmetic is
// bit-exact with [ref: lib/sources/pulp_im2col_fp32.c:157-189 (FW/WG), :193-232 (IG), :668-1012, :1020-1072]
// wherever the reference's own pad test is right (pad <= 1), and mathematically correct beyond.
template <class T>
__global__ void im2row_kernel(const T *__restrict__ src, T *__restrict__ buf, int C, int H, int W, int Hk, int Wk,
                              int Ho, int Wo, int sh, int sw, int padU, int padL, int mode_ig, int hwc, int transposed)
{
    // mode 0: rows = output pixels (Ho x Wo), columns = (c,hk,wk) [CHW] or (hk,wk,c) [HWC], source = input.
    // mode 1: rows = input pixels (H x W), columns = (co,hk,wk) / (hk,wk,co), source = output gradient of
    //         size C x Ho x Wo, "full" correlation window starting at (hi-(Hk-1), wi-(Wk-1)).
    const int rows_h = mode_ig ? H : Ho, rows_w = mode_ig ? W : Wo;
    const long long K = (long long)C * Hk * Wk, total = K * rows_h * rows_w;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        long long row = e / K; int col = (int)(e % K);
        int rh = (int)(row / rows_w), rw = (int)(row % rows_w);
        int c, hk, wk;
        if (!hwc) { wk = col % Wk; hk = (col / Wk) % Hk; c = col / (Wk * Hk); }
        else { c = col % C; wk = (col / C) % Wk; hk = col / (C * Wk); }
        int sh_ = mode_ig ? rh - (Hk - 1) + hk : rh * sh + hk - padU;
        int sw_ = mode_ig ? rw - (Wk - 1) + wk : rw * sw + wk - padL;
        const int SH = mode_ig ? Ho : H, SW = mode_ig ? Wo : W;
        float v = 0.f;
        if (sh_ >= 0 && sh_ < SH && sw_ >= 0 && sw_ < SW)
            v = hwc ? ld(src + ((long long)sh_ * SW + sw_) * C + c) : ld(src + ((long long)c * SH + sh_) * SW + sw_);
        long long dst = transposed ? (long long)col * rows_h * rows_w + row : e;
        st(buf + dst, v);
    }
}

template <class T>
void im2row(const T *src, T *buf, int C, int H, int W, int Hk, int Wk, int Ho, int Wo,
            int sh, int sw, int padU, int padL, int mode_ig, int hwc, int transposed_buf)
{
    long long total = (long long)C * Hk * Wk * (mode_ig ? (long long)H * W : (long long)Ho * Wo);
    int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 16);
    if (blocks < 1) return;
    TL_LAUNCH((im2row_kernel<T>), blocks, 256, 0, src, buf, C, H, W, Hk, Wk, Ho, Wo, sh, sw, padU, padL, mode_ig, hwc, transposed_buf);
}

template <class T>
__global__ void blocktransp_kernel(const T *__restrict__ w, T *__restrict__ bt, int Cin, int Cout, int Hk, int Wk, int hwc)
{
    const int HW = Hk * Wk;
    const long long total = (long long)Cin * Cout * HW;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (long long)gridDim.x * blockDim.x) {
        if (!hwc) {
            int i = e % HW, k = (e / HW) % Cout, c = e / ((long long)HW * Cout);      // destination order [c][k][i]
            bt[e] = w[(HW - 1 - i) + (long long)c * HW + (long long)k * Cin * HW];
        } else {
            int co = e % Cout, wk = (e / Cout) % Wk, hk = (e / ((long long)Cout * Wk)) % Hk, ci = e / ((long long)Cout * HW);
            bt[e] = w[ci + (long long)(Wk - 1 - wk) * Cin + (long long)(Hk - 1 - hk) * Wk * Cin + (long long)co * HW * Cin];
        }
    }
}

template <class T> void blocktransp(const T *w, T *bt, int Cin, int Cout, int Hk, int Wk, int hwc)
{
    long long total = (long long)Cin * Cout * Hk * Wk;
    int blocks = (int)std::min<long long>((total + 255) / 256, (long long)sm_count() * 8);
    if (blocks < 1) return;
    TL_LAUNCH((blocktransp_kernel<T>), blocks, 256, 0, w, bt, Cin, Cout, Hk, Wk, hwc);
}

#define INST(T)                                                                                             \
    template void conv_fw<T>(Scope &, const ConvGeom &, const T *, const T *, const T *, T *);                       \
    template void conv_wg<T>(Scope &, const ConvGeom &, const T *, const T *, T *, T *);                    \
    template void conv_ig<T>(Scope &, const ConvGeom &, const T *, const T *, T *);                                  \
    template void conv_ig_accumulate<T>(Scope &, const ConvGeom &, const T *, const T *, T *);                       \
    template void im2row<T>(const T *, T *, int, int, int, int, int, int, int, int, int, int, int, int, int, int); \
    template void blocktransp<T>(const T *, T *, int, int, int, int, int);
INST(float)
INST(__half)

} // namespace tl
