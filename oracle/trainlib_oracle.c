/*
 * trainlib_oracle.c - CPU restatement of the PULP-TrainLib algorithms on the matmul-centred
 * training-step path.  TEST INFRASTRUCTURE ONLY: this file is the checker that tests, the
 * smoke run and the bench's cpu_baseline leg compare the CUDA library against.  Nothing in the
 * product may call it.
 *
 * Every function restates one reference routine (cited as [ref: file:line], paths relative to
 * the reference repository) with plain pointers and sizes: same formulas, same accumulation
 * order (one fp32 accumulator, ascending index) unless a comment says otherwise.  Where the
 * reference computes a wrong or undefined result, the comment says which result is restated.
 *
 * Pinning: tests/test_oracle_vs_reference.py checks every function here against the reference's
 * own C sources compiled into oracle/_ref/libpulp_ref.so (when present) and against the golden
 * vectors under tests/golden/ generated from that library and from the reference's PyTorch
 * golden model of MHSA.
 *
 * Build: make -C oracle oracle   (gcc -O2 -ffp-contract=off).
 */
#include "trainlib_oracle.h"
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ scalar bit tricks */

/* [ref: lib/sources/pulp_train_utils_fp32.c:1223-1231] Schraudolph exponential. */
float orc_fastexp_gist(float x)
{
    x = 12102203.17133801f * x + 1064986823.010288f;
    if (x < 8388608 || x > 2139095040) x = (x < 8388608) ? 0.0f : 2139095040;
    uint32_t n = (uint32_t)x;
    float r;
    memcpy(&r, &n, sizeof r);
    return r;
}

/* [ref: lib/sources/pulp_train_utils_fp32.c:1234-1247] fast inverse square root, one Newton
 * step; the pun is through a 32-bit integer (what the 32-bit target computes). */
float orc_q_rsqrt(float number)
{
    int32_t i;
    float y = number, x2 = number * 0.5f;
    memcpy(&i, &y, sizeof i);
    i = 0x5f3759df - (i >> 1);
    memcpy(&y, &i, sizeof y);
    return y * (1.5f - (x2 * y * y));
}

/* ------------------------------------------------------------------ matmul */

/* [ref: lib/sources/pulp_matmul_fp32.c:190-262] C[N x M] = A[N x K] * B; B is [K x M] or,
 * with trans_B, [M x K].  [ref: :267-340] mm_add accumulates into C. */
void orc_mm(const float *A, const float *B, float *C, int N, int K, int M, int trans_B, int accumulate)
{
    for (int i = 0; i < N; i++)
        for (int j = 0; j < M; j++) {
            float temp = 0;
            for (int k = 0; k < K; k++) temp += A[i * K + k] * (trans_B ? B[j * K + k] : B[k * M + j]);
            if (accumulate) C[i * M + j] += temp; else C[i * M + j] = temp;
        }
}

/* General strided product used by the attention restatement (same summation order). */
static void mm_strided(const float *A, long ars, long acs, const float *B, long brs, long bcs,
                       float *C, long crs, int N, int K, int M, float alpha, int accumulate)
{
    for (int i = 0; i < N; i++)
        for (int j = 0; j < M; j++) {
            float temp = 0;
            for (int k = 0; k < K; k++) temp += A[i * ars + k * acs] * B[k * brs + j * bcs];
            temp = temp * alpha;
            if (accumulate) C[i * crs + j] += temp; else C[i * crs + j] = temp;
        }
}

/* ------------------------------------------------------------------ im2row / blocktranspose */

/* [ref: lib/sources/pulp_im2col_fp32.c:157-189] mode 0: rows = output pixels, columns = (ci,hk,wk)
 * (CHW) or (hk,wk,ci) (HWC); the zero test is the geometric one (the reference's is equivalent
 * for pad <= 1).  [ref: :193-232] mode 1: rows = input pixels, columns over C_out, source = the
 * output gradient, window starting at (hi-(Hk-1), wi-(Wk-1)).
 * `transposed` stores buf[col][row] as pulp_im2col_fp32 does [ref: :756-775]. */
void orc_im2row(const float *src, float *buf, int C, int H, int W, int Hk, int Wk, int Ho, int Wo,
                int sh, int sw, int padU, int padL, int mode_ig, int hwc, int transposed)
{
    const int rows_h = mode_ig ? H : Ho, rows_w = mode_ig ? W : Wo;
    const int SH = mode_ig ? Ho : H, SW = mode_ig ? Wo : W;
    const long K = (long)C * Hk * Wk, R = (long)rows_h * rows_w;
    for (int rh = 0; rh < rows_h; rh++)
        for (int rw = 0; rw < rows_w; rw++)
            for (int c = 0; c < C; c++)
                for (int hk = 0; hk < Hk; hk++)
                    for (int wk = 0; wk < Wk; wk++) {
                        long row = (long)rh * rows_w + rw;
                        long col = hwc ? ((long)hk * Wk + wk) * C + c : ((long)c * Hk + hk) * Wk + wk;
                        int y = mode_ig ? rh - (Hk - 1) + hk : rh * sh + hk - padU;
                        int x = mode_ig ? rw - (Wk - 1) + wk : rw * sw + wk - padL;
                        float v = 0;
                        if (y >= 0 && y < SH && x >= 0 && x < SW)
                            v = hwc ? src[((long)y * SW + x) * C + c] : src[((long)c * SH + y) * SW + x];
                        buf[transposed ? col * R + row : row * K + col] = v;
                    }
}

/* [ref: lib/sources/pulp_im2col_fp32.c:1041-1052 (CHW), :1056-1065 (HWC)] swap the channel
 * blocks of the filter bank and rotate every filter by 180 degrees. */
void orc_blocktransp(const float *w, float *bt, int Cin, int Cout, int Hk, int Wk, int hwc)
{
    const int HW = Hk * Wk;
    if (!hwc) {
        for (int k = 0; k < Cout; k++)
            for (int c = 0; c < Cin; c++)
                for (int i = 0; i < HW; i++) bt[i + k * HW + c * Cout * HW] = w[(HW - 1 - i) + c * HW + k * Cin * HW];
    } else {
        for (int co = 0; co < Cout; co++)
            for (int hk = 0; hk < Hk; hk++)
                for (int wk = 0; wk < Wk; wk++)
                    for (int ci = 0; ci < Cin; ci++)
                        bt[ci * Hk * Wk * Cout + wk * Cout + hk * Wk * Cout + co] =
                            w[ci + (Wk - 1 - wk) * Cin + (Hk - 1 - hk) * Wk * Cin + co * Wk * Hk * Cin];
    }
}

/* ------------------------------------------------------------------ Conv2D (CHW) */

/* [ref: lib/sources/pulp_conv_naive_fp32.c:198-299] forward, accumulation over (ci,hk,wk). */
void orc_conv2d_fw(const float *x, const float *w, const float *bias, float *y, int Cin, int Hin, int Win,
                   int Cout, int Hk, int Wk, int sh, int sw, int padU, int padD, int padL, int padR)
{
    const int Ho = (Hin - Hk + padU + padD) / sh + 1, Wo = (Win - Wk + padL + padR) / sw + 1;
    for (int co = 0; co < Cout; co++)
        for (int ho = 0; ho < Ho; ho++)
            for (int wo = 0; wo < Wo; wo++) {
                float temp = 0;
                for (int ci = 0; ci < Cin; ci++)
                    for (int hk = 0; hk < Hk; hk++)
                        for (int wk = 0; wk < Wk; wk++) {
                            int hi = sh * ho + hk - padU, wi = sw * wo + wk - padL;
                            if (hi >= 0 && wi >= 0 && hi < Hin && wi < Win)
                                temp += x[wi + hi * Win + ci * Hin * Win] * w[wk + hk * Wk + ci * Hk * Wk + co * Cin * Hk * Wk];
                        }
                y[wo + ho * Wo + co * Ho * Wo] = temp;
                if (bias) y[wo + ho * Wo + co * Ho * Wo] += bias[co];
            }
}

/* [ref: lib/sources/pulp_conv_naive_fp32.c:302-407] weight gradient, accumulation over (ho,wo);
 * bias gradient = sum of the output gradient per channel [ref: :354-361]. */
void orc_conv2d_wg(const float *x, const float *dy, float *dw, float *dbias, int Cin, int Hin, int Win,
                   int Cout, int Hk, int Wk, int sh, int sw, int padU, int padD, int padL, int padR)
{
    const int Ho = (Hin - Hk + padU + padD) / sh + 1, Wo = (Win - Wk + padL + padR) / sw + 1;
    for (int co = 0; co < Cout; co++) {
        for (int hk = 0; hk < Hk; hk++)
            for (int wk = 0; wk < Wk; wk++)
                for (int ci = 0; ci < Cin; ci++) {
                    float temp = 0;
                    for (int ho = 0; ho < Ho; ho++)
                        for (int wo = 0; wo < Wo; wo++) {
                            int hi = sh * ho + hk - padU, wi = sw * wo + wk - padL;
                            if (hi >= 0 && wi >= 0 && hi < Hin && wi < Win)
                                temp += dy[wo + ho * Wo + co * Ho * Wo] * x[wi + hi * Win + ci * Hin * Win];
                        }
                    dw[wk + hk * Wk + ci * Hk * Wk + co * Hk * Wk * Cin] = temp;
                }
        if (dbias) {
            float b = 0;
            for (int p = 0; p < Ho * Wo; p++) b += dy[p + co * Ho * Wo];
            dbias[co] = b;
        }
    }
}

/* [ref: lib/sources/pulp_conv_naive_fp32.c:410-515] input gradient: for every input pixel, the
 * taps (co,hk,wk) whose output position (hi+padU-hk)/sh is integral and in range, visited with
 * the filter index running backwards as the reference does (kernel flipped). */
void orc_conv2d_ig(const float *dy, const float *w, float *dx, int Cin, int Hin, int Win,
                   int Cout, int Hk, int Wk, int sh, int sw, int padU, int padD, int padL, int padR)
{
    const int Ho = (Hin - Hk + padU + padD) / sh + 1, Wo = (Win - Wk + padL + padR) / sw + 1;
    for (int ci = 0; ci < Cin; ci++)
        for (int hi = 0; hi < Hin; hi++)
            for (int wi = 0; wi < Win; wi++) {
                float temp = 0;
                for (int co = 0; co < Cout; co++)
                    for (int hk = Hk - 1; hk >= 0; hk--)          /* flipped index ascending = hk descending */
                        for (int wk = Wk - 1; wk >= 0; wk--) {
                            int t = hi + padU - hk, u = wi + padL - wk;
                            if (t < 0 || u < 0 || t % sh || u % sw) continue;
                            int ho = t / sh, wo = u / sw;
                            if (ho >= Ho || wo >= Wo) continue;
                            temp += w[wk + hk * Wk + ci * Hk * Wk + co * Hk * Wk * Cin] * dy[wo + ho * Wo + co * Ho * Wo];
                        }
                dx[wi + hi * Win + ci * Hin * Win] = temp;
            }
}

/* ------------------------------------------------------------------ depthwise conv */

/* [ref: lib/sources/pulp_conv_naive_fp32.c:29-110] */
void orc_dw_fw(const float *x, const float *w, float *y, int C, int Hin, int Win, int Hk, int Wk,
               int sh, int sw, int padU, int padD, int padL, int padR)
{
    const int Ho = (Hin - Hk + padU + padD) / sh + 1, Wo = (Win - Wk + padL + padR) / sw + 1;
    for (int ch = 0; ch < C; ch++)
        for (int ho = 0; ho < Ho; ho++)
            for (int wo = 0; wo < Wo; wo++) {
                float temp = 0;
                for (int hk = 0; hk < Hk; hk++)
                    for (int wk = 0; wk < Wk; wk++) {
                        int hi = sh * ho + hk - padU, wi = sw * wo + wk - padL;
                        if (hi >= 0 && wi >= 0 && hi < Hin && wi < Win)
                            temp += w[wk + hk * Wk + ch * Hk * Wk] * x[wi + hi * Win + ch * Hin * Win];
                    }
                y[wo + ho * Wo + ch * Ho * Wo] = temp;
            }
}

/* [ref: lib/sources/pulp_conv_naive_fp32.c:113-150] restated with stride and padding honoured
 * (the reference ignores both here and is only valid for stride 1, pad 0). */
void orc_dw_wg(const float *x, const float *dy, float *dw, int C, int Hin, int Win, int Hk, int Wk,
               int sh, int sw, int padU, int padD, int padL, int padR)
{
    const int Ho = (Hin - Hk + padU + padD) / sh + 1, Wo = (Win - Wk + padL + padR) / sw + 1;
    for (int ch = 0; ch < C; ch++)
        for (int hk = 0; hk < Hk; hk++)
            for (int wk = 0; wk < Wk; wk++) {
                float temp = 0;
                for (int ho = 0; ho < Ho; ho++)
                    for (int wo = 0; wo < Wo; wo++) {
                        int hi = sh * ho + hk - padU, wi = sw * wo + wk - padL;
                        if (hi >= 0 && wi >= 0 && hi < Hin && wi < Win)
                            temp += x[wi + hi * Win + ch * Hin * Win] * dy[wo + ho * Wo + ch * Ho * Wo];
                    }
                dw[wk + hk * Wk + ch * Hk * Wk] = temp;
            }
}

/* [ref: lib/sources/pulp_conv_naive_fp32.c:153-194] same remark on stride and padding. */
void orc_dw_ig(const float *dy, const float *w, float *dx, int C, int Hin, int Win, int Hk, int Wk,
               int sh, int sw, int padU, int padD, int padL, int padR)
{
    const int Ho = (Hin - Hk + padU + padD) / sh + 1, Wo = (Win - Wk + padL + padR) / sw + 1;
    for (int ch = 0; ch < C; ch++)
        for (int hi = 0; hi < Hin; hi++)
            for (int wi = 0; wi < Win; wi++) {
                float temp = 0;
                for (int hk = Hk - 1; hk >= 0; hk--)
                    for (int wk = Wk - 1; wk >= 0; wk--) {
                        int t = hi + padU - hk, u = wi + padL - wk;
                        if (t < 0 || u < 0 || t % sh || u % sw) continue;
                        int ho = t / sh, wo = u / sw;
                        if (ho >= Ho || wo >= Wo) continue;
                        temp += w[wk + hk * Wk + ch * Hk * Wk] * dy[wo + ho * Wo + ch * Ho * Wo];
                    }
                dx[wi + hi * Win + ch * Hin * Win] = temp;
            }
}

/* ------------------------------------------------------------------ Linear */

/* [ref: lib/sources/pulp_linear_fp32.c:39-55] y = W x; the bias add follows the fp16 twin
 * [ref: lib/sources/pulp_linear_fp16.c:252-258] (the fp32 forward never adds it). */
void orc_linear_fw(const float *W, const float *x, const float *bias, float *y, int out, int in)
{
    orc_mm(W, x, y, out, in, 1, 0, 0);
    if (bias) for (int o = 0; o < out; o++) y[o] += bias[o];
}
/* [ref: lib/sources/pulp_linear_fp32.c:102-117, :234-262] dW = dy (x) x; db = dy. */
void orc_linear_wg(const float *dy, const float *x, float *dW, float *dbias, int out, int in)
{
    orc_mm(dy, x, dW, out, 1, in, 0, 0);
    if (dbias) for (int o = 0; o < out; o++) dbias[o] = dy[o];
}
/* [ref: lib/sources/pulp_linear_fp32.c:163-180] dx = dy^T W. */
void orc_linear_ig(const float *dy, const float *W, float *dx, int out, int in)
{
    orc_mm(dy, W, dx, 1, out, in, 0, 0);
}

/* ------------------------------------------------------------------ softmax */

/* [ref: lib/sources/pulp_act_fp32.c:187-245; pulp_train_utils_fp32.c:1046-1138] row maximum,
 * Schraudolph exponential of the shifted row, division by the row sum. */
void orc_softmax_fw(const float *in, float *out, int rows, int width)
{
    for (int i = 0; i < rows; i++) {
        float mx = -340282346638528859811704183484516925440.0f, sum = 0.0f;
        for (int j = 0; j < width; j++) if (mx < in[i * width + j]) mx = in[i * width + j];
        for (int j = 0; j < width; j++) { float o = orc_fastexp_gist(in[i * width + j] - mx); out[i * width + j] = o; sum += o; }
        for (int j = 0; j < width; j++) out[i * width + j] = out[i * width + j] / sum;
    }
}
/* [ref: lib/sources/pulp_act_fp32.c:335-392; pulp_train_utils_fp32.c:1140-1189] */
void orc_softmax_bw(const float *out, const float *dout, float *din, int rows, int width)
{
    for (int i = 0; i < rows; i++) {
        float s = 0;
        for (int j = 0; j < width; j++) s += dout[i * width + j] * out[i * width + j];
        for (int j = 0; j < width; j++) din[i * width + j] = (dout[i * width + j] - s) * out[i * width + j];
    }
}

/* ------------------------------------------------------------------ multi-head self-attention */

/* [ref: lib/sources/pulp_mhsa_fp32.c:20-644] x, y: E x L; Wq/Wk/Wv/Wo: E x F; q,k,v,att: F x L;
 * softmax: heads x L x L as [head][query][key].  The reference's transposes are folded into the
 * operand strides; every product keeps its summation order. */
void orc_mhsa_fw(const float *x, const float *wq, const float *wk, const float *wv,
                 const float *bq, const float *bk, const float *bv, const float *wo,
                 float *q, float *k, float *v, float *softmax, float *att, float *y,
                 int L, int E, int F, int heads)
{
    const int H = F / heads;
    const float scaling = orc_q_rsqrt((float)H);
    const float *ws[3] = {wq, wk, wv}, *bs[3] = {bq, bk, bv};
    float *outs[3] = {q, k, v};
    for (int p = 0; p < 3; p++) {
        mm_strided(ws[p], 1, F, x, L, 1, outs[p], L, F, E, L, 1.0f, 0);        /* W^T x  [ref: :87-118] */
        if (bs[p]) for (int f = 0; f < F; f++) for (int l = 0; l < L; l++) outs[p][f * L + l] += bs[p][f];   /* [ref: :152-158] */
    }
    float *scores = (float *)malloc(sizeof(float) * L * L);
    for (int h = 0; h < heads; h++) {
        const float *qh = q + h * H * L, *kh = k + h * H * L, *vh = v + h * H * L;
        /* scores[query][key] = (sum_d k[d][key] q[d][query]) * scaling   [ref: :348-431, :464] */
        for (int a = 0; a < L; a++)
            for (int b = 0; b < L; b++) {
                float temp = 0;
                for (int d = 0; d < H; d++) temp += kh[d * L + b] * qh[d * L + a];
                scores[a * L + b] = temp * scaling;
            }
        orc_softmax_fw(scores, softmax + (long)h * L * L, L, L);               /* [ref: :491] */
        /* att[d][query] = sum_key v[d][key] P[query][key]   [ref: :530-560] */
        mm_strided(vh, L, 1, softmax + (long)h * L * L, 1, L, att + h * H * L, L, H, L, L, 1.0f, 0);
    }
    free(scores);
    orc_mm(wo, att, y, E, F, L, 0, 0);                                          /* [ref: :612] */
}

/* [ref: lib/sources/pulp_mhsa_fp32.c:648-1745] with the third transpose taken as H x L (the
 * shipped {L,H} at :930 is only right for L == H).  Weight gradients of the projections are
 * F x E; dx accumulates into the caller's buffer. */
void orc_mhsa_bw(const float *x, const float *wq, const float *wk, const float *wv, const float *wo,
                 const float *q, const float *k, const float *v, const float *softmax, const float *att,
                 const float *dy, float *dq, float *dk, float *dv, float *dsoftmax, float *datt,
                 float *dwq, float *dwk, float *dwv, float *dwo, float *dx,
                 int L, int E, int F, int heads)
{
    const int H = F / heads;
    const float scaling = orc_q_rsqrt((float)H);
    mm_strided(dy, L, 1, att, 1, L, dwo, F, E, L, F, 1.0f, 0);                  /* dWo = dY att^T  [ref: :704-760] */
    mm_strided(wo, 1, F, dy, L, 1, datt, L, F, E, L, 1.0f, 0);                  /* datt = Wo^T dY  [ref: :783-837] */
    float *dS = (float *)malloc(sizeof(float) * L * L);
    for (int h = 0; h < heads; h++) {
        const float *P = softmax + (long)h * L * L;
        float *dP = dsoftmax + (long)h * L * L;
        const float *qh = q + h * H * L, *kh = k + h * H * L, *vh = v + h * H * L, *dah = datt + h * H * L;
        mm_strided(dah, L, 1, P, L, 1, dv + h * H * L, L, H, L, L, 1.0f, 0);    /* dv = datt P  [ref: :842-895] */
        mm_strided(dah, 1, L, vh, L, 1, dP, L, L, H, L, 1.0f, 0);               /* dP[query][key]  [ref: :923-1050] */
        orc_softmax_bw(P, dP, dS, L, L);                                        /* [ref: :1052-1100] */
        for (int i = 0; i < L * L; i++) dS[i] = dS[i] * scaling;                /* [ref: :1126-1138] */
        mm_strided(qh, L, 1, dS, L, 1, dk + h * H * L, L, H, L, L, 1.0f, 0);    /* dk[d][key]  [ref: :1140-1330] */
        mm_strided(kh, L, 1, dS, 1, L, dq + h * H * L, L, H, L, L, 1.0f, 0);    /* dq[d][query]  [ref: :1340-1400] */
    }
    free(dS);
    const float *dps[3] = {dq, dk, dv}, *ws[3] = {wq, wk, wv};
    float *dws[3] = {dwq, dwk, dwv};
    for (int p = 0; p < 3; p++) mm_strided(dps[p], L, 1, x, 1, L, dws[p], E, F, L, E, 1.0f, 0);   /* [ref: :1426-1600] */
    for (int p = 0; p < 3; p++) mm_strided(ws[p], F, 1, dps[p], L, 1, dx, L, E, F, L, 1.0f, 1);   /* [ref: :1605-1745] */
}

/* Attention of the MobileBERT encoder block ("inference" entry points and their tiled twins)
 * [ref: lib/sources/pulp_mhsa_fp32.c:1749-2035 forward, :2162-2412 the same arithmetic through DMA tiles, :2413-2840
 * backward].  PARITY UNPINNED: these reference functions do not compile against the reference's own headers (they
 * fill `struct transp_args` fields N / M / matrix / transp_matrix that lib/include/pulp_train_utils_fp32.h no longer
 * declares, and the tiled ones need the cluster DMA), so they cannot be run here; this is a restatement of the
 * forward's loops, and the backward is the exact gradient of that forward in the forward's own layouts (the
 * reference's backward reads output.diff as E x L although the forward writes the output as L x N).
 * x: L x E; xb (bottleneck input): L x Kb; Wq, Wk: F x Kb; Wv: F x E; Wo: No x F; biases per output row;
 * q, k, v, att: F x L; softmax: heads x L x L as [head][query][key]; y: L x No. */
void orc_mhsa_mobilebert_fw(const float *x, const float *xb, const float *wq, const float *wk, const float *wv,
                            const float *bq, const float *bk, const float *bv, const float *wo, const float *bo,
                            float *q, float *k, float *v, float *softmax, float *att, float *y,
                            int L, int E, int Kb, int F, int No, int heads)
{
    const int H = F / heads;
    const float scaling = orc_q_rsqrt((float)H);
    mm_strided(wq, Kb, 1, xb, 1, Kb, q, L, F, Kb, L, 1.0f, 0);                 /* Wq xb^T  [ref: :1789-1815] */
    mm_strided(wk, Kb, 1, xb, 1, Kb, k, L, F, Kb, L, 1.0f, 0);                 /* [ref: :1818-1843] */
    mm_strided(wv, E, 1, x, 1, E, v, L, F, E, L, 1.0f, 0);                     /* Wv x^T  [ref: :1918-1943] */
    for (int f = 0; f < F; f++)
        for (int l = 0; l < L; l++) { q[f * L + l] += bq[f]; k[f * L + l] += bk[f]; v[f * L + l] += bv[f]; }
    float *scores = (float *)malloc(sizeof(float) * L * L);
    for (int h = 0; h < heads; h++) {
        const float *qh = q + h * H * L, *kh = k + h * H * L, *vh = v + h * H * L;
        for (int a = 0; a < L; a++)                                             /* [ref: :1846-1915] */
            for (int b = 0; b < L; b++) {
                float temp = 0;
                for (int d = 0; d < H; d++) temp += kh[d * L + b] * qh[d * L + a];
                scores[a * L + b] = temp * scaling;
            }
        orc_softmax_fw(scores, softmax + (long)h * L * L, L, L);
        mm_strided(vh, L, 1, softmax + (long)h * L * L, 1, L, att + h * H * L, L, H, L, L, 1.0f, 0);   /* [ref: :1946-1975] */
    }
    free(scores);
    for (int n = 0; n < No; n++)                                                /* Wo att + bo, stored transposed  [ref: :1978-2034] */
        for (int l = 0; l < L; l++) {
            float temp = 0;
            for (int f = 0; f < F; f++) temp += wo[n * F + f] * att[f * L + l];
            y[l * No + n] = temp + bo[n];
        }
}

/* dy: L x No.  dwq, dwk: F x Kb; dwv: F x E; dwo: No x F; dx: L x E and dxb: L x Kb are accumulated into. */
void orc_mhsa_mobilebert_bw(const float *x, const float *xb, const float *wq, const float *wk, const float *wv, const float *wo,
                            const float *q, const float *k, const float *v, const float *softmax, const float *att, const float *dy,
                            float *dq, float *dk, float *dv, float *dsoftmax, float *datt,
                            float *dwq, float *dwk, float *dwv, float *dwo, float *dx, float *dxb,
                            int L, int E, int Kb, int F, int No, int heads)
{
    const int H = F / heads;
    const float scaling = orc_q_rsqrt((float)H);
    mm_strided(dy, 1, No, att, 1, L, dwo, F, No, L, F, 1.0f, 0);               /* dWo[n][f] = sum_l dy[l][n] att[f][l] */
    mm_strided(wo, 1, F, dy, 1, No, datt, L, F, No, L, 1.0f, 0);               /* datt[f][l] = sum_n wo[n][f] dy[l][n] */
    float *dS = (float *)malloc(sizeof(float) * L * L);
    for (int h = 0; h < heads; h++) {
        const float *P = softmax + (long)h * L * L;
        float *dP = dsoftmax + (long)h * L * L;
        const float *qh = q + h * H * L, *kh = k + h * H * L, *vh = v + h * H * L, *dah = datt + h * H * L;
        mm_strided(dah, L, 1, P, L, 1, dv + h * H * L, L, H, L, L, 1.0f, 0);
        mm_strided(dah, 1, L, vh, L, 1, dP, L, L, H, L, 1.0f, 0);
        orc_softmax_bw(P, dP, dS, L, L);
        for (int i = 0; i < L * L; i++) dS[i] = dS[i] * scaling;
        mm_strided(qh, L, 1, dS, L, 1, dk + h * H * L, L, H, L, L, 1.0f, 0);
        mm_strided(kh, L, 1, dS, 1, L, dq + h * H * L, L, H, L, L, 1.0f, 0);
    }
    free(dS);
    mm_strided(dq, L, 1, xb, Kb, 1, dwq, Kb, F, L, Kb, 1.0f, 0);               /* dWq[f][c] = sum_l dq[f][l] xb[l][c] */
    mm_strided(dk, L, 1, xb, Kb, 1, dwk, Kb, F, L, Kb, 1.0f, 0);
    mm_strided(dv, L, 1, x, E, 1, dwv, E, F, L, E, 1.0f, 0);
    mm_strided(dq, 1, L, wq, Kb, 1, dxb, Kb, L, F, Kb, 1.0f, 1);               /* dxb[l][c] += sum_f dq[f][l] wq[f][c] */
    mm_strided(dk, 1, L, wk, Kb, 1, dxb, Kb, L, F, Kb, 1.0f, 1);
    mm_strided(dv, 1, L, wv, E, 1, dx, E, L, F, E, 1.0f, 1);
}

/* ------------------------------------------------------------------ activations */

/* kind: 0 relu, 1 leaky relu, 2 sigmoid, 3 gelu (rational tanh)
 * [ref: lib/sources/pulp_act_fp32.c:37-180, :714-746] */
void orc_act_fw(int kind, const float *x, float *y, long n, float slope)
{
    for (long i = 0; i < n; i++) {
        float v = x[i];
        if (kind == 0) y[i] = v > 0 ? v : 0;
        else if (kind == 1) y[i] = v > 0 ? v : v * slope;
        else if (kind == 2) { float s = 1 + expf(-v); y[i] = 1 / s; }
        else {
            float half_x = 0.5f * v;
            float val = (((v * v * v * 0.044715f) + v) * 0.7978f);
            float val_2 = val * val;
            float a = (((val_2 + 378.0f) * val_2 + 17325.0f) * val_2 + 135135.0f) * val;
            float b = ((28.0f * val_2 + 3150.0f) * val_2 + 62370.0f) * val_2 + 135135.0f;
            val = a / b;
            if (val > 1) val = 1; else if (val < -1) val = -1;
            y[i] = val * half_x + half_x;
        }
    }
}
/* Backward of relu / leaky relu / sigmoid [ref: lib/sources/pulp_act_fp32.c:52-78, :110-127, :163-180].
 * GELU has no backward in the reference ("parity unpinned"): kind 3 differentiates the forward's
 * own rational approximation analytically. */
void orc_act_bw(int kind, const float *x, const float *y, const float *dy, float *dx, long n, float slope)
{
    for (long i = 0; i < n; i++) {
        if (kind == 0) dx[i] = x[i] > 0 ? dy[i] : 0;
        else if (kind == 1) dx[i] = x[i] > 0 ? dy[i] : dy[i] * slope;
        else if (kind == 2) { float s = y[i]; dx[i] = dy[i] * (s * (1.0f - s)); }
        else {
            double v = x[i];
            double u = (v * v * v * 0.044715 + v) * 0.7978, du = (3 * 0.044715 * v * v + 1) * 0.7978, u2 = u * u;
            double a = (((u2 + 378.0) * u2 + 17325.0) * u2 + 135135.0) * u;
            double b = ((28.0 * u2 + 3150.0) * u2 + 62370.0) * u2 + 135135.0;
            double da = ((7 * u2 + 5 * 378.0) * u2 + 3 * 17325.0) * u2 + 135135.0;
            double db = ((6 * 28.0 * u2 + 4 * 3150.0) * u2 + 2 * 62370.0) * u;
            double t = a / b, dt = (da * b - a * db) / (b * b);
            if (t > 1) { t = 1; dt = 0; } else if (t < -1) { t = -1; dt = 0; }
            dx[i] = (float)(dy[i] * (0.5 * (1 + t) + 0.5 * v * dt * du));
        }
    }
}

/* ------------------------------------------------------------------ norms */

/* [ref: lib/sources/pulp_train_utils_fp32.c:1685-1728] */
static void mean_std(const float *data, int D, float eps, float *mean, float *var, float *std)
{
    float D_inverse = (1 / (float)D), m = 0, v = 0;
    for (int d = 0; d < D; d++) { float t = data[d]; m += t; v += t * t; }
    m = m * D_inverse;
    v = v * D_inverse;
    v -= m * m;
    v = v + eps;
    if (v < 0) v = eps;
    *mean = m; *var = v; *std = sqrtf(v);
}
/* [ref: lib/sources/pulp_instnorm_fp32.c:33-115] gb = [gamma(C), beta(C)] */
void orc_instnorm_fw(const float *x, float *y, const float *gb, float *mean, float *var, float *stdev, int C, int D)
{
    for (int ch = 0; ch < C; ch++) {
        mean_std(x + (long)ch * D, D, 1e-10, &mean[ch], &var[ch], &stdev[ch]);
        float gamma = gb[ch] / stdev[ch], b = gb[C + ch];
        for (int d = 0; d < D; d++) y[(long)ch * D + d] = gamma * (x[(long)ch * D + d] - mean[ch]) + b;
    }
}
/* [ref: lib/sources/pulp_instnorm_fp32.c:117-175] */
void orc_instnorm_bw_input(const float *x, const float *dy, float *dx, const float *gb, const float *mean,
                           const float *var, const float *stdev, int C, int D)
{
    for (int c = 0; c < C; c++) {
        const float *in = x + (long)c * D, *od = dy + (long)c * D;
        float gs = 0, gp = 0;
        for (int i = 0; i < D; i++) { gs -= od[i]; gp -= (in[i] - mean[c]) * od[i]; }
        for (int d = 0; d < D; d++) {
            float grad = gs;
            float mean_d = (in[d] - mean[c]) / var[c];
            grad += gp * mean_d;
            grad += D * od[d];
            grad = grad * gb[c] / (D * stdev[c]);
            dx[(long)c * D + d] = grad;
        }
    }
}
/* [ref: lib/sources/pulp_instnorm_fp32.c:182-230] dgb = [dgamma(C), dbeta(C)] */
void orc_instnorm_bw_param(const float *x, const float *dy, float *dgb, const float *mean, const float *stdev, int C, int D)
{
    for (int c = 0; c < C; c++) {
        float g = 0, b = 0;
        for (int d = 0; d < D; d++) { g += dy[(long)c * D + d] * (x[(long)c * D + d] - mean[c]); b += dy[(long)c * D + d]; }
        dgb[c] = g / stdev[c];
        dgb[C + c] = b;
    }
}
/* [ref: lib/sources/pulp_batchnorm_fp32.c:84-109] x is [B][C][HW] */
void orc_batchnorm_fw(const float *x, float *y, const float *w, const float *b, int B, int C, int HW, float eps)
{
    const int n = B * HW;
    for (int c = 0; c < C; c++) {
        float s1 = 0.0f, s2 = 0.0f;
        for (int bb = 0; bb < B; bb++)
            for (int p = 0; p < HW; p++) { float t = x[((long)bb * C + c) * HW + p]; s1 += t; s2 += t * t; }
        float mean = s1 / n;
        float sqrt_var = (float)sqrt(((s2 - 2 * s1 * mean) / n) + (mean * mean) + eps);
        for (int bb = 0; bb < B; bb++)
            for (int p = 0; p < HW; p++) {
                long i = ((long)bb * C + c) * HW + p;
                y[i] = ((x[i] - mean) / sqrt_var) * w[c] + b[c];
            }
    }
}
/* [ref: lib/sources/pulp_layernorm_fp32.c:60-77] */
void orc_layernorm_fw(const float *x, float *y, const float *w, const float *b, int rows, int width, float eps)
{
    for (int i = 0; i < rows; i++) {
        float s1 = 0.0f, s2 = 0.0f;
        for (int j = 0; j < width; j++) { float t = x[(long)i * width + j]; s1 += t; s2 += t * t; }
        float mean = s1 / width;
        float sqrt_var = (float)sqrt(((s2 - 2 * s1 * mean) / width) + (mean * mean) + eps);
        for (int j = 0; j < width; j++) y[(long)i * width + j] = ((x[(long)i * width + j] - mean) / sqrt_var) * w[j] + b[j];
    }
}

/* Backward of the layer norm above.  The reference has no backward for it ("parity unpinned"): this differentiates
 * the forward formula [ref: lib/sources/pulp_layernorm_fp32.c:60-77]; tests pin it against PyTorch autograd. */
void orc_layernorm_bw(const float *x, const float *w, const float *dy, float *dx, float *dw, float *db, int rows, int width, float eps)
{
    for (int j = 0; j < width; j++) { dw[j] = 0.0f; db[j] = 0.0f; }
    for (int i = 0; i < rows; i++) {
        const float *xr = x + (long)i * width, *gr = dy + (long)i * width;
        float s1 = 0.0f, s2 = 0.0f;
        for (int j = 0; j < width; j++) { s1 += xr[j]; s2 += xr[j] * xr[j]; }
        float mean = s1 / width;
        float sv = (float)sqrt(((s2 - 2 * s1 * mean) / width) + (mean * mean) + eps);
        float a = 0.0f, b = 0.0f;
        for (int j = 0; j < width; j++) { float g = w[j] * gr[j], xh = (xr[j] - mean) / sv; a += g; b += g * xh; }
        a /= width; b /= width;
        for (int j = 0; j < width; j++) {
            float g = w[j] * gr[j], xh = (xr[j] - mean) / sv;
            dx[(long)i * width + j] = (g - a - xh * b) / sv;
            dw[j] += gr[j] * xh; db[j] += gr[j];
        }
    }
}

/* Batched product with NumPy broadcasting of the leading dimensions [ref: lib/sources/pulp_matmul_fp32.c:29-186]:
 * A [..., N, K] x B [..., K, M]; leading dimensions aligned from the right, size 1 (or missing) repeats the matrix;
 * every product is the plain mm of the reference (k ascending, one accumulator). */
void orc_mm_broadcast(const float *A, const float *B, float *C, const int *ad, int la, const int *bd, int lb)
{
    int lead = (la > lb ? la : lb) - 2, N = ad[la - 2], K = ad[la - 1], M = bd[lb - 1];
    long od[8], sa[8], sb[8], total = 1, ra = (long)N * K, rb = (long)K * M;
    for (int d = lead - 1; d >= 0; d--) {
        int ia = d - (lead - (la - 2)), ib = d - (lead - (lb - 2));
        int da = ia >= 0 ? ad[ia] : 1, db = ib >= 0 ? bd[ib] : 1;
        od[d] = da > db ? da : db; sa[d] = da == 1 ? 0 : ra; sb[d] = db == 1 ? 0 : rb;
        ra *= da; rb *= db; total *= od[d];
    }
    for (long i = 0; i < total; i++) {
        long r = i, oa = 0, ob = 0;
        for (int d = lead - 1; d >= 0; d--) { oa += (r % od[d]) * sa[d]; ob += (r % od[d]) * sb[d]; r /= od[d]; }
        const float *a = A + oa, *b = B + ob; float *c = C + i * (long)N * M;
        for (int n = 0; n < N; n++)
            for (int m = 0; m < M; m++) {
                float t = 0.0f;
                for (int k = 0; k < K; k++) t += a[(long)n * K + k] * b[(long)k * M + m];
                c[(long)n * M + m] = t;
            }
    }
}

/* ------------------------------------------------------------------ losses */

/* [ref: lib/sources/pulp_losses_fp32.c:214-275] */
float orc_mse_fw(const float *y, const float *t, int n)
{
    float loss = 0.0f, meanval = 1.0f / n;
    for (int i = 0; i < n; i++) loss += meanval * (t[i] - y[i]) * (t[i] - y[i]);
    return loss;
}
void orc_mse_bw(const float *y, const float *t, float *dy, int n)
{
    float meanval = 1.0f / n;
    for (int i = 0; i < n; i++) dy[i] = meanval * 2.0f * (y[i] - t[i]);
}
/* [ref: lib/sources/pulp_losses_fp32.c:26-88] */
float orc_ce_fw(const float *z, const float *t, int n)
{
    float mx = z[0];
    for (int i = 1; i < n; i++) if (z[i] > mx) mx = z[i];
    float se = 0.0f;
    for (int i = 0; i < n; i++) se += expf(z[i] - mx);
    float lse = logf(se) + mx, dot = 0.0f, sy = 0.0f;
    for (int i = 0; i < n; i++) { dot += t[i] * z[i]; sy += t[i]; }
    if (sy == 0.0f) sy = 1.0f;
    return -(dot - lse * sy);
}
/* [ref: lib/sources/pulp_losses_fp32.c:91-137] */
void orc_ce_bw(const float *z, const float *t, float *dz, int n)
{
    float mx = z[0];
    for (int i = 1; i < n; i++) if (z[i] > mx) mx = z[i];
    float se = 0.0f;
    for (int i = 0; i < n; i++) se += expf(z[i] - mx);
    float inv = 1.0f / se, sy = 0.0f;
    for (int i = 0; i < n; i++) sy += t[i];
    if (sy == 0.0f) sy = 1.0f;
    for (int i = 0; i < n; i++) dz[i] = expf(z[i] - mx) * inv * sy - t[i];
}

/* ------------------------------------------------------------------ optimizer, pooling, helpers */

/* [ref: lib/sources/pulp_optimizers_fp32.c:48-62] weight decay rewrites the gradient in place. */
void orc_sgd(float *w, float *g, long n, float lr, float lambda)
{
    for (long i = 0; i < n; i++) {
        if (lambda != 0) g[i] += lambda * w[i];
        w[i] -= lr * g[i];
    }
}
/* [ref: lib/sources/pulp_pooling_fp32.c:24-66] */
void orc_avgpool_fw(const float *x, float *y, int C, int H, int W, int Hk, int Wk, int sh, int sw)
{
    const int Ho = (H - Hk + sh) / sh, Wo = (W - Wk + sw) / sw;
    for (int k = 0; k < C; k++)
        for (int ha = 0; ha < Ho; ha++)
            for (int wa = 0; wa < Wo; wa++) {
                float s = 0;
                for (int hk = 0; hk < Hk; hk++) for (int wk = 0; wk < Wk; wk++) s += x[wk + wa * sw + (hk + ha * sh) * W + k * H * W];
                y[wa + ha * Wo + k * Ho * Wo] = s / (Hk * Wk);
            }
}
/* [ref: lib/sources/pulp_pooling_fp32.c:69-115] */
void orc_avgpool_bw(const float *dy, float *dx, int C, int H, int W, int Hk, int Wk, int sh, int sw)
{
    const int Ho = (H - Hk + sh) / sh, Wo = (W - Wk + sw) / sw;
    for (long i = 0; i < (long)C * H * W; i++) dx[i] = 0;
    for (int k = 0; k < C; k++)
        for (int ho = 0; ho < Ho; ho++)
            for (int wo = 0; wo < Wo; wo++)
                for (int ha = 0; ha < Hk; ha++)
                    for (int wa = 0; wa < Wk; wa++)
                        dx[(wa + wo * sw) + (ha + ho * sh) * W + k * H * W] += dy[wo + ho * Wo + k * Ho * Wo] / (Hk * Wk);
}
/* [ref: lib/sources/pulp_train_utils_fp32.c:79-185] out = in.transpose(axes) */
void orc_transpose(const float *in, float *out, const int *dims, const int *axes, int nd)
{
    long total = 1, in_stride[8], out_dims[8], src_stride[8];
    for (int i = nd - 1; i >= 0; i--) { in_stride[i] = total; total *= dims[i]; }
    for (int i = 0; i < nd; i++) { out_dims[i] = dims[axes[i]]; src_stride[i] = in_stride[axes[i]]; }
    for (long e = 0; e < total; e++) {
        long rem = e, src = 0;
        for (int k = nd - 1; k >= 0; k--) { src += (rem % out_dims[k]) * src_stride[k]; rem /= out_dims[k]; }
        out[e] = in[src];
    }
}
/* [ref: lib/sources/pulp_train_utils_fp32.c:225-806] NumPy-style broadcast add */
void orc_broadcast_add(const float *a, const float *b, float *c, const int *da, int na, const int *db, int nb)
{
    int n = na > nb ? na : nb;
    long d[8], sa[8], sb[8], total = 1, stra = 1, strb = 1;
    for (int k = 0; k < n; k++) {
        int ea = k < na ? da[na - 1 - k] : 1, eb = k < nb ? db[nb - 1 - k] : 1, e = ea > eb ? ea : eb;
        d[n - 1 - k] = e; sa[n - 1 - k] = ea == 1 ? 0 : stra; sb[n - 1 - k] = eb == 1 ? 0 : strb;
        stra *= ea; strb *= eb; total *= e;
    }
    for (long e = 0; e < total; e++) {
        long rem = e, ia = 0, ib = 0;
        for (int k = n - 1; k >= 0; k--) { long qq = rem % d[k]; ia += qq * sa[k]; ib += qq * sb[k]; rem /= d[k]; }
        c[e] = a[ia] + b[ib];
    }
}
/* [ref: lib/sources/pulp_train_utils_fp32.c:929-988] geometric zero test (the reference's
 * `wt > W` is equivalent only for left/up pad 1). */
void orc_pad(const float *src, float *dst, int C, int H, int W, int padL, int padR, int padU, int padD, int hwc)
{
    const int Ho = H + padU + padD, Wo = W + padL + padR;
    for (int c = 0; c < C; c++)
        for (int ht = 0; ht < Ho; ht++)
            for (int wt = 0; wt < Wo; wt++) {
                int hs = ht - padU, ws = wt - padL;
                int inside = hs >= 0 && hs < H && ws >= 0 && ws < W;
                long o = hwc ? ((long)ht * Wo + wt) * C + c : ((long)c * Ho + ht) * Wo + wt;
                long i = hwc ? ((long)hs * W + ws) * C + c : ((long)c * H + hs) * W + ws;
                dst[o] = inside ? src[i] : 0;
            }
}
