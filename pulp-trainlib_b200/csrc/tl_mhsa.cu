// Multi-head self-attention, forward and backward, composed from strided GEMMs and the row
// softmax kernels.  The reference materialises eight transposes per pass
// [ref: lib/sources/pulp_mhsa_fp32.c:20-644 (FW), :648-1745 (BW)]; here every transposed
// operand is expressed through GEMM strides and the per-head products run as one batched launch.
//
// Layouts (reference convention): x, y are E x L (token index fastest); Wq/Wk/Wv/Wo are E x F;
// q, k, v, att are F x L; softmax is heads x L x L indexed [head][query][key].
#include "tl_kernels.h"

namespace tl {

// 32-bit restatement of the reference's fast inverse square root (one Newton step)
// [ref: lib/sources/pulp_train_utils_fp32.c:1234-1247; the `long` pun there is 64-bit on LP64].
static float q_rsqrt_host(float number)
{
    union { float f; int32_t i; } u;
    float x2 = number * 0.5f;
    u.f = number;
    u.i = 0x5f3759df - (u.i >> 1);
    return u.f * (1.5f - (x2 * u.f * u.f));
}

template <class T>
void mhsa_fw(Scope &sc, const MhsaDims &d, const T *x, const T *wq, const T *wk, const T *wv,
             const T *bq, const T *bk, const T *bv, const T *wo,
             T *q, T *k, T *v, T *softmax, T *att, T *y)
{
    const int L = d.L, E = d.E, F = d.F, NH = d.heads, H = F / NH;
    const float scaling = q_rsqrt_host((float)H);

    // projections: q = Wq^T x (+ bq per row)  [ref: pulp_mhsa_fp32.c:87-158 and twins for k, v]
    // the three are one launch (separate allocations, one shape): 192 tiles instead of three times 64 on 148 SMs
    {
        GemmDesc<T> g;
        g.a_rs = 1; g.a_cs = F; g.b_rs = L; g.b_cs = 1; g.c_rs = L;
        g.N = F; g.K = E; g.M = L; g.bias_mode = 1;
        const GemmList<T> l = {{wq, wk, wv}, {x, x, x}, {bq, bk, bv}, {q, k, v}};
        gemm_list<T>(g, l, 3);
    }
    if (attn_fused_ok(L, H) && gemm_path() != 1) {
        // scores, softmax and the product with v in one kernel per (head, query tile)   [ref: :348-560]
        attn_fw<T>(q, k, v, softmax, att, L, H, NH, scaling);
        mm_contract<T>(wo, att, y, E, F, L, 0, false);
        return;
    }
    // scores[h][query][key] = scaling * sum_d q[h,d,query] k[h,d,key]   [ref: :348-431]
    T *scores = sc.scratch<T>((size_t)NH * L * L);
    if (!scores) return;
    {
        GemmDesc<T> g;
        g.A = q; g.a_rs = 1; g.a_cs = L; g.a_bs = (long long)H * L;
        g.B = k; g.b_rs = L; g.b_cs = 1; g.b_bs = (long long)H * L;
        g.C = scores; g.c_rs = L; g.c_bs = (long long)L * L;
        g.N = L; g.K = H; g.M = L; g.batch = NH; g.alpha = scaling;
        gemm<T>(g);
    }
    // softmax over keys   [ref: :464-491]
    softmax_fw<T>(scores, softmax, (T *)nullptr, (T *)nullptr, L, L, NH);
    // att[h,d,query] = sum_key v[h,d,key] P[h,query,key]   [ref: :530-560]
    {
        GemmDesc<T> g;
        g.A = v; g.a_rs = L; g.a_cs = 1; g.a_bs = (long long)H * L;
        g.B = softmax; g.b_rs = 1; g.b_cs = L; g.b_bs = (long long)L * L;
        g.C = att; g.c_rs = L; g.c_bs = (long long)H * L;
        g.N = H; g.K = L; g.M = L; g.batch = NH;
        gemm<T>(g);
    }
    // y = Wo att   [ref: :612]
    mm_contract<T>(wo, att, y, E, F, L, 0, false);
}

template <class T>
void mhsa_bw(Scope &sc, const MhsaDims &d, const T *x, const T *wq, const T *wk, const T *wv,
             const T *wo, const T *q, const T *k, const T *v, const T *softmax, const T *att,
             const T *dy, T *dq, T *dk, T *dv, T *dsoftmax, T *datt, T *grad_scratch,
             T *dwq, T *dwk, T *dwv, T *dwo, T *dx)
{
    (void)grad_scratch;
    const int L = d.L, E = d.E, F = d.F, NH = d.heads, H = F / NH;
    const float scaling = q_rsqrt_host((float)H);
    const long long HL = (long long)H * L, LL = (long long)L * L;

    // dWo = dY att^T   [ref: pulp_mhsa_fp32.c:704-760]
    { GemmDesc<T> g; g.A = dy; g.a_rs = L; g.B = att; g.b_rs = 1; g.b_cs = L; g.C = dwo; g.c_rs = F; g.N = E; g.K = L; g.M = F; gemm<T>(g); }
    // datt = Wo^T dY   [ref: :783-837]
    { GemmDesc<T> g; g.A = wo; g.a_rs = 1; g.a_cs = F; g.B = dy; g.b_rs = L; g.C = datt; g.c_rs = L; g.N = F; g.K = E; g.M = L; gemm<T>(g); }
    const bool fused = attn_fused_ok(L, H) && gemm_path() != 1;
    if (fused) {
        // dP, dS (never stored), dq, dk, dv in two kernels   [ref: :842-1400]
        float *rowdot = sc.scratch<float>((size_t)NH * L);
        if (!rowdot) return;
        attn_bw<T>(datt, q, k, v, softmax, dsoftmax, rowdot, dq, dk, dv, L, H, NH, scaling);
    }
    else {
    // dv[h,d,key] = sum_query datt[h,d,query] P[h,query,key]   [ref: :842-895]
    { GemmDesc<T> g; g.A = datt; g.a_rs = L; g.a_bs = HL; g.B = softmax; g.b_rs = L; g.b_bs = LL; g.C = dv; g.c_rs = L; g.c_bs = HL;
      g.N = H; g.K = L; g.M = L; g.batch = NH; gemm<T>(g); }
    // dP[h,query,key] = sum_d datt[h,d,query] v[h,d,key]   [ref: :923-1050, with the corrected V transpose]
    { GemmDesc<T> g; g.A = datt; g.a_rs = 1; g.a_cs = L; g.a_bs = HL; g.B = v; g.b_rs = L; g.b_bs = HL; g.C = dsoftmax; g.c_rs = L; g.c_bs = LL;
      g.N = L; g.K = H; g.M = L; g.batch = NH; gemm<T>(g); }
    // dS = softmax backward   [ref: :1052-1100]
    T *dS = sc.scratch<T>((size_t)NH * LL);
    if (!dS) return;
    softmax_bw<T>(softmax, dsoftmax, dS, (T *)nullptr, L, L, NH);
    // dk[h,d,key] = scaling * sum_query q[h,d,query] dS[h,query,key]   [ref: :1140-1330]
    { GemmDesc<T> g; g.A = q; g.a_rs = L; g.a_bs = HL; g.B = dS; g.b_rs = L; g.b_bs = LL; g.C = dk; g.c_rs = L; g.c_bs = HL;
      g.N = H; g.K = L; g.M = L; g.batch = NH; g.alpha = scaling; gemm<T>(g); }
    // dq[h,d,query] = scaling * sum_key k[h,d,key] dS[h,query,key]   [ref: :1340-1400]
    { GemmDesc<T> g; g.A = k; g.a_rs = L; g.a_bs = HL; g.B = dS; g.b_rs = 1; g.b_cs = L; g.b_bs = LL; g.C = dq; g.c_rs = L; g.c_bs = HL;
      g.N = H; g.K = L; g.M = L; g.batch = NH; g.alpha = scaling; gemm<T>(g); }
    }
    // projection weight grads, stored F x E: dW = dproj x^T   [ref: :1426-1600]
    const T *dps[3] = {dq, dk, dv}; const T *ws[3] = {wq, wk, wv};
    {
        GemmDesc<T> g; g.a_rs = L; g.b_rs = 1; g.b_cs = L; g.c_rs = E; g.N = F; g.K = L; g.M = E;                // one launch for the three
        const GemmList<T> l = {{dq, dk, dv}, {x, x, x}, {nullptr, nullptr, nullptr}, {dwq, dwk, dwv}};
        gemm_list<T>(g, l, 3);
    }
    // dx += Wq dq + Wk dk + Wv dv (the caller zeroes dx; same order as the reference)   [ref: :1605-1745]
    for (int p = 0; p < 3; p++) {
        GemmDesc<T> g; g.A = ws[p]; g.a_rs = F; g.B = dps[p]; g.b_rs = L; g.C = dx; g.c_rs = L; g.N = E; g.K = F; g.M = L; g.accumulate = true;
        gemm<T>(g);
    }
}

// Attention of the MobileBERT encoder block: token-major activations (x: L x E, bottleneck input xb: L x Kb, output
// y: L x No), row-major weights (Wq, Wk: F x Kb; Wv: F x E; Wo: No x F), a bias on every projection
// [ref: lib/sources/pulp_mhsa_fp32.c:1749-2035; :2162-2412 is the same arithmetic cut into DMA tiles].  q, k, v, att
// and the probabilities keep the layouts of the training path, so the attention core is the same fused kernel; the
// reference's final transpose is the output stride of the last GEMM.
template <class T>
void mhsa_mobilebert_fw(Scope &sc, const MobileBertDims &d, const T *x, const T *xb, const T *wq, const T *wk, const T *wv,
                        const T *bq, const T *bk, const T *bv, const T *wo, const T *bo,
                        T *q, T *k, T *v, T *softmax, T *att, T *y)
{
    const int L = d.L, E = d.E, Kb = d.Kb, F = d.F, No = d.No, NH = d.heads, H = F / NH;
    const float scaling = q_rsqrt_host((float)H);
    const T *ws[3] = {wq, wk, wv}; const T *bs[3] = {bq, bk, bv}; T *outs[3] = {q, k, v};
    for (int p = 0; p < 3; p++) {
        const int K = p == 2 ? E : Kb;
        GemmDesc<T> g;
        g.A = ws[p]; g.a_rs = K; g.a_cs = 1;
        g.B = p == 2 ? x : xb; g.b_rs = 1; g.b_cs = K;
        g.C = outs[p]; g.c_rs = L;
        g.N = F; g.K = K; g.M = L;
        if (bs[p]) { g.bias = bs[p]; g.bias_mode = 1; }
        gemm<T>(g);
    }
    if (attn_fused_ok(L, H) && gemm_path() != 1) attn_fw<T>(q, k, v, softmax, att, L, H, NH, scaling);
    else {
        T *scores = sc.scratch<T>((size_t)NH * L * L);
        if (!scores) return;
        { GemmDesc<T> g; g.A = q; g.a_rs = 1; g.a_cs = L; g.a_bs = (long long)H * L; g.B = k; g.b_rs = L; g.b_cs = 1; g.b_bs = (long long)H * L;
          g.C = scores; g.c_rs = L; g.c_bs = (long long)L * L; g.N = L; g.K = H; g.M = L; g.batch = NH; g.alpha = scaling; gemm<T>(g); }
        softmax_fw<T>(scores, softmax, (T *)nullptr, (T *)nullptr, L, L, NH);
        { GemmDesc<T> g; g.A = v; g.a_rs = L; g.a_cs = 1; g.a_bs = (long long)H * L; g.B = softmax; g.b_rs = 1; g.b_cs = L; g.b_bs = (long long)L * L;
          g.C = att; g.c_rs = L; g.c_bs = (long long)H * L; g.N = H; g.K = L; g.M = L; g.batch = NH; gemm<T>(g); }
    }
    // y[l][n] = sum_f Wo[n][f] att[f][l] + bo[n]
    { GemmDesc<T> g; g.A = wo; g.a_rs = F; g.a_cs = 1; g.B = att; g.b_rs = L; g.b_cs = 1; g.C = y; g.c_rs = 1; g.c_cs = No;
      g.N = No; g.K = F; g.M = L; if (bo) { g.bias = bo; g.bias_mode = 1; } gemm<T>(g); }
}

// Gradient of the forward above in the forward's own layouts: dy is L x No; dWq, dWk: F x Kb; dWv: F x E; dWo: No x F;
// dx (L x E) and dxb (L x Kb) are added to what the caller's buffers hold, as the reference's backward does for its
// input gradient [ref: lib/sources/pulp_mhsa_fp32.c:2413-2840, which reads output.diff as E x L although the forward
// writes the output as L x No: only consistent for square shapes, where both give these formulas].
template <class T>
void mhsa_mobilebert_bw(Scope &sc, const MobileBertDims &d, const T *x, const T *xb, const T *wq, const T *wk, const T *wv, const T *wo,
                        const T *q, const T *k, const T *v, const T *softmax, const T *att, const T *dy,
                        T *dq, T *dk, T *dv, T *dsoftmax, T *datt, T *dwq, T *dwk, T *dwv, T *dwo, T *dx, T *dxb)
{
    const int L = d.L, E = d.E, Kb = d.Kb, F = d.F, No = d.No, NH = d.heads, H = F / NH;
    const float scaling = q_rsqrt_host((float)H);
    const long long HL = (long long)H * L, LL = (long long)L * L;
    // dWo[n][f] = sum_l dy[l][n] att[f][l];  datt[f][l] = sum_n Wo[n][f] dy[l][n]
    { GemmDesc<T> g; g.A = dy; g.a_rs = 1; g.a_cs = No; g.B = att; g.b_rs = 1; g.b_cs = L; g.C = dwo; g.c_rs = F; g.N = No; g.K = L; g.M = F; gemm<T>(g); }
    { GemmDesc<T> g; g.A = wo; g.a_rs = 1; g.a_cs = F; g.B = dy; g.b_rs = 1; g.b_cs = No; g.C = datt; g.c_rs = L; g.N = F; g.K = No; g.M = L; gemm<T>(g); }
    if (attn_fused_ok(L, H) && gemm_path() != 1) {
        float *rowdot = sc.scratch<float>((size_t)NH * L);
        if (!rowdot) return;
        attn_bw<T>(datt, q, k, v, softmax, dsoftmax, rowdot, dq, dk, dv, L, H, NH, scaling);
    } else {
        { GemmDesc<T> g; g.A = datt; g.a_rs = L; g.a_bs = HL; g.B = softmax; g.b_rs = L; g.b_bs = LL; g.C = dv; g.c_rs = L; g.c_bs = HL;
          g.N = H; g.K = L; g.M = L; g.batch = NH; gemm<T>(g); }
        { GemmDesc<T> g; g.A = datt; g.a_rs = 1; g.a_cs = L; g.a_bs = HL; g.B = v; g.b_rs = L; g.b_bs = HL; g.C = dsoftmax; g.c_rs = L; g.c_bs = LL;
          g.N = L; g.K = H; g.M = L; g.batch = NH; gemm<T>(g); }
        T *dS = sc.scratch<T>((size_t)NH * LL);
        if (!dS) return;
        softmax_bw<T>(softmax, dsoftmax, dS, (T *)nullptr, L, L, NH);
        { GemmDesc<T> g; g.A = q; g.a_rs = L; g.a_bs = HL; g.B = dS; g.b_rs = L; g.b_bs = LL; g.C = dk; g.c_rs = L; g.c_bs = HL;
          g.N = H; g.K = L; g.M = L; g.batch = NH; g.alpha = scaling; gemm<T>(g); }
        { GemmDesc<T> g; g.A = k; g.a_rs = L; g.a_bs = HL; g.B = dS; g.b_rs = 1; g.b_cs = L; g.b_bs = LL; g.C = dq; g.c_rs = L; g.c_bs = HL;
          g.N = H; g.K = L; g.M = L; g.batch = NH; g.alpha = scaling; gemm<T>(g); }
    }
    const T *dps[3] = {dq, dk, dv}; T *dws[3] = {dwq, dwk, dwv}; const T *ws[3] = {wq, wk, wv};
    for (int p = 0; p < 3; p++) {
        const int K = p == 2 ? E : Kb;
        // dW[f][c] = sum_l dproj[f][l] in[l][c]
        { GemmDesc<T> g; g.A = dps[p]; g.a_rs = L; g.a_cs = 1; g.B = p == 2 ? x : xb; g.b_rs = K; g.b_cs = 1; g.C = dws[p]; g.c_rs = K; g.N = F; g.K = L; g.M = K; gemm<T>(g); }
        // din[l][c] += sum_f dproj[f][l] W[f][c]
        T *din = p == 2 ? dx : dxb;
        if (din) { GemmDesc<T> g; g.A = dps[p]; g.a_rs = 1; g.a_cs = L; g.B = ws[p]; g.b_rs = K; g.b_cs = 1; g.C = din; g.c_rs = K; g.N = L; g.K = F; g.M = K; g.accumulate = true; gemm<T>(g); }
    }
}

#define INST(T)                                                                                                        \
    template void mhsa_fw<T>(Scope &, const MhsaDims &, const T *, const T *, const T *, const T *, const T *, const T *, \
                             const T *, const T *, T *, T *, T *, T *, T *, T *);                                      \
    template void mhsa_bw<T>(Scope &, const MhsaDims &, const T *, const T *, const T *, const T *, const T *, const T *, \
                             const T *, const T *, const T *, const T *, const T *, T *, T *, T *, T *, T *, T *, T *, T *, T *, T *, T *);
INST(float)
INST(__half)
#undef INST
#define INST(T)                                                                                                        \
    template void mhsa_mobilebert_fw<T>(Scope &, const MobileBertDims &, const T *, const T *, const T *, const T *, const T *, const T *, \
                                        const T *, const T *, const T *, const T *, T *, T *, T *, T *, T *, T *);       \
    template void mhsa_mobilebert_bw<T>(Scope &, const MobileBertDims &, const T *, const T *, const T *, const T *, const T *, const T *, \
                                        const T *, const T *, const T *, const T *, const T *, const T *, T *, T *, T *, T *, T *, T *, T *, T *, T *, T *, T *);
INST(float)
INST(__half)

} // namespace tl
