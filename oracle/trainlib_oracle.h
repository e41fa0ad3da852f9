/*
 * trainlib_oracle.h - prototypes of the CPU restatement in trainlib_oracle.c.
 * TEST INFRASTRUCTURE ONLY (checker for tests, the smoke run and the bench's CPU leg);
 * nothing in the product includes this file.  See trainlib_oracle.c for the reference
 * routine each function restates.
 */
#ifndef TRAINLIB_ORACLE_H
#define TRAINLIB_ORACLE_H
#ifdef __cplusplus
extern "C" {
#endif

float orc_fastexp_gist(float x);
float orc_q_rsqrt(float number);
void orc_mm(const float *A, const float *B, float *C, int N, int K, int M, int trans_B, int accumulate);
void orc_im2row(const float *src, float *buf, int C, int H, int W, int Hk, int Wk, int Ho, int Wo, int sh, int sw, int padU, int padL, int mode_ig, int hwc, int transposed);
void orc_blocktransp(const float *w, float *bt, int Cin, int Cout, int Hk, int Wk, int hwc);
void orc_conv2d_fw(const float *x, const float *w, const float *bias, float *y, int Cin, int Hin, int Win, int Cout, int Hk, int Wk, int sh, int sw, int padU, int padD, int padL, int padR);
void orc_conv2d_wg(const float *x, const float *dy, float *dw, float *dbias, int Cin, int Hin, int Win, int Cout, int Hk, int Wk, int sh, int sw, int padU, int padD, int padL, int padR);
void orc_conv2d_ig(const float *dy, const float *w, float *dx, int Cin, int Hin, int Win, int Cout, int Hk, int Wk, int sh, int sw, int padU, int padD, int padL, int padR);
void orc_dw_fw(const float *x, const float *w, float *y, int C, int Hin, int Win, int Hk, int Wk, int sh, int sw, int padU, int padD, int padL, int padR);
void orc_dw_wg(const float *x, const float *dy, float *dw, int C, int Hin, int Win, int Hk, int Wk, int sh, int sw, int padU, int padD, int padL, int padR);
void orc_dw_ig(const float *dy, const float *w, float *dx, int C, int Hin, int Win, int Hk, int Wk, int sh, int sw, int padU, int padD, int padL, int padR);
void orc_linear_fw(const float *W, const float *x, const float *bias, float *y, int out, int in);
void orc_linear_wg(const float *dy, const float *x, float *dW, float *dbias, int out, int in);
void orc_linear_ig(const float *dy, const float *W, float *dx, int out, int in);
void orc_softmax_fw(const float *in, float *out, int rows, int width);
void orc_softmax_bw(const float *out, const float *dout, float *din, int rows, int width);
void orc_mhsa_fw(const float *x, const float *wq, const float *wk, const float *wv, const float *bq, const float *bk, const float *bv, const float *wo, float *q, float *k, float *v, float *softmax, float *att, float *y, int L, int E, int F, int heads);
void orc_mhsa_bw(const float *x, const float *wq, const float *wk, const float *wv, const float *wo, const float *q, const float *k, const float *v, const float *softmax, const float *att, const float *dy, float *dq, float *dk, float *dv, float *dsoftmax, float *datt, float *dwq, float *dwk, float *dwv, float *dwo, float *dx, int L, int E, int F, int heads);
void orc_mhsa_mobilebert_fw(const float *x, const float *xb, const float *wq, const float *wk, const float *wv, const float *bq, const float *bk, const float *bv, const float *wo, const float *bo, float *q, float *k, float *v, float *softmax, float *att, float *y, int L, int E, int Kb, int F, int No, int heads);
void orc_mhsa_mobilebert_bw(const float *x, const float *xb, const float *wq, const float *wk, const float *wv, const float *wo, const float *q, const float *k, const float *v, const float *softmax, const float *att, const float *dy, float *dq, float *dk, float *dv, float *dsoftmax, float *datt, float *dwq, float *dwk, float *dwv, float *dwo, float *dx, float *dxb, int L, int E, int Kb, int F, int No, int heads);
void orc_act_fw(int kind, const float *x, float *y, long n, float slope);
void orc_act_bw(int kind, const float *x, const float *y, const float *dy, float *dx, long n, float slope);
void orc_instnorm_fw(const float *x, float *y, const float *gb, float *mean, float *var, float *stdev, int C, int D);
void orc_instnorm_bw_input(const float *x, const float *dy, float *dx, const float *gb, const float *mean, const float *var, const float *stdev, int C, int D);
void orc_instnorm_bw_param(const float *x, const float *dy, float *dgb, const float *mean, const float *stdev, int C, int D);
void orc_batchnorm_fw(const float *x, float *y, const float *w, const float *b, int B, int C, int HW, float eps);
void orc_layernorm_fw(const float *x, float *y, const float *w, const float *b, int rows, int width, float eps);
void orc_mm_broadcast(const float *A, const float *B, float *C, const int *a_dims, int a_len, const int *b_dims, int b_len);
void orc_layernorm_bw(const float *x, const float *w, const float *dy, float *dx, float *dw, float *db, int rows, int width, float eps);
float orc_mse_fw(const float *y, const float *t, int n);
void orc_mse_bw(const float *y, const float *t, float *dy, int n);
float orc_ce_fw(const float *z, const float *t, int n);
void orc_ce_bw(const float *z, const float *t, float *dz, int n);
void orc_sgd(float *w, float *g, long n, float lr, float lambda);
void orc_avgpool_fw(const float *x, float *y, int C, int H, int W, int Hk, int Wk, int sh, int sw);
void orc_avgpool_bw(const float *dy, float *dx, int C, int H, int W, int Hk, int Wk, int sh, int sw);
void orc_transpose(const float *in, float *out, const int *dims, const int *axes, int nd);
void orc_broadcast_add(const float *a, const float *b, float *c, const int *da, int na, const int *db, int nb);
void orc_pad(const float *src, float *dst, int C, int H, int W, int padL, int padR, int padU, int padD, int hwc);

#ifdef __cplusplus
}
#endif
#endif
