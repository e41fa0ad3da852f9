// Entry points of the rest of the element-wise family: L1 / berHu losses, max pooling, NoNorm, RMS norm, SwiGLU, the
// vector softmax and the per-row pieces of the reference's softmax, with their fp16 twins.  Same conventions as the
// other entry points: host pointers are staged, device pointers pass through, errors latch.
#include "tl_kernels.h"
#include <cmath>
#include <cstdio>

using namespace tl;

namespace {

#define TL_REQUIRE(cond, ...)                                        \
    do { if (!(cond)) { set_error(TL_ERR_BAD_ARGS, __VA_ARGS__); return; } } while (0)

inline float f(float v) { return v; }
inline float f(__half v) { return __half2float(v); }

// L1 (kind 0) and berHu (kind 1); loss_args and berHu_loss_args share their first three fields
template <class T, class A> void l1_impl(void *args, bool berhu, float alpha, int backward)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->output, "loss: null arguments");
    const int dim = a->output->dim, n = streams();
    TL_REQUIRE(dim > 0, "loss: empty output");
    Scope sc;
    const T *y = (const T *)sc.in((T *)a->output->data, (size_t)n * dim), *t = (const T *)sc.in((T *)a->target, (size_t)n * dim);
    if (!backward) {
        T *loss = sc.out((T *)a->wr_loss, (size_t)n);
        if (sc.ok()) l1_fw<T>(y, t, loss, dim, n, berhu, alpha);
    } else {
        T *dy = sc.out((T *)a->output->diff, (size_t)n * dim);
        if (sc.ok()) l1_bw<T>(y, t, dy, dim, n, berhu, alpha);
    }
}

template <class T, class A> void maxpool_impl(void *args, int backward)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->input && a->output, "pulp_maxpool: null arguments");
    const int C = a->input->C, H = a->input->H, W = a->input->W, Ho = a->output->H, Wo = a->output->W, n = streams();
    TL_REQUIRE(a->Hstride >= 1 && a->Wstride >= 1 && a->Hker >= 1 && a->Wker >= 1 && a->Hker <= H && a->Wker <= W, "pulp_maxpool: kernel/stride out of range");
    // the reference's own size check, its Hstride in the width formula included [ref: lib/sources/pulp_pooling_fp32.c:139-141]
    if ((H - a->Hker + a->Hstride) / a->Hstride != Ho || (W - a->Wker + a->Hstride) / a->Wstride != Wo) {
        printf("\n[pulp_maxpool] Invalid pooling kernel size or output size!\n");
        set_error(TL_ERR_BAD_ARGS, "pulp_maxpool: output %dx%d does not match kernel/stride", Ho, Wo);
        return;
    }
    TL_REQUIRE((Ho - 1) * a->Hstride + a->Hker <= H && (Wo - 1) * a->Wstride + a->Wker <= W, "pulp_maxpool: windows leave the input");
    Scope sc;
    const size_t nx = (size_t)n * C * H * W, ny = (size_t)n * C * Ho * Wo;
    const T *x = (const T *)sc.in((T *)a->input->data, nx);
    if (!backward) { T *y = sc.out((T *)a->output->data, ny); if (sc.ok()) maxpool_fw<T>(x, y, (long long)n * C, H, W, Ho, Wo, a->Hker, a->Wker, a->Hstride, a->Wstride); }
    else { const T *dy = (const T *)sc.in((T *)a->output->diff, ny); T *dx = sc.out((T *)a->input->diff, nx);
           if (sc.ok()) maxpool_bw<T>(x, dy, dx, (long long)n * C, H, W, Ho, Wo, a->Hker, a->Wker, a->Hstride, a->Wstride); }
}

template <class T, class A> void nonorm_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->input && a->coeff && a->bias && a->output, "pulp_nonorm: null arguments");
    const int rows = a->input->H, width = a->input->W;
    TL_REQUIRE(rows > 0 && width > 0, "pulp_nonorm: H=%d W=%d", rows, width);
    Scope sc;
    const size_t n = (size_t)rows * width;
    const T *x = (const T *)sc.in((T *)a->input->data, n), *w = (const T *)sc.in((T *)a->coeff->data, (size_t)width), *b = (const T *)sc.in((T *)a->bias->data, (size_t)width);
    T *y = sc.out((T *)a->output->data, n);
    if (sc.ok()) nonorm_fw<T>(x, w, b, y, rows, width);
}

template <class T, class A> void wscale_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->size > 0, "weighted_scaling: empty");
    Scope sc;
    const size_t n = a->size;
    const T *x = (const T *)sc.in((T *)a->in, n), *w = (const T *)sc.in((T *)a->w, n);
    T *y = sc.out((T *)a->out, n);
    if (sc.ok()) weighted_scaling<T>(x, w, y, (long long)n, f(a->scaling_factor), (const T *)nullptr);
}
template <class T, class A> void sumsq_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->size > 0, "sum_of_squares: empty");
    Scope sc;
    const T *x = (const T *)sc.in((T *)a->in, (size_t)a->size);
    T *o = sc.out((T *)a->out, 1);
    if (sc.ok()) sum_of_squares<T>(x, o, (long long)a->size);
}
// o = weight * x / sqrt(mean(x^2) + 1e-5); buffer_n_cores[0] receives the sum of squares [ref: lib/sources/pulp_rmsnorm_fp32.c:29-60]
template <class T> void rmsnorm_impl(T *o, T *x, T *weight, T *buffer, int size)
{
    TL_REQUIRE(o && x && weight && buffer && size > 0, "rmsnorm_parallelized: bad arguments");
    Scope sc;
    const T *xs = (const T *)sc.in(x, (size_t)size), *w = (const T *)sc.in(weight, (size_t)size);
    T *buf = sc.out(buffer, 1), *y = sc.out(o, (size_t)size);
    if (!sc.ok()) return;
    sum_of_squares<T>(xs, buf, size);
    weighted_scaling<T>(xs, w, y, size, 0.f, buf);
}
template <class T, class A> void swiglu_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->dim > 0, "pulp_swiglu: empty");
    Scope sc;
    const T *p = (const T *)sc.in((T *)a->in1, (size_t)a->dim), *q = (const T *)sc.in((T *)a->in2, (size_t)a->dim);
    T *y = sc.out((T *)a->out, (size_t)a->dim);
    if (sc.ok()) swiglu<T>(p, q, y, a->dim);
}
template <class T> void vsoftmax_impl(T *out, T *in, unsigned int size)
{
    TL_REQUIRE(out && in && size > 0, "pulp_vector_softmax: bad arguments");
    Scope sc;
    const T *x = (const T *)sc.in(in, (size_t)size);
    T *y = sc.out(out, (size_t)size);
    if (sc.ok()) vector_softmax<T>(x, y, size);
}
template <class T, class A> void vmax_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->W > 0, "pulp_max: W must be positive");
    Scope sc;
    const T *x = (const T *)sc.in((T *)a->input, (size_t)a->W);
    T *m = sc.out((T *)a->maxes, 1);
    if (sc.ok()) vec_max<T>(x, m, a->W);
}
template <class T, class A> void vdiv_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->dim > 0, "pulp_div: empty");
    Scope sc;
    T *io = sc.inout((T *)a->input, (size_t)a->dim);
    if (sc.ok()) vec_div<T>(io, a->dim, f(a->n));
}
template <class T, class A> void vexpsum_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->dim > 0, "vector_exp_sum: empty");
    Scope sc;
    const T *x = (const T *)sc.in((T *)a->input, (size_t)a->dim);
    T *y = sc.out((T *)a->output, (size_t)a->dim), *s = sc.out((T *)a->sums, 1);
    if (sc.ok()) vec_exp_sum<T>(x, y, s, a->dim, f(a->max));
}
template <class T, class A> void op1_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->H > 0 && a->W > 0, "pulp_sm_bw_op_1: H and W must be positive");
    Scope sc;
    const size_t n = (size_t)a->H * a->W;
    const T *A_ = (const T *)sc.in((T *)a->A, n), *B_ = (const T *)sc.in((T *)a->B, n);
    T *S = sc.out((T *)a->S, (size_t)a->H);
    if (sc.ok()) sm_bw_op1<T>(A_, B_, S, a->H, a->W);
}
template <class T, class A> void op2_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->H > 0 && a->W > 0, "pulp_sm_bw_op_2: H and W must be positive");
    Scope sc;
    const size_t n = (size_t)a->H * a->W;
    const T *A_ = (const T *)sc.in((T *)a->A, n), *B_ = (const T *)sc.in((T *)a->B, n), *S = (const T *)sc.in((T *)a->S, (size_t)a->H);
    T *o = sc.out((T *)a->output, n);
    if (sc.ok()) sm_bw_op2<T>(A_, B_, S, o, a->H, a->W);
}
template <class T, class A> void rowmax16_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->H > 0 && a->W > 0, "pulp_row_max: H=%d W=%d", a->H, a->W);
    Scope sc;
    const T *in = (const T *)sc.in((T *)a->input, (size_t)a->H * a->W); T *mx = sc.inout((T *)a->maxes, (size_t)a->H);
    if (sc.ok()) row_max<T>(in, mx, a->H, a->W);
}
template <class T, class A> void expsum16_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->H > 0 && a->W > 0, "pulp_exp_sum: H=%d W=%d", a->H, a->W);
    Scope sc;
    const size_t n = (size_t)a->H * a->W;
    const T *in = (const T *)sc.in((T *)a->input, n), *mx = (const T *)sc.in((T *)a->maxes, (size_t)a->H);
    T *out = sc.out((T *)a->output, n), *sm = sc.inout((T *)a->sums, (size_t)a->H);
    if (sc.ok()) exp_sum<T>(in, out, mx, sm, a->H, a->W);
}
template <class T, class A> void rowdiv16_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->H > 0 && a->W > 0, "pulp_row_div: H=%d W=%d", a->H, a->W);
    Scope sc;
    T *io = sc.inout((T *)a->input, (size_t)a->H * a->W); const T *sm = (const T *)sc.in((T *)a->sums, (size_t)a->H);
    if (sc.ok()) row_div<T>(io, sm, a->H, a->W);
}
template <class T, class A> void meanstd16_impl(void *args)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->dim > 0, "pulp_mean_std: dim=%d", a->dim);
    Scope sc;
    const T *x = (const T *)sc.in((T *)a->input, (size_t)a->dim);
    T *m = sc.out((T *)a->mean, 1), *v = sc.out((T *)a->var, 1), *s = sc.out((T *)a->std, 1);
    if (sc.ok()) mean_std<T>(x, m, v, s, a->dim, f(a->epsilon));
}

} // namespace

#define TL_EXPORT extern "C" __attribute__((visibility("default")))
typedef __half H;

TL_EXPORT void pulp_L1Loss(void *a) { l1_impl<float, loss_args>(a, false, 0.f, 0); }
TL_EXPORT void pulp_L1Loss_backward(void *a) { l1_impl<float, loss_args>(a, false, 0.f, 1); }
TL_EXPORT void pulp_L1Loss_fp16(void *a) { l1_impl<H, loss_args_fp16>(a, false, 0.f, 0); }
TL_EXPORT void pulp_L1Loss_backward_fp16(void *a) { l1_impl<H, loss_args_fp16>(a, false, 0.f, 1); }
TL_EXPORT void pulp_berHuLoss(void *a) { if (a) l1_impl<float, berHu_loss_args>(a, true, ((berHu_loss_args *)a)->alpha, 0); }
TL_EXPORT void pulp_berHuLoss_backward(void *a) { if (a) l1_impl<float, berHu_loss_args>(a, true, ((berHu_loss_args *)a)->alpha, 1); }
TL_EXPORT void pulp_berHuLoss_fp16(void *a) { if (a) l1_impl<H, berHu_loss_args_fp16>(a, true, f(*(H *)&((berHu_loss_args_fp16 *)a)->alpha), 0); }
TL_EXPORT void pulp_berHuLoss_backward_fp16(void *a) { if (a) l1_impl<H, berHu_loss_args_fp16>(a, true, f(*(H *)&((berHu_loss_args_fp16 *)a)->alpha), 1); }
TL_EXPORT void pulp_maxpool_fp32_fw_cl(void *a) { maxpool_impl<float, pool_args>(a, 0); }
TL_EXPORT void pulp_maxpool_fp32_bw_cl(void *a) { maxpool_impl<float, pool_args>(a, 1); }
TL_EXPORT void pulp_maxpool_fp16_fw_cl(void *a) { maxpool_impl<H, pool_args_fp16>(a, 0); }
TL_EXPORT void pulp_maxpool_fp16_bw_cl(void *a) { maxpool_impl<H, pool_args_fp16>(a, 1); }
TL_EXPORT void pulp_nonorm_fp32_fw_cl(void *a) { nonorm_impl<float, Nonorm_args>(a); }
TL_EXPORT void pulp_nonorm_fp16_fw_cl(void *a) { nonorm_impl<H, Nonorm_args_fp16>(a); }
TL_EXPORT void weighted_scaling_fp32_cl(void *a) { wscale_impl<float, weighted_scaling_args>(a); }
TL_EXPORT void weighted_scaling_fp16_cl(void *a) { wscale_impl<H, weighted_scaling_args_fp16>(a); }
TL_EXPORT void sum_of_squares_fp32_cl(void *a) { sumsq_impl<float, sum_of_squares_args>(a); }
TL_EXPORT void sum_of_squares_fp16_cl(void *a) { sumsq_impl<H, sum_of_squares_args_fp16>(a); }
TL_EXPORT void rmsnorm_parallelized_fp32(float *o, float *x, float *w, float *buf, int size) { rmsnorm_impl<float>(o, x, w, buf, size); }
TL_EXPORT void rmsnorm_parallelized_fp16(fp16 *o, fp16 *x, fp16 *w, fp16 *buf, int size) { rmsnorm_impl<H>((H *)o, (H *)x, (H *)w, (H *)buf, size); }
TL_EXPORT void pulp_swiglu_fp32_cl(void *a) { swiglu_impl<float, swiglu_args>(a); }
TL_EXPORT void pulp_swiglu_fp16_cl(void *a) { swiglu_impl<H, swiglu_args_fp16>(a); }
TL_EXPORT void pulp_vector_softmax_fp32(float *out, float *in, float *, unsigned int size) { vsoftmax_impl<float>(out, in, size); }
TL_EXPORT void pulp_vector_softmax_fp16(fp16 *out, fp16 *in, fp16 *, unsigned int size) { vsoftmax_impl<H>((H *)out, (H *)in, size); }
TL_EXPORT void pulp_max_fp32_cl(void *a) { vmax_impl<float, max_args>(a); }
TL_EXPORT void pulp_max_fp16_cl(void *a) { vmax_impl<H, max_args_fp16>(a); }
TL_EXPORT void pulp_div_fp32_cl(void *a) { vdiv_impl<float, div_args>(a); }
TL_EXPORT void pulp_div_fp16_cl(void *a) { vdiv_impl<H, div_args_fp16>(a); }
TL_EXPORT void pulp_shift_sum_fp32_cl(void *args)
{
    auto *a = (shift_sum_args *)args;
    TL_REQUIRE(a && a->dim > 0, "pulp_shift_sum: dim must be positive");
    Scope sc;
    const size_t n = (size_t)a->dim * a->dim;
    const float *x = sc.in(a->input, n), *m = sc.in(a->maxes, (size_t)a->dim);
    float *y = sc.out(a->output, n), *s = sc.out(a->sums, (size_t)a->dim);
    if (sc.ok()) shift_sum<float>(x, m, y, s, a->dim);
}
TL_EXPORT void vector_exp_sum_fp32_cl(void *a) { vexpsum_impl<float, vector_exp_sum_args>(a); }
TL_EXPORT void vector_exp_sum_fp16_cl(void *a) { vexpsum_impl<H, vector_exp_sum_args_fp16>(a); }
TL_EXPORT void pulp_sm_bw_op_1(void *a) { op1_impl<float, sm_bw_op_1_args>(a); }
TL_EXPORT void pulp_sm_bw_op_1_fp16(void *a) { op1_impl<H, sm_bw_op_1_args_fp16>(a); }
TL_EXPORT void pulp_sm_bw_op_2(void *a) { op2_impl<float, sm_bw_op_2_args>(a); }
TL_EXPORT void pulp_sm_bw_op_2_fp16(void *a) { op2_impl<H, sm_bw_op_2_args_fp16>(a); }
TL_EXPORT void pulp_row_max_fp16_cl(void *a) { rowmax16_impl<H, max_args_fp16>(a); }
TL_EXPORT void pulp_exp_sum_fp16_cl(void *a) { expsum16_impl<H, exp_sum_args_fp16>(a); }
TL_EXPORT void pulp_row_div_fp16_cl(void *a) { rowdiv16_impl<H, row_div_args_fp16>(a); }
TL_EXPORT void pulp_mean_std_fp16_cl(void *a) { meanstd16_impl<H, mean_std_args_fp16>(a); }
