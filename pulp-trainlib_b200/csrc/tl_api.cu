// The exported C ABI: every entry point takes the reference library's argument struct through
// a void pointer, resolves the tensors it touches (device pointers in place, host pointers via
// the staging scope) and launches the kernels.  fp32 and fp16 twins share one template each;
// the struct families have identical field names.
#include "tl_kernels.h"
#include <cmath>
#include <cstring>

using namespace tl;

namespace {

struct F32 {
    typedef float T;
    typedef ::blob blob_t;
    typedef ::matMul_args matMul_t;           typedef ::mm_manager_args manager_t;
    typedef ::im2col_args im2col_t;           typedef ::blocktransp_args blocktransp_t;
    typedef ::Conv2D_args conv2d_t;           typedef ::Linear_args linear_t;
    typedef ::PointWise_Conv_args pw_t;       typedef ::DepthWise_Conv_args dw_t;
    typedef ::Mhsa_args mhsa_t;               typedef ::act_args act_t;
    typedef ::leakyrelu_args leaky_t;         typedef ::softmax_args softmax_t;
    typedef ::InstNorm_args instnorm_t;       typedef ::loss_args loss_t;
    typedef ::optim_args optim_t;             typedef ::SkipConn_args skip_t;
    typedef ::pool_args pool_t;               typedef ::transp_args transp_t;
    typedef ::copy_args copy_t;               typedef ::set_to_value_args setval_t;
    typedef ::vect_sum_args vsum_t;           typedef ::array_broadcast_sum_fp32_args bcast_t;
    typedef ::pad_args pad_t;                 typedef ::scalar_mul_args smul_t;
    typedef ::mm_bias_add_args biasadd_t;
    static float f(float v) { return v; }
    static int dw_stride_h(const dw_t *a) { return a->stride_h; }
    static int dw_stride_w(const dw_t *a) { return a->stride_w; }
};
struct F16 {
    typedef __half T;
    typedef ::blob_fp16 blob_t;
    typedef ::matMul_args_fp16 matMul_t;      typedef ::mm_manager_args_fp16 manager_t;
    typedef ::im2col_args_fp16 im2col_t;      typedef ::blocktransp_args_fp16 blocktransp_t;
    typedef ::Conv2D_args_fp16 conv2d_t;      typedef ::Linear_args_fp16 linear_t;
    typedef ::PointWise_Conv_args_fp16 pw_t;  typedef ::DepthWise_Conv_args_fp16 dw_t;
    typedef ::Mhsa_args_fp16 mhsa_t;          typedef ::act_args_fp16 act_t;
    typedef ::leakyrelu_args_fp16 leaky_t;    typedef ::softmax_args_fp16 softmax_t;
    typedef ::InstNorm_args_fp16 instnorm_t;  typedef ::loss_args_fp16 loss_t;
    typedef ::optim_args_fp16 optim_t;        typedef ::SkipConn_args_fp16 skip_t;
    typedef ::pool_args_fp16 pool_t;          typedef ::transp_args_fp16 transp_t;
    typedef ::copy_args_fp16 copy_t;          typedef ::set_to_value_args_fp16 setval_t;
    typedef ::vect_sum_args_fp16 vsum_t;      typedef ::array_broadcast_sum_fp16_args bcast_t;
    typedef ::pad_args_fp16 pad_t;            typedef ::scalar_mul_args_fp16 smul_t;
    typedef ::mm_bias_add_args_fp16 biasadd_t;
    static float f(__half v) { return __half2float(v); }
    static int dw_stride_h(const dw_t *) { return 1; }
    static int dw_stride_w(const dw_t *) { return 1; }
};

#define TL_REQUIRE(cond, ...)                                        \
    do { if (!(cond)) { set_error(TL_ERR_BAD_ARGS, __VA_ARGS__); return; } } while (0)

// ------------------------------------------------------------------ matmul family
template <class F> void mm_impl(void *void_args, bool accumulate)
{
    auto *a = (typename F::matMul_t *)void_args;
    typedef typename F::T T;
    TL_REQUIRE(a && a->N > 0 && a->M > 0 && a->K > 0, "mm: N=%d M=%d K=%d must be positive", a ? a->N : 0, a ? a->M : 0, a ? a->K : 0);
    Scope sc;
    const T *A = sc.in(a->A, (size_t)a->N * a->K);
    const T *B = sc.in(a->B, (size_t)a->K * a->M);
    T *C = accumulate ? sc.inout(a->C, (size_t)a->N * a->M) : sc.out(a->C, (size_t)a->N * a->M);
    if (!sc.ok()) return;
    mm_contract<T>(A, B, C, a->N, a->K, a->M, a->trans_B ? 1 : 0, accumulate);
}

// Batched product with NumPy broadcasting of the leading dimensions [ref: lib/sources/pulp_matmul_fp32.c:29-186]:
// A is [..., N, K], B is [..., K, M]; the leading dimensions are aligned from the right, a dimension of size 1 (or a
// missing one) repeats its matrix, C holds the product matrices back to back in row-major order of the broadcast
// batch shape.  The dimension arrays are read on the host.  Consecutive output matrices whose operand offsets advance by
// a constant step go out as one batched launch.
template <class T, class A_t> static void mm_broadcast_impl(void *void_args)
{
    auto *a = (A_t *)void_args;
    TL_REQUIRE(a && a->A_dims && a->B_dims && a->A_dims_len >= 2 && a->B_dims_len >= 2 && a->A_dims_len <= 8 && a->B_dims_len <= 8,
               "mm_broadcast: operands need 2..8 dimensions");
    const int la = a->A_dims_len, lb = a->B_dims_len, lead = (la > lb ? la : lb) - 2;
    const int N = a->A_dims[la - 2], K = a->A_dims[la - 1], M = a->B_dims[lb - 1];
    TL_REQUIRE(N > 0 && K > 0 && M > 0 && a->B_dims[lb - 2] == K, "mm_broadcast: inner dimensions %d and %d differ or are empty", K, a->B_dims[lb - 2]);
    long long out_dim[8], sa[8], sb[8], total = 1, count_a = (long long)N * K, count_b = (long long)K * M;
    {
        long long run_a = (long long)N * K, run_b = (long long)K * M;
        for (int d = lead - 1; d >= 0; d--) {              // d counts leading dimensions from the right-aligned batch shape
            const int ia = d - (lead - (la - 2)), ib = d - (lead - (lb - 2));
            const int da = ia >= 0 ? a->A_dims[ia] : 1, db = ib >= 0 ? a->B_dims[ib] : 1;
            TL_REQUIRE(da > 0 && db > 0 && (da == db || da == 1 || db == 1), "mm_broadcast: batch dimensions %d and %d do not broadcast", da, db);
            out_dim[d] = da > db ? da : db;
            sa[d] = da == 1 ? 0 : run_a; sb[d] = db == 1 ? 0 : run_b;
            run_a *= da; run_b *= db;
            total *= out_dim[d];
        }
        count_a = run_a; count_b = run_b;
    }
    Scope sc;
    const T *A = sc.in(a->A, (size_t)count_a), *B = sc.in(a->B, (size_t)count_b);
    T *C = sc.out(a->C, (size_t)total * N * M);
    if (!sc.ok()) return;
    auto offsets = [&](long long i, long long &oa, long long &ob) {
        oa = ob = 0;
        for (int d = lead - 1; d >= 0; d--) { const long long r = i % out_dim[d]; i /= out_dim[d]; oa += r * sa[d]; ob += r * sb[d]; }
    };
    long long i = 0;
    while (i < total) {
        long long oa0, ob0, oa1 = 0, ob1 = 0;
        offsets(i, oa0, ob0);
        long long run = 1, da = 0, db = 0;
        if (i + 1 < total) {
            offsets(i + 1, oa1, ob1);
            da = oa1 - oa0; db = ob1 - ob0;
            run = 2;
            while (i + run < total) {
                long long oa, ob;
                offsets(i + run, oa, ob);
                if (oa - oa0 != run * da || ob - ob0 != run * db) break;
                run++;
            }
        }
        GemmDesc<T> d;
        d.A = A + oa0; d.a_rs = K; d.B = B + ob0; d.b_rs = M; d.C = C + i * (long long)N * M; d.c_rs = M;
        d.N = N; d.K = K; d.M = M;
        d.batch = (int)run; d.a_bs = da; d.b_bs = db; d.c_bs = (long long)N * M;
        gemm<T>(d);
        i += run;
    }
}

// Dispatcher [ref: lib/sources/pulp_train_utils_fp32.c:1330-1683]: one GEMM whatever matmul_type
// says; bias add after the product when mm_args->USE_BIASES == 1 (t = bias_transposed).
template <class F> void mm_manager_impl(void *void_args)
{
    auto *m = (typename F::manager_t *)void_args;
    typedef typename F::T T;
    if (!m || !m->mm_args) { set_error(TL_ERR_BAD_ARGS, "mm_manager: null arguments"); return; }
    if (m->layer_type != LAYER_CONV2D && m->layer_type != LAYER_PW_CONV && m->layer_type != LAYER_LINEAR) {
        printf("\nWrong layer_type selection!!\n");
        set_error(TL_ERR_BAD_ARGS, "mm_manager: layer_type %d has no matmul branch", m->layer_type);
        return;
    }
    if (m->step_type != STEP_FW && m->step_type != STEP_WGT_GRAD && m->step_type != STEP_IN_GRAD) {
        printf("\nWrong step selection!!\n");
        set_error(TL_ERR_BAD_ARGS, "mm_manager: step_type %d", m->step_type);
        return;
    }
    auto *a = m->mm_args;
    TL_REQUIRE(a->N > 0 && a->M > 0 && a->K > 0, "mm_manager: N=%d M=%d K=%d must be positive", a->N, a->M, a->K);
    Scope sc;
    const T *A = sc.in(a->A, (size_t)a->N * a->K);
    const T *B = sc.in(a->B, (size_t)a->K * a->M);
    T *C = sc.out(a->C, (size_t)a->N * a->M);
    const bool use_bias = (a->USE_BIASES == 1) && a->bias;
    const T *bias = use_bias ? sc.in(a->bias, (size_t)(a->bias_transposed ? a->N : a->M)) : nullptr;
    if (!sc.ok()) return;
    mm_contract<T>(A, B, C, a->N, a->K, a->M, a->trans_B ? 1 : 0, false);
    if (use_bias) bias_add_rows<T>(C, bias, a->N, a->M, a->bias_transposed ? 1 : 0);
}

// ------------------------------------------------------------------ convolution geometry
template <class A> bool conv_geom(const A *a, ConvGeom &g, const char *who)
{
    g.Cin = a->input->C; g.Hin = a->input->H; g.Win = a->input->W;
    g.Cout = a->output->C; g.Hk = a->coeff->H; g.Wk = a->coeff->W;
    g.sh = a->stride_h; g.sw = a->stride_w; g.padU = a->Upad; g.padL = a->Lpad;
    g.n = streams(); g.depthwise = false; g.hwc = false;
    if (g.sh < 1 || g.sw < 1 || g.Hk < 1 || g.Wk < 1 || g.Cin < 1 || g.Cout < 1 || g.Hin < 1 || g.Win < 1) {
        set_error(TL_ERR_BAD_ARGS, "%s: invalid geometry (C_in %d, %dx%d, C_out %d, kernel %dx%d, stride %d,%d)", who,
                  g.Cin, g.Hin, g.Win, g.Cout, g.Hk, g.Wk, g.sh, g.sw);
        return false;
    }
    // [ref: lib/sources/pulp_conv_naive_fp32.c:222-223] output size of the naive kernels
    g.Hout = (g.Hin - g.Hk + a->Upad + a->Dpad) / g.sh + 1;
    g.Wout = (g.Win - g.Wk + a->Lpad + a->Rpad) / g.sw + 1;
    if (g.Hout < 1 || g.Wout < 1 || g.Hout != a->output->H || g.Wout != a->output->W) {
        set_error(TL_ERR_BAD_ARGS, "%s: output blob is %dx%d but the geometry gives %dx%d", who, a->output->H, a->output->W, g.Hout, g.Wout);
        return false;
    }
    return true;
}

template <class A> bool conv_flags_ok(const A *a, const char *who)
{
    if (a->USE_IM2COL != 0 && a->USE_IM2COL != 1) {
        printf("[%s:] Invalid selection of the conv2d algorithm (im2col or not)\n", who);
        set_error(TL_ERR_BAD_ARGS, "%s: USE_IM2COL = %d", who, a->USE_IM2COL);
        return false;
    }
    if (a->HWC != 0 && a->HWC != 1) {
        printf("[%s:] Invalid data layout format (HWC or CHW)!\n", who); set_error(TL_ERR_BAD_ARGS, "%s: HWC = %d", who, a->HWC);
        return false;
    }
    return true;
}

// HWC layout [ref: lib/sources/pulp_conv2d_fp32.c:115-238 (forward), :334-452 (weight gradient), :550-660 (input gradient)]:
// activations [H][W][C], weights [Cout][Hk][Wk][Cin].  The kernels work on CHW, so HWC operands are permuted into
// scratch on the way in and results permuted back on the way out (one pass over each tensor; the convolution itself
// then runs on the same tensor-core / FFMA kernels as the CHW layout).
template <class T> static const T *hwc_in(Scope &sc, const T *src, int n, int C, int H, int W)
{
    T *dst = sc.scratch<T>((size_t)n * C * H * W);
    if (!dst) return nullptr;
    const int dims[4] = {n, H, W, C}, axes[4] = {0, 3, 1, 2};
    transpose_nd<T>(src, dst, dims, axes, 4);
    return dst;
}
template <class T> static void hwc_out(const T *chw, T *dst, int n, int C, int H, int W)
{
    const int dims[4] = {n, C, H, W}, axes[4] = {0, 2, 3, 1};
    transpose_nd<T>(chw, dst, dims, axes, 4);
}

template <class F> void conv2d_fw_impl(void *args)
{
    auto *a = (typename F::conv2d_t *)args; typedef typename F::T T;
    if (!conv_flags_ok(a, "pulp_conv2d_fw_cl")) return;
    ConvGeom g; if (!conv_geom(a, g, "pulp_conv2d_fw_cl")) return;
    Scope sc;
    const T *x = sc.in(a->input->data, (size_t)g.n * g.Cin * g.Hin * g.Win);
    const T *w = sc.in(a->coeff->data, (size_t)g.Cout * g.Cin * g.Hk * g.Wk);
    const T *b = (a->USE_BIASES == 1 && a->bias) ? sc.in(a->bias->data, (size_t)g.Cout) : nullptr;
    T *y = sc.out(a->output->data, (size_t)g.n * g.Cout * g.Hout * g.Wout);
    if (!sc.ok()) return;
    if (a->HWC == 1) {
        const T *xc = hwc_in<T>(sc, x, g.n, g.Cin, g.Hin, g.Win), *wc = hwc_in<T>(sc, w, g.Cout, g.Cin, g.Hk, g.Wk);
        T *yc = sc.scratch<T>((size_t)g.n * g.Cout * g.Hout * g.Wout);
        if (!xc || !wc || !yc) return;
        conv_fw<T>(sc, g, xc, wc, b, yc);
        hwc_out<T>(yc, y, g.n, g.Cout, g.Hout, g.Wout);
        return;
    }
    conv_fw<T>(sc, g, x, w, b, y);
}
template <class F> void conv2d_wg_impl(void *args)
{
    auto *a = (typename F::conv2d_t *)args; typedef typename F::T T;
    if (!conv_flags_ok(a, "pulp_conv2d_bw_param_grads_cl")) return;
    ConvGeom g; if (!conv_geom(a, g, "pulp_conv2d_bw_param_grads_cl")) return;
    Scope sc;
    const T *x = sc.in(a->input->data, (size_t)g.n * g.Cin * g.Hin * g.Win);
    const T *dy = sc.in(a->output->diff, (size_t)g.n * g.Cout * g.Hout * g.Wout);
    T *dw = sc.out(a->coeff->diff, (size_t)g.Cout * g.Cin * g.Hk * g.Wk);
    T *db = (a->USE_BIASES == 1 && a->bias) ? sc.out(a->bias->diff, (size_t)g.Cout) : nullptr;
    if (!sc.ok()) return;
    if (a->HWC == 1) {
        const T *xc = hwc_in<T>(sc, x, g.n, g.Cin, g.Hin, g.Win), *dyc = hwc_in<T>(sc, dy, g.n, g.Cout, g.Hout, g.Wout);
        T *dwc = sc.scratch<T>((size_t)g.Cout * g.Cin * g.Hk * g.Wk);
        if (!xc || !dyc || !dwc) return;
        sc.no_deferral();                           // the permutation below reads dwc at once
        conv_wg<T>(sc, g, xc, dyc, dwc, db);
        hwc_out<T>(dwc, dw, g.Cout, g.Cin, g.Hk, g.Wk);
        return;
    }
    conv_wg<T>(sc, g, x, dy, dw, db);
}
template <class F> void conv2d_ig_impl(void *args, bool accumulate = false)
{
    auto *a = (typename F::conv2d_t *)args; typedef typename F::T T;
    if (!conv_flags_ok(a, "pulp_conv2d_bw_input_grads_cl")) return;
    ConvGeom g; if (!conv_geom(a, g, "pulp_conv2d_bw_input_grads_cl")) return;
    Scope sc;
    const T *dy = sc.in(a->output->diff, (size_t)g.n * g.Cout * g.Hout * g.Wout);
    const T *w = sc.in(a->coeff->data, (size_t)g.Cout * g.Cin * g.Hk * g.Wk);
    const size_t nx = (size_t)g.n * g.Cin * g.Hin * g.Win;
    T *dx = accumulate ? sc.inout(a->input->diff, nx) : sc.out(a->input->diff, nx);
    if (!sc.ok()) return;
    if (accumulate) {
        TL_REQUIRE(a->HWC == 0, "trainlib_conv2d_bw_input_grads_acc_cl: HWC=%d (CHW only)", a->HWC);
        conv_ig_accumulate<T>(sc, g, dy, w, dx);
        return;
    }
    if (a->HWC == 1) {
        const T *dyc = hwc_in<T>(sc, dy, g.n, g.Cout, g.Hout, g.Wout), *wc = hwc_in<T>(sc, w, g.Cout, g.Cin, g.Hk, g.Wk);
        T *dxc = sc.scratch<T>((size_t)g.n * g.Cin * g.Hin * g.Win);
        if (!dyc || !wc || !dxc) return;
        conv_ig<T>(sc, g, dyc, wc, dxc);
        hwc_out<T>(dxc, dx, g.n, g.Cin, g.Hin, g.Win);
        return;
    }
    conv_ig<T>(sc, g, dy, w, dx);
}

// Naive kernels on matMul_args [ref: lib/sources/pulp_conv_naive_fp32.c:198-515]:
// A = input (or its gradient), B = weights (or their gradient), C = output (or its gradient).
template <class F> bool naive_geom(const typename F::matMul_t *a, ConvGeom &g)
{
    g.Cin = a->pCin; g.Hin = a->H; g.Win = a->W; g.Cout = a->pCout; g.Hk = a->pH; g.Wk = a->pW;
    g.sh = a->stride_h; g.sw = a->stride_w; g.padU = a->Upad; g.padL = a->Lpad;
    g.n = streams(); g.depthwise = false; g.hwc = false;
    if (g.sh < 1 || g.sw < 1 || g.Hk < 1 || g.Wk < 1 || g.Cin < 1 || g.Cout < 1) { set_error(TL_ERR_BAD_ARGS, "naive conv2d: invalid geometry"); return false; }
    g.Hout = (g.Hin - g.Hk + a->Upad + a->Dpad) / g.sh + 1;
    g.Wout = (g.Win - g.Wk + a->Lpad + a->Rpad) / g.sw + 1;
    if (g.Hout < 1 || g.Wout < 1) { set_error(TL_ERR_BAD_ARGS, "naive conv2d: empty output"); return false; }
    return true;
}
template <class F> void naive_impl(void *args, int step)
{
    auto *a = (typename F::matMul_t *)args; typedef typename F::T T;
    ConvGeom g; if (!naive_geom<F>(a, g)) return;
    Scope sc;
    const size_t nx = (size_t)g.n * g.Cin * g.Hin * g.Win, nw = (size_t)g.Cout * g.Cin * g.Hk * g.Wk, ny = (size_t)g.n * g.Cout * g.Hout * g.Wout;
    const bool ub = (a->USE_BIASES == 1) && a->bias;
    if (step == STEP_FW) {
        const T *x = sc.in(a->A, nx), *w = sc.in(a->B, nw), *b = ub ? sc.in(a->bias, (size_t)g.Cout) : nullptr;
        T *y = sc.out(a->C, ny);
        if (sc.ok()) conv_fw<T>(sc, g, x, w, b, y);
    } else if (step == STEP_WGT_GRAD) {
        const T *x = sc.in(a->A, nx), *dy = sc.in(a->C, ny);
        T *dw = sc.out(a->B, nw), *db = ub ? sc.out(a->bias, (size_t)g.Cout) : nullptr;
        if (sc.ok()) conv_wg<T>(sc, g, x, dy, dw, db);
    } else {
        const T *dy = sc.in(a->C, ny), *w = sc.in(a->B, nw);
        T *dx = sc.out(a->A, nx);
        if (sc.ok()) conv_ig<T>(sc, g, dy, w, dx);
    }
}

// ------------------------------------------------------------------ im2row / im2col / blocktransp
template <class F> void im2row_impl(void *args, int transposed_buf)
{
    auto *a = (typename F::im2col_t *)args; typedef typename F::T T;
    const char *who = transposed_buf ? "pulp_im2col" : "pulp_im2row";
    TL_REQUIRE(a && a->input && a->c && a->output && a->pBuffer, "%s: null arguments", who);
    const int Cin = a->input->C, Hin = a->input->H, Win = a->input->W, Hk = a->c->H, Wk = a->c->W, Co = a->output->C;
    TL_REQUIRE(a->HWC == 0 || a->HWC == 1, "%s: HWC = %d", who, a->HWC);
    Scope sc;
    if (a->mod == 0) {
        TL_REQUIRE(a->stride_h >= 1 && a->stride_w >= 1, "%s: strides must be >= 1", who);
        // [ref: lib/sources/pulp_im2col_fp32.c:125-128] strides that do not tile the padded input are rejected
        if ((Hin - Hk + a->Upad + a->Dpad + a->stride_h) % a->stride_h > 0 || (Win - Wk + a->Lpad + a->Rpad + a->stride_w) % a->stride_w > 0) {
            printf("\n[%s] Invalid stride (non multiple sizes)\n", who);
            set_error(TL_ERR_BAD_ARGS, "%s: stride does not divide the padded extent", who);
            return;
        }
        const int Ho = (Hin - Hk + a->Upad + a->Dpad + a->stride_h) / a->stride_h, Wo = (Win - Wk + a->Lpad + a->Rpad + a->stride_w) / a->stride_w;
        const T *x = sc.in(a->input->data, (size_t)Cin * Hin * Win);
        T *buf = sc.out(a->pBuffer, (size_t)Ho * Wo * Cin * Hk * Wk);
        if (sc.ok()) im2row<T>(x, buf, Cin, Hin, Win, Hk, Wk, Ho, Wo, a->stride_h, a->stride_w, a->Upad, a->Lpad, 0, a->HWC, transposed_buf);
    } else {
        if (transposed_buf) { set_error(TL_ERR_UNSUPPORTED, "pulp_im2col: mod = 1 is not implemented"); return; }
        const int Ho = a->output->H, Wo = a->output->W;
        const T *dy = sc.in(a->output->diff, (size_t)Co * Ho * Wo);
        T *buf = sc.out(a->pBuffer, (size_t)Hin * Win * Co * Hk * Wk);
        if (sc.ok()) im2row<T>(dy, buf, Co, Hin, Win, Hk, Wk, Ho, Wo, 1, 1, 0, 0, 1, a->HWC, 0);
    }
}
template <class F> void blocktransp_impl(void *args)
{
    auto *a = (typename F::blocktransp_t *)args; typedef typename F::T T;
    TL_REQUIRE(a && a->weights && a->bt_weights, "pulp_blocktransp: null arguments");
    if (a->HWC != 0 && a->HWC != 1) { printf("[pulp_blocktransp] Invalid data layout (not 0 or 1)!!\n"); set_error(TL_ERR_BAD_ARGS, "pulp_blocktransp: HWC = %d", a->HWC); return; }
    const size_t n = (size_t)a->Cin * a->Cout * a->Hk * a->Wk;
    Scope sc;
    const T *w = sc.in(a->weights, n);
    T *bt = sc.out(a->bt_weights, n);
    if (sc.ok()) blocktransp<T>(w, bt, a->Cin, a->Cout, a->Hk, a->Wk, a->HWC);
}

// ------------------------------------------------------------------ pointwise conv
// CHW: Y[Cout x HW] = W[Cout x Cin] X[Cin x HW]; HWC: Y[HW x Cout] = X[HW x Cin] W[Cin x Cout]
// [ref: lib/sources/pulp_conv_pw_fp32.c:27-330].
template <class F> void pw_impl(void *args, int step)
{
    auto *a = (typename F::pw_t *)args; typedef typename F::T T;
    const int Cin = a->input->C, Cout = a->output->C, HW = a->input->H * a->input->W, n = streams();
    if (a->HWC != 0 && a->HWC != 1) { printf("[pulp_conv_pw] Invalid HWC parameter!\n"); set_error(TL_ERR_BAD_ARGS, "pulp_conv_pw: HWC = %d", a->HWC); return; }
    TL_REQUIRE(a->output->H * a->output->W == HW, "pulp_conv_pw: input and output planes differ");
    TL_REQUIRE(!(a->HWC == 1 && n > 1), "pulp_conv_pw: HWC layout supports a single stream");
    Scope sc;
    const size_t nx = (size_t)n * Cin * HW, ny = (size_t)n * Cout * HW, nw = (size_t)Cin * Cout;
    if (a->HWC == 0 && n > 1) {                      // many streams: the conv kernels batch over streams
        ConvGeom g = {Cin, a->input->H, a->input->W, Cout, 1, 1, a->input->H, a->input->W, 1, 1, 0, 0, n, false, false};
        if (step == STEP_FW) { const T *x = sc.in(a->input->data, nx), *w = sc.in(a->coeff->data, nw); T *y = sc.out(a->output->data, ny); if (sc.ok()) conv_fw<T>(sc, g, x, w, (const T *)nullptr, y); }
        else if (step == STEP_WGT_GRAD) { const T *x = sc.in(a->input->data, nx), *dy = sc.in(a->output->diff, ny); T *dw = sc.out(a->coeff->diff, nw); if (sc.ok()) conv_wg<T>(sc, g, x, dy, dw, (T *)nullptr); }
        else { const T *dy = sc.in(a->output->diff, ny), *w = sc.in(a->coeff->data, nw); T *dx = sc.out(a->input->diff, nx); if (sc.ok()) conv_ig<T>(sc, g, dy, w, dx); }
        return;
    }
    GemmDesc<T> d;
    if (step == STEP_FW) {
        const T *x = sc.in(a->input->data, nx), *w = sc.in(a->coeff->data, nw); T *y = sc.out(a->output->data, ny);
        if (!sc.ok()) return;
        if (a->HWC == 0) { d.A = w; d.a_rs = Cin; d.B = x; d.b_rs = HW; d.C = y; d.c_rs = HW; d.N = Cout; d.K = Cin; d.M = HW; }
        else { d.A = x; d.a_rs = Cin; d.B = w; d.b_rs = Cout; d.C = y; d.c_rs = Cout; d.N = HW; d.K = Cin; d.M = Cout; }
    } else if (step == STEP_WGT_GRAD) {
        const T *x = sc.in(a->input->data, nx), *dy = sc.in(a->output->diff, ny); T *dw = sc.out(a->coeff->diff, nw);
        if (!sc.ok()) return;
        if (a->HWC == 0) { d.A = dy; d.a_rs = HW; d.B = x; d.b_rs = 1; d.b_cs = HW; d.C = dw; d.c_rs = Cin; d.N = Cout; d.K = HW; d.M = Cin; }
        else { d.A = x; d.a_rs = 1; d.a_cs = Cin; d.B = dy; d.b_rs = Cout; d.C = dw; d.c_rs = Cout; d.N = Cin; d.K = HW; d.M = Cout; }
    } else {
        const T *dy = sc.in(a->output->diff, ny), *w = sc.in(a->coeff->data, nw); T *dx = sc.out(a->input->diff, nx);
        if (!sc.ok()) return;
        if (a->HWC == 0) { d.A = w; d.a_rs = 1; d.a_cs = Cin; d.B = dy; d.b_rs = HW; d.C = dx; d.c_rs = HW; d.N = Cin; d.K = Cout; d.M = HW; }
        else { d.A = dy; d.a_rs = Cout; d.B = w; d.b_rs = 1; d.b_cs = Cout; d.C = dx; d.c_rs = Cin; d.N = HW; d.K = Cout; d.M = Cin; }
    }
    gemm<T>(d);
}

// ------------------------------------------------------------------ depthwise conv
template <class F> void dw_impl(void *args, int step)
{
    auto *a = (typename F::dw_t *)args; typedef typename F::T T;
    TL_REQUIRE(a->HWC == 0, "pulp_conv_dw: only the CHW layout exists");
    ConvGeom g;
    g.Cin = g.Cout = a->input->C; g.Hin = a->input->H; g.Win = a->input->W; g.Hk = a->coeff->H; g.Wk = a->coeff->W;
    g.sh = F::dw_stride_h(a); g.sw = F::dw_stride_w(a); g.padU = a->Upad; g.padL = a->Lpad;
    if (g.sh < 1) g.sh = 1;
    if (g.sw < 1) g.sw = 1;
    g.Hout = a->output->H; g.Wout = a->output->W; g.n = streams(); g.depthwise = true; g.hwc = false;
    TL_REQUIRE(g.Hout == (g.Hin - g.Hk + a->Upad + a->Dpad) / g.sh + 1 && g.Wout == (g.Win - g.Wk + a->Lpad + a->Rpad) / g.sw + 1,
               "pulp_conv_dw: output blob %dx%d does not match the geometry", g.Hout, g.Wout);
    Scope sc;
    const size_t nx = (size_t)g.n * g.Cin * g.Hin * g.Win, ny = (size_t)g.n * g.Cin * g.Hout * g.Wout, nw = (size_t)g.Cin * g.Hk * g.Wk;
    if (step == STEP_FW) { const T *x = sc.in(a->input->data, nx), *w = sc.in(a->coeff->data, nw); T *y = sc.out(a->output->data, ny); if (sc.ok()) conv_fw<T>(sc, g, x, w, (const T *)nullptr, y); }
    else if (step == STEP_WGT_GRAD) { const T *x = sc.in(a->input->data, nx), *dy = sc.in(a->output->diff, ny); T *dw = sc.out(a->coeff->diff, nw); if (sc.ok()) conv_wg<T>(sc, g, x, dy, dw, (T *)nullptr); }
    else { const T *dy = sc.in(a->output->diff, ny), *w = sc.in(a->coeff->data, nw); T *dx = sc.out(a->input->diff, nx); if (sc.ok()) conv_ig<T>(sc, g, dy, w, dx); }
}

// the forkable workers of the depthwise layer: same kernels, geometry from kernel_DW_args
// [ref: lib/sources/pulp_conv_naive_fp32.c:29-330]
template <class T, class A> void dwk_impl(void *args, int step, int sh, int sw, int pl, int pr, int pu, int pd)
{
    auto *a = (A *)args;
    TL_REQUIRE(a && a->input && a->weights && a->output, "dw_kernel: null arguments");
    ConvGeom g;
    g.Cin = g.Cout = a->input->C; g.Hin = a->input->H; g.Win = a->input->W; g.Hk = a->weights->H; g.Wk = a->weights->W;
    g.sh = sh < 1 ? 1 : sh; g.sw = sw < 1 ? 1 : sw; g.padU = pu; g.padL = pl;
    g.Hout = a->output->H; g.Wout = a->output->W; g.n = streams(); g.depthwise = true; g.hwc = false;
    TL_REQUIRE(g.Hout == (g.Hin - g.Hk + pu + pd) / g.sh + 1 && g.Wout == (g.Win - g.Wk + pl + pr) / g.sw + 1,
               "dw_kernel: output blob %dx%d does not match the geometry", g.Hout, g.Wout);
    Scope sc;
    const size_t nx = (size_t)g.n * g.Cin * g.Hin * g.Win, ny = (size_t)g.n * g.Cin * g.Hout * g.Wout, nw = (size_t)g.Cin * g.Hk * g.Wk;
    if (step == STEP_FW) { const T *x = sc.in((T *)a->input->data, nx), *w = sc.in((T *)a->weights->data, nw); T *y = sc.out((T *)a->output->data, ny); if (sc.ok()) conv_fw<T>(sc, g, x, w, (const T *)nullptr, y); }
    else if (step == STEP_WGT_GRAD) { const T *x = sc.in((T *)a->input->data, nx), *dy = sc.in((T *)a->output->diff, ny); T *dw = sc.out((T *)a->weights->diff, nw); if (sc.ok()) conv_wg<T>(sc, g, x, dy, dw, (T *)nullptr); }
    else { const T *dy = sc.in((T *)a->output->diff, ny), *w = sc.in((T *)a->weights->data, nw); T *dx = sc.out((T *)a->input->diff, nx); if (sc.ok()) conv_ig<T>(sc, g, dy, w, dx); }
}

// ------------------------------------------------------------------ linear
// W is [out x in]; y = W x (+ b); dW = dy (x) x, db = dy; dx = W^T dy
// [ref: lib/sources/pulp_linear_fp32.c:25-267].  With n streams the three become GEMMs.
template <class F> void linear_impl(void *args, int step)
{
    auto *a = (typename F::linear_t *)args; typedef typename F::T T;
    const int in = a->input->dim, out = a->output->dim, n = streams();
    TL_REQUIRE(in > 0 && out > 0, "pulp_linear: empty layer");
    const bool ub = (a->use_biases == 1) && a->bias;
    Scope sc;
    if (step == STEP_FW) {
        const T *w = sc.in(a->coeff->data, (size_t)out * in), *x = sc.in(a->input->data, (size_t)n * in);
        const T *b = ub ? sc.in(a->bias->data, (size_t)out) : nullptr;
        T *y = sc.out(a->output->data, (size_t)n * out);
        if (!sc.ok()) return;
        if (n == 1) linear_fw_gemv<T>(w, x, b, y, out, in);
        else {
            GemmDesc<T> d; d.A = x; d.a_rs = in; d.B = w; d.b_rs = 1; d.b_cs = in; d.C = y; d.c_rs = out; d.N = n; d.K = in; d.M = out;
            if (b) { d.bias = b; d.bias_mode = 2; }
            gemm<T>(d);
        }
    } else if (step == STEP_WGT_GRAD) {
        const T *dy = sc.in(a->output->diff, (size_t)n * out), *x = sc.in(a->input->data, (size_t)n * in);
        T *dw = sc.out(a->coeff->diff, (size_t)out * in);
        T *db = ub ? sc.out(a->bias->diff, (size_t)out) : nullptr;
        if (!sc.ok()) return;
        if (n == 1) linear_wg_outer<T>(dy, x, dw, out, in);
        else if (linear_wg_streams<T>(sc, dy, x, dw, n, out, in)) { /* contraction over the streams, split into blocks */ }
        else {
            GemmDesc<T> d; d.A = dy; d.a_rs = 1; d.a_cs = out; d.B = x; d.b_rs = in; d.C = dw; d.c_rs = in; d.N = out; d.K = n; d.M = in;
            gemm<T>(d);
        }
        if (db) column_sum<T>(sc, dy, db, n, out);
    } else {
        const T *dy = sc.in(a->output->diff, (size_t)n * out), *w = sc.in(a->coeff->data, (size_t)out * in);
        T *dx = sc.out(a->input->diff, (size_t)n * in);
        if (!sc.ok()) return;
        if (n == 1) linear_ig_gemv<T>(sc, w, dy, dx, out, in);
        else {
            GemmDesc<T> d; d.A = dy; d.a_rs = out; d.B = w; d.b_rs = in; d.C = dx; d.c_rs = in; d.N = n; d.K = out; d.M = in;
            gemm<T>(d);
        }
    }
}

// pulp_linear_*_bw_cl with both gradients wanted, one stream: one launch for the two [ref: lib/sources/pulp_linear_fp32.c:60-75]
template <class F> bool linear_bw_both(void *args)
{
    auto *a = (typename F::linear_t *)args; typedef typename F::T T;
    const int in = a->input->dim, out = a->output->dim;
    if (streams() != 1 || in <= 0 || out <= 0 || gemm_path() == 1) return false;
    const bool ub = (a->use_biases == 1) && a->bias;
    // what the kernel needs is checked before anything is staged: 16-byte strips (host buffers get aligned device mirrors)
    if (in % (16 / (int)sizeof(T)) != 0 || in / (16 / (int)sizeof(T)) > 8192 * 32) return false;
    const void *ptrs[4] = {a->coeff->data, a->coeff->diff, a->input->data, a->input->diff};
    for (const void *q : ptrs)
        if (!q || (is_device_pointer(q) && (((uintptr_t)q) & 15) != 0)) return false;
    Scope sc;
    const T *dy = sc.in(a->output->diff, (size_t)out), *x = sc.in(a->input->data, (size_t)in), *w = sc.in(a->coeff->data, (size_t)out * in);
    T *dw = sc.out(a->coeff->diff, (size_t)out * in), *dx = sc.out(a->input->diff, (size_t)in);
    T *db = ub ? sc.out(a->bias->diff, (size_t)out) : nullptr;
    if (!sc.ok()) return true;                                     // the error is set; the separate calls would fail the same way
    if (!linear_bw_fused<T>(sc, w, dy, x, dw, dx, out, in)) return true;   // only a failed scratch allocation is left: the error is set
    if (db) column_sum<T>(sc, dy, db, 1, out);
    return true;
}

// ------------------------------------------------------------------ MHSA
template <class F> bool mhsa_dims(const typename F::mhsa_t *a, MhsaDims &d)
{
    d.L = a->input->H; d.E = a->input->W; d.F = a->attention_map->W; d.heads = a->n_heads;
    if (d.L < 1 || d.E < 1 || d.F < 1 || d.heads < 1 || d.F % d.heads) {
        set_error(TL_ERR_BAD_ARGS, "pulp_mhsa: L=%d E=%d F=%d heads=%d", d.L, d.E, d.F, d.heads);
        return false;
    }
    if (streams() != 1) { set_error(TL_ERR_UNSUPPORTED, "pulp_mhsa: streams mode is not available for attention"); return false; }
    return true;
}
template <class F> void mhsa_fw_impl(void *args)
{
    auto *a = (typename F::mhsa_t *)args; typedef typename F::T T;
    MhsaDims d; if (!mhsa_dims<F>(a, d)) return;
    const size_t EL = (size_t)d.E * d.L, EF = (size_t)d.E * d.F, FL = (size_t)d.F * d.L, SM = (size_t)d.heads * d.L * d.L;
    Scope sc;
    const T *x = sc.in(a->input->data, EL);
    const T *wq = sc.in(a->coeff_in_q->data, EF), *wk = sc.in(a->coeff_in_k->data, EF), *wv = sc.in(a->coeff_in_v->data, EF);
    const T *bq = a->bias_in_q ? sc.in(a->bias_in_q->data, (size_t)d.F) : nullptr;
    const T *bk = a->bias_in_k ? sc.in(a->bias_in_k->data, (size_t)d.F) : nullptr;
    const T *bv = a->bias_in_v ? sc.in(a->bias_in_v->data, (size_t)d.F) : nullptr;
    const T *wo = sc.in(a->coeff_out->data, EF);
    T *q = sc.out(a->q->data, FL), *k = sc.out(a->k->data, FL), *v = sc.out(a->v->data, FL);
    T *sm = sc.out(a->softmax_buffer->data, SM), *att = sc.out(a->attention_map->data, FL), *y = sc.out(a->output->data, EL);
    if (!sc.ok()) return;
    mhsa_fw<T>(sc, d, x, wq, wk, wv, bq, bk, bv, wo, q, k, v, sm, att, y);
}
template <class F> void mhsa_bw_impl(void *args)
{
    auto *a = (typename F::mhsa_t *)args; typedef typename F::T T;
    MhsaDims d; if (!mhsa_dims<F>(a, d)) return;
    const size_t EL = (size_t)d.E * d.L, EF = (size_t)d.E * d.F, FL = (size_t)d.F * d.L, SM = (size_t)d.heads * d.L * d.L;
    Scope sc;
    const T *x = sc.in(a->input->data, EL);
    const T *wq = sc.in(a->coeff_in_q->data, EF), *wk = sc.in(a->coeff_in_k->data, EF), *wv = sc.in(a->coeff_in_v->data, EF), *wo = sc.in(a->coeff_out->data, EF);
    const T *q = sc.in(a->q->data, FL), *k = sc.in(a->k->data, FL), *v = sc.in(a->v->data, FL);
    const T *sm = sc.in(a->softmax_buffer->data, SM), *att = sc.in(a->attention_map->data, FL), *dy = sc.in(a->output->diff, EL);
    T *dq = sc.out(a->q->diff, FL), *dk = sc.out(a->k->diff, FL), *dv = sc.out(a->v->diff, FL);
    T *dsm = sc.out(a->softmax_buffer->diff, SM), *datt = sc.out(a->attention_map->diff, FL);
    T *dwq = sc.out(a->coeff_in_q->diff, EF), *dwk = sc.out(a->coeff_in_k->diff, EF), *dwv = sc.out(a->coeff_in_v->diff, EF), *dwo = sc.out(a->coeff_out->diff, EF);
    T *dx = sc.inout(a->input->diff, EL);
    if (!sc.ok()) return;
    mhsa_bw<T>(sc, d, x, wq, wk, wv, wo, q, k, v, sm, att, dy, dq, dk, dv, dsm, datt, (T *)nullptr, dwq, dwk, dwv, dwo, dx);
}

// MobileBERT attention: `tiled` reads the sizes from the coefficient blobs as tiled_mhsa_fp32 does
// [ref: lib/sources/pulp_mhsa_fp32.c:2201, :2213-2214, :2365-2366], else F = Kb = No = input_bn->W [ref: :1784].
template <class F> bool mobilebert_dims(const typename F::mhsa_t *a, MobileBertDims &d, bool tiled, const char *who)
{
    if (!a || !a->input || !a->input_bn || !a->output || !a->coeff_in_q || !a->coeff_in_k || !a->coeff_in_v || !a->coeff_out ||
        !a->q || !a->k || !a->v || !a->attention_map || !a->softmax_buffer) { set_error(TL_ERR_BAD_ARGS, "%s: null blob", who); return false; }
    d.L = a->input->H; d.E = a->input->W; d.heads = a->n_heads;
    if (tiled) { d.F = a->coeff_in_q->H; d.Kb = a->coeff_in_q->W; d.No = a->coeff_out->H; }
    else { d.F = d.Kb = d.No = a->input_bn->W; }
    if (d.L < 1 || d.E < 1 || d.F < 1 || d.Kb < 1 || d.No < 1 || d.heads < 1 || d.F % d.heads || (tiled && a->coeff_out->W != d.F)) {
        set_error(TL_ERR_BAD_ARGS, "%s: L=%d E=%d Kb=%d F=%d No=%d heads=%d", who, d.L, d.E, d.Kb, d.F, d.No, d.heads);
        return false;
    }
    if (streams() != 1) { set_error(TL_ERR_UNSUPPORTED, "%s: streams mode is not available for attention", who); return false; }
    return true;
}
template <class F> void mobilebert_fw_impl(void *args, bool tiled)
{
    auto *a = (typename F::mhsa_t *)args; typedef typename F::T T;
    MobileBertDims d; if (!mobilebert_dims<F>(a, d, tiled, "mobilebert attention forward")) return;
    const size_t FL = (size_t)d.F * d.L, SM = (size_t)d.heads * d.L * d.L;
    Scope sc;
    const T *x = sc.in(a->input->data, (size_t)d.L * d.E), *xb = sc.in(a->input_bn->data, (size_t)d.L * d.Kb);
    const T *wq = sc.in(a->coeff_in_q->data, (size_t)d.F * d.Kb), *wk = sc.in(a->coeff_in_k->data, (size_t)d.F * d.Kb);
    const T *wv = sc.in(a->coeff_in_v->data, (size_t)d.F * d.E), *wo = sc.in(a->coeff_out->data, (size_t)d.No * d.F);
    const T *bq = a->bias_in_q ? sc.in(a->bias_in_q->data, (size_t)d.F) : nullptr;
    const T *bk = a->bias_in_k ? sc.in(a->bias_in_k->data, (size_t)d.F) : nullptr;
    const T *bv = a->bias_in_v ? sc.in(a->bias_in_v->data, (size_t)d.F) : nullptr;
    const T *bo = a->bias_out ? sc.in(a->bias_out->data, (size_t)d.No) : nullptr;
    T *q = sc.out(a->q->data, FL), *k = sc.out(a->k->data, FL), *v = sc.out(a->v->data, FL);
    T *sm = sc.out(a->softmax_buffer->data, SM), *att = sc.out(a->attention_map->data, FL), *y = sc.out(a->output->data, (size_t)d.L * d.No);
    if (!sc.ok()) return;
    mhsa_mobilebert_fw<T>(sc, d, x, xb, wq, wk, wv, bq, bk, bv, wo, bo, q, k, v, sm, att, y);
}
template <class F> void mobilebert_bw_impl(void *args)
{
    auto *a = (typename F::mhsa_t *)args; typedef typename F::T T;
    MobileBertDims d; if (!mobilebert_dims<F>(a, d, false, "mobilebert attention backward")) return;
    const size_t FL = (size_t)d.F * d.L, SM = (size_t)d.heads * d.L * d.L;
    Scope sc;
    const T *x = sc.in(a->input->data, (size_t)d.L * d.E), *xb = sc.in(a->input_bn->data, (size_t)d.L * d.Kb);
    const T *wq = sc.in(a->coeff_in_q->data, (size_t)d.F * d.Kb), *wk = sc.in(a->coeff_in_k->data, (size_t)d.F * d.Kb);
    const T *wv = sc.in(a->coeff_in_v->data, (size_t)d.F * d.E), *wo = sc.in(a->coeff_out->data, (size_t)d.No * d.F);
    const T *q = sc.in(a->q->data, FL), *k = sc.in(a->k->data, FL), *v = sc.in(a->v->data, FL);
    const T *sm = sc.in(a->softmax_buffer->data, SM), *att = sc.in(a->attention_map->data, FL), *dy = sc.in(a->output->diff, (size_t)d.L * d.No);
    T *dq = sc.out(a->q->diff, FL), *dk = sc.out(a->k->diff, FL), *dv = sc.out(a->v->diff, FL);
    T *dsm = sc.out(a->softmax_buffer->diff, SM), *datt = sc.out(a->attention_map->diff, FL);
    T *dwq = sc.out(a->coeff_in_q->diff, (size_t)d.F * d.Kb), *dwk = sc.out(a->coeff_in_k->diff, (size_t)d.F * d.Kb);
    T *dwv = sc.out(a->coeff_in_v->diff, (size_t)d.F * d.E), *dwo = sc.out(a->coeff_out->diff, (size_t)d.No * d.F);
    T *dx = sc.inout(a->input->diff, (size_t)d.L * d.E);
    T *dxb = nullptr;
    if (a->input_bn->diff && a->input_bn->diff != a->input->diff) dxb = sc.inout(a->input_bn->diff, (size_t)d.L * d.Kb);
    else if (d.Kb == d.E) dxb = dx;
    if (!sc.ok()) return;
    mhsa_mobilebert_bw<T>(sc, d, x, xb, wq, wk, wv, wo, q, k, v, sm, att, dy, dq, dk, dv, dsm, datt, dwq, dwk, dwv, dwo, dx, dxb);
}
// tiled_matmul_mhsa: the product of its matMul_args with the bias handling of mm_manager [ref: pulp_mhsa_fp32.c:2037-2109]
template <class F> void tiled_matmul_impl(void *mm_args)
{
    typename F::manager_t m;
    memset(&m, 0, sizeof(m));
    m.mm_args = (decltype(m.mm_args))mm_args; m.layer_type = LAYER_LINEAR; m.step_type = STEP_FW; m.matmul_type = 0;
    mm_manager_impl<F>(&m);
}

// ------------------------------------------------------------------ activations / softmax
template <class F, class A> void act_fw_impl(void *args, int kind, float slope)
{
    auto *a = (A *)args; typedef typename F::T T;
    const size_t n = (size_t)streams() * a->input->dim;
    Scope sc;
    const T *x = sc.in(a->input->data, n); T *y = sc.out(a->output->data, n);
    if (sc.ok()) act_fw<T>(kind, x, y, (long long)n, slope);
}
template <class F, class A> void act_bw_impl(void *args, int kind, float slope)
{
    auto *a = (A *)args; typedef typename F::T T;
    const size_t n = (size_t)streams() * a->input->dim;
    Scope sc;
    const T *x = (kind != ACT_SIGMOID) ? sc.in(a->input->data, n) : nullptr;
    const T *y = (kind == ACT_SIGMOID) ? sc.in(a->output->data, n) : nullptr;
    const T *dy = sc.in(a->output->diff, n); T *dx = sc.out(a->input->diff, n);
    if (sc.ok()) act_bw<T>(kind, x, y, dy, dx, (long long)n, slope);
}
template <class F> void softmax_fw_impl(void *args)
{
    auto *a = (typename F::softmax_t *)args; typedef typename F::T T;
    TL_REQUIRE(a->H > 0 && a->W > 0, "pulp_softmax_fw: H=%d W=%d", a->H, a->W);
    const size_t n = (size_t)a->H * a->W;
    Scope sc;
    const T *in = sc.in(a->input_data, n); T *out = sc.out(a->output_data, n);
    T *mx = a->maxes ? sc.out(a->maxes, (size_t)a->H) : nullptr, *sm = a->sums ? sc.out(a->sums, (size_t)a->H) : nullptr;
    if (sc.ok()) softmax_fw<T>(in, out, mx, sm, a->H, a->W, 1);
}
template <class F> void softmax_bw_impl(void *args)
{
    auto *a = (typename F::softmax_t *)args; typedef typename F::T T;
    TL_REQUIRE(a->H > 0 && a->W > 0, "pulp_softmax_bw: H=%d W=%d", a->H, a->W);
    const size_t n = (size_t)a->H * a->W;
    Scope sc;
    const T *out = sc.in(a->output_data, n), *dout = sc.in(a->output_diff, n);
    T *din = sc.out(a->input_diff, n), *sm = a->sums ? sc.out(a->sums, (size_t)a->H) : nullptr;
    if (sc.ok()) softmax_bw<T>(out, dout, din, sm, a->H, a->W, 1);
}

// ------------------------------------------------------------------ norms
static constexpr int STEP_BOTH_GRADS = 100;   // internal: parameter and input gradients in one pass
template <class F> void instnorm_impl(void *args, int step)
{
    auto *a = (typename F::instnorm_t *)args; typedef typename F::T T;
    const int C = a->input->C, D = a->input->H * a->input->W, n = streams();
    TL_REQUIRE(C > 0 && D > 0, "pulp_instnorm: C=%d HxW=%d", C, D);
    const size_t nx = (size_t)n * C * D, ns = (size_t)n * C;
    Scope sc;
    if (step == STEP_FW) {
        const bool frozen = a->freeze_running_params != 0;
        const T *x = sc.in(a->input->data, nx), *gb = sc.in(a->coeff->data, (size_t)2 * C);
        T *y = sc.out(a->output->data, nx);
        T *m = frozen ? sc.inout(a->running_mean, ns) : sc.out(a->running_mean, ns);
        T *v = frozen ? sc.inout(a->running_var, ns) : sc.out(a->running_var, ns);
        T *s = frozen ? sc.inout(a->running_stdev, ns) : sc.out(a->running_stdev, ns);
        if (sc.ok()) instnorm_fw<T>(x, y, gb, m, v, s, n, C, D, frozen, (float)EPSILON);
    } else if (step == STEP_IN_GRAD) {
        const T *x = sc.in(a->input->data, nx), *dy = sc.in(a->output->diff, nx), *gb = sc.in(a->coeff->data, (size_t)2 * C);
        const T *m = sc.in(a->running_mean, ns), *v = sc.in(a->running_var, ns), *s = sc.in(a->running_stdev, ns);
        T *dx = sc.out(a->input->diff, nx);
        if (sc.ok()) instnorm_bw_input<T>(x, dy, dx, gb, m, v, s, n, C, D);
    } else if (step == STEP_BOTH_GRADS) {
        const T *x = sc.in(a->input->data, nx), *dy = sc.in(a->output->diff, nx), *gb = sc.in(a->coeff->data, (size_t)2 * C);
        const T *m = sc.in(a->running_mean, ns), *v = sc.in(a->running_var, ns), *s = sc.in(a->running_stdev, ns);
        T *dx = sc.out(a->input->diff, nx);
        T *dgb = sc.out(a->coeff->diff, (size_t)2 * C);
        if (sc.ok()) instnorm_bw_both<T>(sc, x, dy, dx, dgb, gb, m, v, s, n, C, D);
    } else {
        const T *x = sc.in(a->input->data, nx), *dy = sc.in(a->output->diff, nx);
        const T *m = sc.in(a->running_mean, ns), *s = sc.in(a->running_stdev, ns);
        T *dgb = sc.out(a->coeff->diff, (size_t)2 * C);
        if (sc.ok()) instnorm_bw_param<T>(sc, x, dy, dgb, m, s, n, C, D);
    }
}

// Instance norm + optional skip sum + optional ReLU (extension; see the public header).
template <class F> void instnorm_act_impl(void *args, int backward)
{
    auto *f = (trainlib_instnorm_act_args *)args; typedef typename F::T T;
    TL_REQUIRE(f && f->norm, "trainlib_instnorm_act: norm=%p", f ? f->norm : nullptr);
    auto *a = (typename F::instnorm_t *)f->norm;
    auto *skip = (typename F::blob_t *)f->skip;
    const int C = a->input->C, D = a->input->H * a->input->W, n = streams();
    TL_REQUIRE(C > 0 && D > 0, "trainlib_instnorm_act: C=%d HxW=%d", C, D);
    const size_t nx = (size_t)n * C * D, ns = (size_t)n * C;
    Scope sc;
    if (!backward) {
        TL_REQUIRE(!skip || skip->dim == a->output->dim, "trainlib_instnorm_act_fw: skip dim %d, output dim %d", skip->dim, a->output->dim);
        const bool frozen = a->freeze_running_params != 0;
        const T *x = sc.in(a->input->data, nx), *gb = sc.in(a->coeff->data, (size_t)2 * C), *k = skip ? sc.in(skip->data, nx) : nullptr;
        T *y = sc.out(a->output->data, nx);
        T *m = frozen ? sc.inout(a->running_mean, ns) : sc.out(a->running_mean, ns);
        T *v = frozen ? sc.inout(a->running_var, ns) : sc.out(a->running_var, ns);
        T *s = frozen ? sc.inout(a->running_stdev, ns) : sc.out(a->running_stdev, ns);
        if (sc.ok()) instnorm_act_fw<T>(x, y, k, gb, m, v, s, n, C, D, frozen, (float)EPSILON, f->relu != 0);
        return;
    }
    TL_REQUIRE(f->relu != 0 && !skip, "trainlib_instnorm_act_bw: relu=%d skip=%p (mask the sum's gradient with pulp_relu_bw and call pulp_instnorm_bw)", f->relu, f->skip);
    const T *x = sc.in(a->input->data, nx), *y = sc.in(a->output->data, nx), *gb = sc.in(a->coeff->data, (size_t)2 * C);
    const T *m = sc.in(a->running_mean, ns), *v = sc.in(a->running_var, ns), *s = sc.in(a->running_stdev, ns);
    const T *dy2 = f->diff2 ? sc.in((const T *)f->diff2, nx) : nullptr;
    T *dy = sc.inout(a->output->diff, nx), *dx = sc.out(a->input->diff, nx), *dgb = sc.out(a->coeff->diff, (size_t)2 * C);
    if (sc.ok()) instnorm_relu_bw<T>(sc, x, y, dy, dy2, dx, dgb, gb, m, v, s, n, C, D);
}

// ------------------------------------------------------------------ losses, optimizer, residual, pooling
template <class F> void loss_impl(void *args, int kind, int backward)
{
    auto *a = (typename F::loss_t *)args; typedef typename F::T T;
    const int dim = a->output->dim, n = streams();
    TL_REQUIRE(dim > 0, "loss: empty output");
    Scope sc;
    const T *y = sc.in(a->output->data, (size_t)n * dim), *t = sc.in(a->target, (size_t)n * dim);
    if (!backward) {
        T *loss = sc.out(a->wr_loss, (size_t)n);
        if (!sc.ok()) return;
        if (kind == 0) mse_fw<T>(y, t, loss, dim, n); else ce_fw<T>(y, t, loss, dim, n);
    } else {
        T *dy = sc.out(a->output->diff, (size_t)n * dim);
        if (!sc.ok()) return;
        if (kind == 0) mse_bw<T>(y, t, dy, dim, n); else ce_bw<T>(y, t, dy, dim, n);
    }
}
template <class F> void sgd_impl(void *args)
{
    auto *a = (typename F::optim_t *)args; typedef typename F::T T;
    const float lr = F::f(a->learning_rate), lambda = F::f(a->weight_decay_lambda);
    if (ready()) defer_flush();                                   // the gradients read here may have their sums pending
    Scope sc;
    {
        const size_t n = (size_t)a->weights->dim;
        T *w = sc.inout(a->weights->data, n);
        T *g = lambda != 0.f ? sc.inout(a->weights->diff, n) : (T *)sc.in(a->weights->diff, n);
        if (sc.ok()) sgd<T>(w, g, (long long)n, lr, lambda);
    }
    if (a->use_biases == 1 && a->biases) {
        const size_t n = (size_t)a->biases->dim;
        T *w = sc.inout(a->biases->data, n);
        T *g = lambda != 0.f ? sc.inout(a->biases->diff, n) : (T *)sc.in(a->biases->diff, n);
        if (sc.ok()) sgd<T>(w, g, (long long)n, lr, lambda);
    }
}
template <class F> void residual_impl(void *args, int which)
{
    auto *a = (typename F::skip_t *)args; typedef typename F::T T;
    const int n = streams();
    Scope sc;
    if (which == 0) {            // out = skip + lout
        if (a->skip->dim != a->lout->dim || a->lout->dim != a->output->dim) {
            printf("\n[pulp_residualconn_fw]: Sizes of input and output activations not matching!!\n");
            set_error(TL_ERR_BAD_ARGS, "pulp_residualconn_fw: dims %d, %d, %d", a->skip->dim, a->lout->dim, a->output->dim);
            return;
        }
        const size_t m = (size_t)n * a->output->dim;
        const T *s = sc.in(a->skip->data, m), *l = sc.in(a->lout->data, m); T *o = sc.out(a->output->data, m);
        if (sc.ok()) add<T>(s, l, o, (long long)m);
    } else if (which == 1) {     // skip.diff += out.diff
        if (a->skip_in_grad != 0) return;
        if (a->skip->dim != a->output->dim) {
            printf("[pulp_sumnode_bw]: Sizes of input and output activations not matching!!\n");
            set_error(TL_ERR_BAD_ARGS, "pulp_sumnode_bw: dims %d, %d", a->skip->dim, a->output->dim);
            return;
        }
        const size_t m = (size_t)n * a->skip->dim;
        const T *o = sc.in(a->output->diff, m); T *s = sc.inout(a->skip->diff, m);
        if (sc.ok()) add<T>(o, s, s, (long long)m);
    } else {                     // lout.diff = out.diff
        if (a->lout->dim != a->output->dim) {
            printf("[pulp_residualconn_bw]: Sizes of input and output activations not matching!!\n");
            set_error(TL_ERR_BAD_ARGS, "pulp_residualconn_bw: dims %d, %d", a->lout->dim, a->output->dim);
            return;
        }
        const size_t m = (size_t)n * a->output->dim;
        const T *o = sc.in(a->output->diff, m); T *l = sc.out(a->lout->diff, m);
        if (sc.ok()) copy_n<T>(o, l, (long long)m);
    }
}
template <class F> void avgpool_impl(void *args, int backward)
{
    auto *a = (typename F::pool_t *)args; typedef typename F::T T;
    const int C = a->input->C, H = a->input->H, W = a->input->W, Ho = a->output->H, Wo = a->output->W, n = streams();
    TL_REQUIRE(a->Hstride >= 1 && a->Wstride >= 1 && a->Hker >= 1 && a->Wker >= 1, "pulp_avgpool: kernel/stride must be >= 1");
    if ((H - a->Hker + a->Hstride) / a->Hstride != Ho || (W - a->Wker + a->Wstride) / a->Wstride != Wo) {
        printf("\n[pulp_avgpool] Invalid pooling kernel size or output size!\n");
        set_error(TL_ERR_BAD_ARGS, "pulp_avgpool: output %dx%d does not match kernel/stride", Ho, Wo);
        return;
    }
    Scope sc;
    const size_t nx = (size_t)n * C * H * W, ny = (size_t)n * C * Ho * Wo;
    if (!backward) { const T *x = sc.in(a->input->data, nx); T *y = sc.out(a->output->data, ny); if (sc.ok()) avgpool_fw<T>(x, y, n, C, H, W, Ho, Wo, a->Hker, a->Wker, a->Hstride, a->Wstride); }
    else { const T *dy = sc.in(a->output->diff, ny); T *dx = sc.out(a->input->diff, nx); if (sc.ok()) avgpool_bw<T>(dy, dx, n, C, H, W, Ho, Wo, a->Hker, a->Wker, a->Hstride, a->Wstride); }
}

// ------------------------------------------------------------------ tensor helpers
template <class F> void transpose_matrix_impl(void *args)
{
    auto a = *(typename F::transp_t *)args; typedef typename F::T T;
    TL_REQUIRE(a.N > 0 && a.M > 0, "transpose_matrix: N=%d M=%d", a.N, a.M);
    int dims[2] = {a.N, a.M}, axes[2] = {1, 0};
    Scope sc;
    const T *in = sc.in(a.in_matrix, (size_t)a.N * a.M); T *out = sc.out(a.out_matrix, (size_t)a.N * a.M);
    if (sc.ok()) transpose_nd<T>(in, out, dims, axes, 2);
}
template <class F> void transpose_impl(void *args)
{
    auto a = *(typename F::transp_t *)args; typedef typename F::T T;
    TL_REQUIRE(a.n_dim >= 1 && a.n_dim <= 8 && a.dim && a.transposed_axes, "transpose: n_dim=%d", a.n_dim);
    size_t total = 1;
    for (int i = 0; i < a.n_dim; i++) total *= (size_t)a.dim[i];
    Scope sc;
    const T *in = sc.in(a.in_matrix, total); T *out = sc.out(a.out_matrix, total);
    if (sc.ok()) transpose_nd<T>(in, out, a.dim, a.transposed_axes, a.n_dim);
}
template <class F> void copy_impl(void *args)
{
    auto a = *(typename F::copy_t *)args; typedef typename F::T T;
    if (a.size <= 0) return;
    Scope sc;
    const T *f = sc.in(a.from, (size_t)a.size); T *t = sc.out(a.to, (size_t)a.size);
    if (sc.ok()) copy_n<T>(f, t, a.size);
}
template <class F> void setval_impl(void *args)
{
    auto a = *(typename F::setval_t *)args; typedef typename F::T T;
    if (a.size <= 0) return;
    Scope sc;
    T *t = sc.out(a.to, (size_t)a.size);
    if (sc.ok()) fill<T>(t, F::f(a.value), a.size);
}
template <class F> void vsum_impl(void *args)
{
    auto *a = (typename F::vsum_t *)args; typedef typename F::T T;
    if (a->size <= 0) return;
    Scope sc;
    const T *x = sc.in(a->op_1, (size_t)a->size), *y = sc.in(a->op_2, (size_t)a->size); T *d = sc.out(a->dest, (size_t)a->size);
    if (sc.ok()) add<T>(x, y, d, a->size);
}
template <class F> void bcast_impl(void *args)
{
    auto *a = (typename F::bcast_t *)args; typedef typename F::T T;
    TL_REQUIRE(a->op_1_dims_len >= 1 && a->op_2_dims_len >= 1 && a->op_1_dims_len <= 8 && a->op_2_dims_len <= 8, "array_broadcast_sum: rank outside 1..8");
    size_t n1 = 1, n2 = 1, no = 1;
    const int n = a->op_1_dims_len > a->op_2_dims_len ? a->op_1_dims_len : a->op_2_dims_len;
    for (int i = 0; i < a->op_1_dims_len; i++) n1 *= (size_t)a->op_1_dims[i];
    for (int i = 0; i < a->op_2_dims_len; i++) n2 *= (size_t)a->op_2_dims[i];
    for (int k = 0; k < n; k++) {
        int e1 = k < a->op_1_dims_len ? a->op_1_dims[a->op_1_dims_len - 1 - k] : 1, e2 = k < a->op_2_dims_len ? a->op_2_dims[a->op_2_dims_len - 1 - k] : 1;
        no *= (size_t)(e1 > e2 ? e1 : e2);
    }
    Scope sc;
    const T *x = sc.in(a->op_1, n1), *y = sc.in(a->op_2, n2); T *d = sc.out(a->dest, no);
    if (sc.ok()) broadcast_add<T>(x, y, d, a->op_1_dims, a->op_1_dims_len, a->op_2_dims, a->op_2_dims_len);
}
template <class F> void pad_impl(void *args)
{
    auto *a = (typename F::pad_t *)args; typedef typename F::T T;
    if (a->HWC_lay != 0 && a->HWC_lay != 1) { printf("[pad_tensor] HWC layout not implemented!!"); set_error(TL_ERR_BAD_ARGS, "pad_tensor: HWC_lay = %d", a->HWC_lay); return; }
    TL_REQUIRE(a->C > 0 && a->H > 0 && a->W > 0 && a->T_LPAD >= 0 && a->T_RPAD >= 0 && a->T_UPAD >= 0 && a->T_DPAD >= 0, "pad_tensor: invalid sizes");
    Scope sc;
    const T *s = sc.in(a->source, (size_t)a->C * a->H * a->W);
    T *d = sc.out(a->dest, (size_t)a->C * (a->H + a->T_UPAD + a->T_DPAD) * (a->W + a->T_LPAD + a->T_RPAD));
    if (sc.ok()) pad2d<T>(s, d, a->C, a->H, a->W, a->T_LPAD, a->T_RPAD, a->T_UPAD, a->T_DPAD, a->HWC_lay);
}
template <class F> void smul_impl(void *args)
{
    auto *a = (typename F::smul_t *)args; typedef typename F::T T;
    if (a->dim <= 0) return;
    Scope sc;
    T *x = sc.inout(a->input, (size_t)a->dim);
    if (sc.ok()) scale<T>(x, F::f(a->scalar), a->dim);
}
template <class F> void biasadd_impl(void *args)
{
    auto *a = (typename F::biasadd_t *)args; typedef typename F::T T;
    TL_REQUIRE(a->H > 0 && a->W > 0, "mm_bias_add_transposed: H=%d W=%d", a->H, a->W);
    Scope sc;
    T *m = sc.inout(a->mat, (size_t)a->H * a->W);
    const T *b = sc.in(a->bias, (size_t)(a->t ? a->H : a->W));
    if (sc.ok()) bias_add_rows<T>(m, b, a->H, a->W, a->t ? 1 : 0);
}

// HWC <-> CHW in place through the caller's buffer [ref: lib/sources/pulp_train_utils_fp32.c:821-927]
template <class T, class A_t> void layout_impl(void *args, int to_chw)
{
    auto *a = (A_t *)args;
    const int C = a->tensor->C, HW = a->tensor->H * a->tensor->W;
    const size_t n = (size_t)C * HW;
    int dims[2], axes[2] = {1, 0};
    if (to_chw) { dims[0] = HW; dims[1] = C; } else { dims[0] = C; dims[1] = HW; }
    T *targets[2] = {a->transpose_data == 1 ? (T *)a->tensor->data : nullptr, a->transpose_grad == 1 ? (T *)a->tensor->diff : nullptr};
    for (int t = 0; t < 2; t++) {
        if (!targets[t]) continue;
        Scope sc;
        T *x = sc.inout(targets[t], n);
        T *buf = sc.out((T *)a->transp_buffer, n);
        if (!sc.ok()) return;
        transpose_nd<T>(x, buf, dims, axes, 2);
        copy_n<T>(buf, x, (long long)n);
    }
}

} // namespace

// ==================================================================== exported symbols
#define TL_EXPORT extern "C" __attribute__((visibility("default")))

// ---- matmul family: every unrolled variant is the same product
#define TL_MM_VARIANTS(X)                                                                                        \
    X(mm) X(mm_M) X(mm_u2) X(mm_unroll_1x2) X(mm_unroll_1x4) X(mm_unroll_1x8) X(mm_unroll_2x1) X(mm_unroll_4x1)   \
    X(mm_unroll_8x1) X(mm_unroll_2x2) X(mm_unroll_2x4) X(mm_unroll_4x2) X(mm_unroll_4x4) X(mm_M_u2)               \
    X(mm_M_unroll_2x1) X(mm_M_unroll_4x1) X(mm_M_unroll_8x1) X(mm_M_unroll_1x2) X(mm_M_unroll_1x4)                \
    X(mm_M_unroll_1x8) X(mm_M_unroll_2x2) X(mm_M_unroll_4x2) X(mm_M_unroll_2x4) X(mm_M_unroll_4x4)
#define X(name) TL_EXPORT void name(void *a) { mm_impl<F32>(a, false); }
TL_MM_VARIANTS(X)
#undef X
TL_EXPORT void mm_add(void *a) { mm_impl<F32>(a, true); }
TL_EXPORT void mm_fp16(void *a) { mm_impl<F16>(a, false); }
TL_EXPORT void mm_M_fp16(void *a) { mm_impl<F16>(a, false); }
// fp16 variants by name [ref: lib/include/pulp_matmul_fp16.h:56-134]: mm_manager_fp16 selects them by matmul_type and the
// reference's tests fork them directly; every one is the same product (the matrix-vector forms are M = 1 products)
#define TL_MM16_VARIANTS(X) X(mm_fp16_SIMD_2x4) X(mm_fp16_SIMD_4x8) X(mm_fp16_unroll_8x1) X(mm_fp16_unroll_4x1) X(mm_fp16_unroll_2x1) \
    X(mm_M_fp16_SIMD_2x4) X(mm_M_fp16_SIMD_4x8) X(mv_fp16_SIMD_2x1) X(mv_fp16_SIMD_4x1) X(mv_fp16_SIMD_8x1)
#define X(name) TL_EXPORT void name(void *a) { mm_impl<F16>(a, false); }
TL_MM16_VARIANTS(X)
#undef X
TL_EXPORT void mm_manager(void *a) { mm_manager_impl<F32>(a); }
TL_EXPORT void mm_manager_fp16(void *a) { mm_manager_impl<F16>(a); }

// ---- the rest, fp32 name / fp16 name pairs
#define TL_PAIR(name32, name16, call32, call16)             \
    TL_EXPORT void name32(void *a) { call32; }              \
    TL_EXPORT void name16(void *a) { call16; }

TL_PAIR(pulp_im2row_fp32, pulp_im2row_fp16, im2row_impl<F32>(a, 0), im2row_impl<F16>(a, 0))
TL_PAIR(pulp_im2col_fp32, pulp_im2col_fp16, im2row_impl<F32>(a, 1), im2row_impl<F16>(a, 1))
TL_PAIR(pulp_blocktransp_fp32, pulp_blocktransp_fp16, blocktransp_impl<F32>(a), blocktransp_impl<F16>(a))

TL_PAIR(pulp_conv2d_fp32_fw_cl, pulp_conv2d_fp16_fw_cl, conv2d_fw_impl<F32>(a), conv2d_fw_impl<F16>(a))
TL_PAIR(pulp_conv2d_fp32_bw_param_grads_cl, pulp_conv2d_fp16_bw_param_grads_cl, conv2d_wg_impl<F32>(a), conv2d_wg_impl<F16>(a))
TL_PAIR(pulp_conv2d_fp32_bw_input_grads_cl, pulp_conv2d_fp16_bw_input_grads_cl, conv2d_ig_impl<F32>(a), conv2d_ig_impl<F16>(a))
TL_PAIR(trainlib_conv2d_fp32_bw_input_grads_acc_cl, trainlib_conv2d_fp16_bw_input_grads_acc_cl, conv2d_ig_impl<F32>(a, true), conv2d_ig_impl<F16>(a, true))
TL_EXPORT void pulp_conv2d_fp32_bw_cl(void *a)
{
    auto *c = (Conv2D_args *)a;
    if (c->skip_wg_grad == 0) pulp_conv2d_fp32_bw_param_grads_cl(a);
    if (c->skip_in_grad == 0) pulp_conv2d_fp32_bw_input_grads_cl(a);
}
TL_EXPORT void pulp_conv2d_fp16_bw_cl(void *a)
{
    auto *c = (Conv2D_args_fp16 *)a;
    if (c->skip_wg_grad == 0) pulp_conv2d_fp16_bw_param_grads_cl(a);
    if (c->skip_in_grad == 0) pulp_conv2d_fp16_bw_input_grads_cl(a);
}
TL_EXPORT void naive_conv2d_fw_kernel_CHW(void *a) { naive_impl<F32>(a, STEP_FW); }
TL_EXPORT void naive_conv2d_param_grad_kernel_CHW(void *a) { naive_impl<F32>(a, STEP_WGT_GRAD); }
TL_EXPORT void naive_conv2d_in_grad_kernel_CHW(void *a) { naive_impl<F32>(a, STEP_IN_GRAD); }
TL_EXPORT void naive_conv2d_fw_kernel_CHW_fp16(void *a) { naive_impl<F16>(a, STEP_FW); }
TL_EXPORT void naive_conv2d_param_grad_kernel_CHW_fp16(void *a) { naive_impl<F16>(a, STEP_WGT_GRAD); }
TL_EXPORT void naive_conv2d_in_grad_kernel_CHW_fp16(void *a) { naive_impl<F16>(a, STEP_IN_GRAD); }
// The fixed-geometry forms [ref: lib/sources/pulp_conv_naive_fp32.c:520-700]: kernel size, stride 2 and padding 1 are
// constants of the function, whatever the struct says; the remaining fields are read as by the generic kernels.
template <class F> static void naive_fixed(void *args, int step, int k)
{
    if (!args) { set_error(TL_ERR_BAD_ARGS, "naive conv2d: null arguments"); return; }
    typename F::matMul_t a = *(typename F::matMul_t *)args;
    a.pH = a.pW = k; a.stride_h = a.stride_w = 2; a.Lpad = a.Rpad = a.Upad = a.Dpad = 1;
    naive_impl<F>(&a, step);
}
#define TL_NAIVE_FIXED(K)                                                                                                              \
    TL_EXPORT void naive_conv2d_fw_kernel_CHW_k##K##x##K##_s2_p1(void *a) { naive_fixed<F32>(a, STEP_FW, K); }                           \
    TL_EXPORT void naive_conv2d_param_grad_kernel_CHW_k##K##x##K##_s2_p1(void *a) { naive_fixed<F32>(a, STEP_WGT_GRAD, K); }             \
    TL_EXPORT void naive_conv2d_in_grad_kernel_CHW_k##K##x##K##_s2_p1(void *a) { naive_fixed<F32>(a, STEP_IN_GRAD, K); }                 \
    TL_EXPORT void naive_conv2d_fw_kernel_CHW_k##K##x##K##_s2_p1_fp16(void *a) { naive_fixed<F16>(a, STEP_FW, K); }                      \
    TL_EXPORT void naive_conv2d_param_grad_kernel_CHW_k##K##x##K##_s2_p1_fp16(void *a) { naive_fixed<F16>(a, STEP_WGT_GRAD, K); }        \
    TL_EXPORT void naive_conv2d_in_grad_kernel_CHW_k##K##x##K##_s2_p1_fp16(void *a) { naive_fixed<F16>(a, STEP_IN_GRAD, K); }
TL_NAIVE_FIXED(3)
TL_NAIVE_FIXED(5)
#undef TL_NAIVE_FIXED

// Workers that the reference's layer functions fork with a mm_manager_args [ref: lib/sources/pulp_linear_fp32.c:199-267,
// lib/sources/pulp_conv2d_fp32.c:669-800]: the product of mm_args, then the worker's own bias step.
template <class F> static void manager_worker(void *args, int kind)
{
    auto *m = (typename F::manager_t *)args; typedef typename F::T T;
    if (!m || !m->mm_args) { set_error(TL_ERR_BAD_ARGS, "matmul worker: null arguments"); return; }
    auto *a = m->mm_args;
    mm_impl<F>(a, false);
    if (a->USE_BIASES != 1 || !a->bias) return;
    if (kind == 1) {                       // Linear weight gradient: the bias gradient is the output gradient (batch 1)
        Scope sc;
        const T *dy = sc.in(a->A, (size_t)a->N); T *db = sc.out(a->bias, (size_t)a->N);
        if (sc.ok()) copy_n<T>(dy, db, a->N);
    } else if (kind == 2) {                // im2col convolution forward: C is [C_out][pH*pW] (pH, pW = the output plane there), bias per row
        Scope sc;
        T *c = sc.inout(a->C, (size_t)a->N * a->M); const T *b = sc.in(a->bias, (size_t)a->N);
        if (sc.ok()) bias_add_rows<T>(c, b, a->N, a->M, 1);
    }
}
TL_EXPORT void pulp_linear_fp32_fw_cl_kernel(void *a) { manager_worker<F32>(a, 0); }               // (the reference leaves its bias step commented out)
TL_EXPORT void pulp_linear_fp16_fw_cl_kernel(void *a) { manager_worker<F16>(a, 0); }
TL_EXPORT void pulp_linear_fp32_bw_param_grads_cl_kernel(void *a) { manager_worker<F32>(a, 1); }
TL_EXPORT void pulp_linear_fp16_bw_param_grads_cl_kernel(void *a) { manager_worker<F16>(a, 1); }
TL_EXPORT void im2col_conv2d_fw_kernel(void *a) { manager_worker<F32>(a, 2); }
TL_EXPORT void im2col_conv2d_fw_kernel_fp16(void *a) { manager_worker<F16>(a, 2); }
// (weight gradient worker: the product only; the reference's bias-gradient loop there sums a tensor of the wrong
// shape, the layer-level entry point computes the channel sums itself)
TL_EXPORT void im2col_conv2d_param_grad_kernel(void *a) { manager_worker<F32>(a, 0); }
TL_EXPORT void im2col_conv2d_param_grad_kernel_fp16(void *a) { manager_worker<F16>(a, 0); }

TL_PAIR(pulp_conv_pw_fp32_fw_cl, pulp_conv_pw_fp16_fw_cl, pw_impl<F32>(a, STEP_FW), pw_impl<F16>(a, STEP_FW))
TL_PAIR(pulp_conv_pw_fp32_bw_param_grads_cl, pulp_conv_pw_fp16_bw_param_grads_cl, pw_impl<F32>(a, STEP_WGT_GRAD), pw_impl<F16>(a, STEP_WGT_GRAD))
TL_PAIR(pulp_conv_pw_fp32_bw_input_grads_cl, pulp_conv_pw_fp16_bw_input_grads_cl, pw_impl<F32>(a, STEP_IN_GRAD), pw_impl<F16>(a, STEP_IN_GRAD))
TL_EXPORT void pulp_conv_pw_fp32_bw_cl(void *a)
{
    auto *c = (PointWise_Conv_args *)a;
    if (c->skip_wg_grad == 0) pulp_conv_pw_fp32_bw_param_grads_cl(a);
    if (c->skip_in_grad == 0) pulp_conv_pw_fp32_bw_input_grads_cl(a);
}
TL_EXPORT void pulp_conv_pw_fp16_bw_cl(void *a)
{
    auto *c = (PointWise_Conv_args_fp16 *)a;
    if (c->skip_wg_grad == 0) pulp_conv_pw_fp16_bw_param_grads_cl(a);
    if (c->skip_in_grad == 0) pulp_conv_pw_fp16_bw_input_grads_cl(a);
}

#define DWK32(step) do { auto *k = (kernel_DW_args *)a; if (k) dwk_impl<float, kernel_DW_args>(a, step, k->stride_h, k->stride_w, k->Lpad, k->Rpad, k->Upad, k->Dpad); } while (0)
TL_EXPORT void dw_kernel_forward(void *a) { DWK32(STEP_FW); }
TL_EXPORT void dw_kernel_weight_grad(void *a) { DWK32(STEP_WGT_GRAD); }
TL_EXPORT void dw_kernel_input_grad(void *a) { DWK32(STEP_IN_GRAD); }
TL_EXPORT void dw_kernel_forward_fp16(void *a) { dwk_impl<__half, kernel_DW_args_fp16>(a, STEP_FW, 1, 1, 0, 0, 0, 0); }
TL_EXPORT void dw_kernel_weight_grad_fp16(void *a) { dwk_impl<__half, kernel_DW_args_fp16>(a, STEP_WGT_GRAD, 1, 1, 0, 0, 0, 0); }
TL_EXPORT void dw_kernel_input_grad_fp16(void *a) { dwk_impl<__half, kernel_DW_args_fp16>(a, STEP_IN_GRAD, 1, 1, 0, 0, 0, 0); }
TL_PAIR(pulp_conv_dw_fp32_fw_cl, pulp_conv_dw_fp16_fw_cl, dw_impl<F32>(a, STEP_FW), dw_impl<F16>(a, STEP_FW))
TL_PAIR(pulp_conv_dw_fp32_bw_param_grads_cl, pulp_conv_dw_fp16_bw_param_grads_cl, dw_impl<F32>(a, STEP_WGT_GRAD), dw_impl<F16>(a, STEP_WGT_GRAD))
TL_PAIR(pulp_conv_dw_fp32_bw_input_grads_cl, pulp_conv_dw_fp16_bw_input_grads_cl, dw_impl<F32>(a, STEP_IN_GRAD), dw_impl<F16>(a, STEP_IN_GRAD))
TL_EXPORT void pulp_conv_dw_fp32_bw_cl(void *a)
{
    auto *c = (DepthWise_Conv_args *)a;
    if (c->skip_wg_grad == 0) pulp_conv_dw_fp32_bw_param_grads_cl(a);
    if (c->skip_in_grad == 0) pulp_conv_dw_fp32_bw_input_grads_cl(a);
}
TL_EXPORT void pulp_conv_dw_fp16_bw_cl(void *a)
{
    auto *c = (DepthWise_Conv_args_fp16 *)a;
    if (c->skip_wg_grad == 0) pulp_conv_dw_fp16_bw_param_grads_cl(a);
    if (c->skip_in_grad == 0) pulp_conv_dw_fp16_bw_input_grads_cl(a);
}

TL_EXPORT void mm_broadcast_fp32(void *a) { mm_broadcast_impl<float, broadcastMatMul_args_fp32>(a); }
TL_EXPORT void mm_broadcast_fp16(void *a) { mm_broadcast_impl<__half, broadcastMatMul_args_fp16>(a); }
TL_PAIR(pulp_linear_fp32_fw_cl, pulp_linear_fp16_fw_cl, linear_impl<F32>(a, STEP_FW), linear_impl<F16>(a, STEP_FW))
TL_PAIR(pulp_linear_fp32_bw_param_grads_cl, pulp_linear_fp16_bw_param_grads_cl, linear_impl<F32>(a, STEP_WGT_GRAD), linear_impl<F16>(a, STEP_WGT_GRAD))
TL_PAIR(pulp_linear_fp32_bw_input_grads_cl, pulp_linear_fp16_bw_input_grads_cl, linear_impl<F32>(a, STEP_IN_GRAD), linear_impl<F16>(a, STEP_IN_GRAD))
TL_EXPORT void pulp_linear_fp32_bw_cl(void *a)
{
    auto *c = (Linear_args *)a;
    if (c->skip_wg_grad == 0 && c->skip_in_grad == 0 && linear_bw_both<F32>(a)) return;
    if (c->skip_wg_grad == 0) pulp_linear_fp32_bw_param_grads_cl(a);
    if (c->skip_in_grad == 0) pulp_linear_fp32_bw_input_grads_cl(a);
}
TL_EXPORT void pulp_linear_fp16_bw_cl(void *a)
{
    auto *c = (Linear_args_fp16 *)a;
    if (c->skip_wg_grad == 0 && c->skip_in_grad == 0 && linear_bw_both<F16>(a)) return;
    if (c->skip_wg_grad == 0) pulp_linear_fp16_bw_param_grads_cl(a);
    if (c->skip_in_grad == 0) pulp_linear_fp16_bw_input_grads_cl(a);
}

TL_PAIR(pulp_mhsa_fp32_fw_cl, pulp_mhsa_fp16_fw_cl, mhsa_fw_impl<F32>(a), mhsa_fw_impl<F16>(a))
TL_PAIR(pulp_mhsa_fp32_bw_cl, pulp_mhsa_fp16_bw_cl, mhsa_bw_impl<F32>(a), mhsa_bw_impl<F16>(a))
TL_PAIR(pulp_mhsa_mobilebert_inference_fp32_fw_cl, pulp_mhsa_mobilebert_inference_fp16_fw_cl, mobilebert_fw_impl<F32>(a, false), mobilebert_fw_impl<F16>(a, false))
TL_PAIR(pulp_mhsa_mobilebert_inference_fp32_bw_cl, pulp_mhsa_mobilebert_inference_fp16_bw_cl, mobilebert_bw_impl<F32>(a), mobilebert_bw_impl<F16>(a))
TL_EXPORT void tiled_mhsa_fp32(void *a, void *) { mobilebert_fw_impl<F32>(a, true); }
TL_EXPORT void tiled_mhsa_fp16(void *a, void *) { mobilebert_fw_impl<F16>(a, true); }
TL_EXPORT void tiled_matmul_mhsa(void *a, void *, int) { tiled_matmul_impl<F32>(a); }
TL_EXPORT void tiled_matmul_mhsa_fp16(void *a, void *, int) { tiled_matmul_impl<F16>(a); }

#define ACT32(kind) act_fw_impl<F32, act_args>(a, kind, 0.f)
#define ACT16(kind) act_fw_impl<F16, act_args_fp16>(a, kind, 0.f)
#define ACTB32(kind) act_bw_impl<F32, act_args>(a, kind, 0.f)
#define ACTB16(kind) act_bw_impl<F16, act_args_fp16>(a, kind, 0.f)
TL_PAIR(pulp_relu_fp32_fw_cl, pulp_relu_fp16_fw_cl, ACT32(ACT_RELU), ACT16(ACT_RELU))
TL_PAIR(pulp_relu_fp32_bw_cl, pulp_relu_fp16_bw_cl, ACTB32(ACT_RELU), ACTB16(ACT_RELU))
TL_PAIR(relu_core_fw_fp32, relu_core_fw_fp16, ACT32(ACT_RELU), ACT16(ACT_RELU))
TL_PAIR(relu_core_bw_fp32, relu_core_bw_fp16, ACTB32(ACT_RELU), ACTB16(ACT_RELU))
TL_PAIR(pulp_sigmoid_fp32_fw_cl, pulp_sigmoid_fp16_fw_cl, ACT32(ACT_SIGMOID), ACT16(ACT_SIGMOID))
TL_PAIR(pulp_sigmoid_fp32_bw_cl, pulp_sigmoid_fp16_bw_cl, ACTB32(ACT_SIGMOID), ACTB16(ACT_SIGMOID))
TL_EXPORT void sigmoid_core_fw_fp32(void *a) { ACT32(ACT_SIGMOID); }
TL_EXPORT void sigmoid_core_bw_fp32(void *a) { ACTB32(ACT_SIGMOID); }
TL_EXPORT void sigmoid_core_fw_fp16(void *a) { ACT16(ACT_SIGMOID); }
TL_EXPORT void sigmoid_core_bw_fp16(void *a) { ACTB16(ACT_SIGMOID); }
TL_PAIR(pulp_gelu_tanh_approx_fp32_fw_cl, pulp_gelu_fp16_fw_cl, ACT32(ACT_GELU), ACT16(ACT_GELU))
TL_EXPORT void pulp_leakyrelu_fp32_fw_cl(void *a) { act_fw_impl<F32, leakyrelu_args>(a, ACT_LEAKY, ((leakyrelu_args *)a)->negative_slope); }
TL_EXPORT void pulp_leakyrelu_fp32_bw_cl(void *a) { act_bw_impl<F32, leakyrelu_args>(a, ACT_LEAKY, ((leakyrelu_args *)a)->negative_slope); }
TL_EXPORT void leakyrelu_core_fw_fp32(void *a) { pulp_leakyrelu_fp32_fw_cl(a); }
TL_EXPORT void leakyrelu_core_bw_fp32(void *a) { pulp_leakyrelu_fp32_bw_cl(a); }
TL_EXPORT void pulp_leakyrelu_fp16_fw_cl(void *a) { act_fw_impl<F16, leakyrelu_args_fp16>(a, ACT_LEAKY, __half2float(((leakyrelu_args_fp16 *)a)->negative_slope)); }
TL_EXPORT void pulp_leakyrelu_fp16_bw_cl(void *a) { act_bw_impl<F16, leakyrelu_args_fp16>(a, ACT_LEAKY, __half2float(((leakyrelu_args_fp16 *)a)->negative_slope)); }
TL_EXPORT void leakyrelu_core_fw_fp16(void *a) { pulp_leakyrelu_fp16_fw_cl(a); }
TL_EXPORT void leakyrelu_core_bw_fp16(void *a) { pulp_leakyrelu_fp16_bw_cl(a); }
TL_PAIR(pulp_softmax_fp32_fw_cl, pulp_softmax_fp16_fw_cl, softmax_fw_impl<F32>(a), softmax_fw_impl<F16>(a))
TL_PAIR(pulp_softmax_fp32_bw_cl, pulp_softmax_fp16_bw_cl, softmax_bw_impl<F32>(a), softmax_bw_impl<F16>(a))

TL_PAIR(pulp_instnorm_fp32_fw_cl, pulp_instnorm_fp16_fw_cl, instnorm_impl<F32>(a, STEP_FW), instnorm_impl<F16>(a, STEP_FW))
TL_PAIR(pulp_instnorm_fp32_bw_param_grads_cl, pulp_instnorm_fp16_bw_param_grads_cl, instnorm_impl<F32>(a, STEP_WGT_GRAD), instnorm_impl<F16>(a, STEP_WGT_GRAD))
TL_PAIR(pulp_instnorm_fp32_bw_input_grads_cl, pulp_instnorm_fp16_bw_input_grads_cl, instnorm_impl<F32>(a, STEP_IN_GRAD), instnorm_impl<F16>(a, STEP_IN_GRAD))
TL_PAIR(trainlib_instnorm_act_fp32_fw_cl, trainlib_instnorm_act_fp16_fw_cl, instnorm_act_impl<F32>(a, 0), instnorm_act_impl<F16>(a, 0))
TL_PAIR(trainlib_instnorm_act_fp32_bw_cl, trainlib_instnorm_act_fp16_bw_cl, instnorm_act_impl<F32>(a, 1), instnorm_act_impl<F16>(a, 1))
TL_EXPORT void pulp_instnorm_parallelized_fp32_fw_cl(void *a) { instnorm_impl<F32>(a, STEP_FW); }
TL_EXPORT void pulp_instnorm_parallelized_fp32_bw_input_grads_cl(void *a) { instnorm_impl<F32>(a, STEP_IN_GRAD); }
TL_EXPORT void pulp_instnorm_parallelized_fp32_bw_param_grads_cl(void *a) { instnorm_impl<F32>(a, STEP_WGT_GRAD); }
TL_EXPORT void pulp_instnorm_parallelized_fp16_fw_cl(void *a) { instnorm_impl<F16>(a, STEP_FW); }
TL_EXPORT void pulp_instnorm_parallelized_fp16_bw_input_grads_cl(void *a) { instnorm_impl<F16>(a, STEP_IN_GRAD); }
TL_EXPORT void pulp_instnorm_parallelized_fp16_bw_param_grads_cl(void *a) { instnorm_impl<F16>(a, STEP_WGT_GRAD); }
TL_EXPORT void pulp_instnorm_fp32_bw_cl(void *a)
{
    auto *c = (InstNorm_args *)a;
    if (c->skip_wg_grad == 0 && c->skip_in_grad == 0) { instnorm_impl<F32>(a, STEP_BOTH_GRADS); return; }
    if (c->skip_wg_grad == 0) instnorm_impl<F32>(a, STEP_WGT_GRAD);
    if (c->skip_in_grad == 0) instnorm_impl<F32>(a, STEP_IN_GRAD);
}
TL_EXPORT void pulp_instnorm_fp16_bw_cl(void *a)
{
    auto *c = (InstNorm_args_fp16 *)a;
    if (c->skip_wg_grad == 0 && c->skip_in_grad == 0) { instnorm_impl<F16>(a, STEP_BOTH_GRADS); return; }
    if (c->skip_wg_grad == 0) instnorm_impl<F16>(a, STEP_WGT_GRAD);
    if (c->skip_in_grad == 0) instnorm_impl<F16>(a, STEP_IN_GRAD);
}
TL_EXPORT void pulp_batch_norm_fp32_fw_cl(void *args)
{
    auto *a = (BatchNorm_args_fp32 *)args;
    TL_REQUIRE(a->B > 0 && a->C > 0 && a->H > 0 && a->W > 0 && a->eps, "pulp_batch_norm: B=%d C=%d H=%d W=%d", a->B, a->C, a->H, a->W);
    const int n = streams();
    const size_t tot = (size_t)n * a->B * a->C * a->H * a->W;
    Scope sc;
    const float *x = sc.in(a->input->data, tot), *w = sc.in(a->weight_data, (size_t)a->C), *b = sc.in(a->bias_data, (size_t)a->C);
    const float *eps = sc.in(a->eps, 1);
    float *y = sc.out(a->output->data, tot);
    if (!sc.ok()) return;
    float eps_h = 0.f;
    if (is_device_pointer(a->eps)) { if (trainlib_memcpy_d2h(&eps_h, eps, sizeof(float)) != TL_OK) return; } else eps_h = a->eps[0];
    batchnorm_fw<float>(x, y, w, b, n, a->B, a->C, a->H * a->W, eps_h);
}
TL_EXPORT void pulp_batch_norm_parallelized_fp32_fw_cl(void *a) { pulp_batch_norm_fp32_fw_cl(a); }
template <class T> static bool layernorm_eps(Scope &sc, void *eps_ptr, float &eps_h)
{
    // eps is consumed on the host: a host pointer is read in place (no staging, no synchronisation, so the call can be
    // recorded into a CUDA graph); a device pointer costs one blocking copy
    (void)sc;
    T h;
    if (is_device_pointer(eps_ptr)) { if (trainlib_memcpy_d2h(&h, eps_ptr, sizeof(T)) != TL_OK) return false; } else h = *(T *)eps_ptr;
    eps_h = (float)h;
    return true;
}
TL_EXPORT void pulp_layerNorm_fp32_fw_cl(void *args)
{
    auto *a = (LayerNorm_args_fp32 *)args;
    TL_REQUIRE(a->size > 0 && a->step_size > 0 && a->size % a->step_size == 0 && a->eps, "pulp_layerNorm: size=%d step_size=%d", a->size, a->step_size);
    Scope sc;
    const float *x = sc.in(a->x, (size_t)a->size), *w = sc.in(a->weight, (size_t)a->step_size), *b = sc.in(a->bias, (size_t)a->step_size);
    float *y = sc.out(a->output, (size_t)a->size);
    if (!sc.ok()) return;
    float eps_h = 0.f;
    if (!layernorm_eps<float>(sc, a->eps, eps_h)) return;
    layernorm_fw<float>(x, y, w, b, a->size / a->step_size, a->step_size, eps_h);
}

// layer norm for fp16 and the backward passes (extensions: the reference stops at the fp32 forward)
template <class T> static void layernorm_ext(void *args, bool backward)
{
    auto *a = (trainlib_layernorm_args *)args;
    TL_REQUIRE(a && a->size > 0 && a->step_size > 0 && a->size % a->step_size == 0 && a->eps, "trainlib_layernorm: size=%d step_size=%d", a ? a->size : 0, a ? a->step_size : 0);
    const int rows = a->size / a->step_size, width = a->step_size;
    Scope sc;
    float eps_h = 0.f;
    if (!layernorm_eps<T>(sc, a->eps, eps_h)) return;
    const T *x = sc.in((T *)a->x, (size_t)a->size), *w = sc.in((T *)a->weight, (size_t)width);
    if (!backward) {
        const T *b = sc.in((T *)a->bias, (size_t)width);
        T *y = sc.out((T *)a->output, (size_t)a->size);
        if (sc.ok()) layernorm_fw<T>(x, y, w, b, rows, width, eps_h);
    } else {
        const T *dy = sc.in((T *)a->dy, (size_t)a->size);
        T *dx = sc.out((T *)a->dx, (size_t)a->size), *dw = sc.out((T *)a->dweight, (size_t)width), *db = sc.out((T *)a->dbias, (size_t)width);
        if (sc.ok()) layernorm_bw<T>(sc, x, w, dy, dx, dw, db, rows, width, eps_h);
    }
}
TL_EXPORT void trainlib_layernorm_fp16_fw_cl(void *a) { layernorm_ext<__half>(a, false); }
TL_EXPORT void trainlib_layernorm_fp32_bw_cl(void *a) { layernorm_ext<float>(a, true); }
TL_EXPORT void trainlib_layernorm_fp16_bw_cl(void *a) { layernorm_ext<__half>(a, true); }
TL_EXPORT void trainlib_gelu_fp32_bw_cl(void *a) { ACTB32(ACT_GELU); }
TL_EXPORT void trainlib_gelu_fp16_bw_cl(void *a) { ACTB16(ACT_GELU); }

TL_PAIR(pulp_MSELoss, pulp_MSELoss_fp16, loss_impl<F32>(a, 0, 0), loss_impl<F16>(a, 0, 0))
TL_PAIR(pulp_MSELoss_backward, pulp_MSELoss_backward_fp16, loss_impl<F32>(a, 0, 1), loss_impl<F16>(a, 0, 1))
TL_PAIR(pulp_CrossEntropyLoss, pulp_CrossEntropyLoss_fp16, loss_impl<F32>(a, 1, 0), loss_impl<F16>(a, 1, 0))
TL_PAIR(pulp_CrossEntropyLoss_backward, pulp_CrossEntropyLoss_backward_fp16, loss_impl<F32>(a, 1, 1), loss_impl<F16>(a, 1, 1))
TL_PAIR(pulp_gradient_descent_fp32, pulp_gradient_descent_fp16, sgd_impl<F32>(a), sgd_impl<F16>(a))
TL_PAIR(pulp_residualconn_fp32_fw, pulp_residualconn_fp16_fw, residual_impl<F32>(a, 0), residual_impl<F16>(a, 0))
TL_PAIR(pulp_sumnode_fp32_bw, pulp_sumnode_fp16_bw, residual_impl<F32>(a, 1), residual_impl<F16>(a, 1))
TL_PAIR(pulp_residualconn_fp32_bw, pulp_residualconn_fp16_bw, residual_impl<F32>(a, 2), residual_impl<F16>(a, 2))
TL_PAIR(pulp_avgpool_fp32_fw_cl, pulp_avgpool_fp16_fw_cl, avgpool_impl<F32>(a, 0), avgpool_impl<F16>(a, 0))
TL_PAIR(pulp_avgpool_fp32_bw_cl, pulp_avgpool_fp16_bw_cl, avgpool_impl<F32>(a, 1), avgpool_impl<F16>(a, 1))

TL_PAIR(transpose_matrix, transpose_matrix_fp16, transpose_matrix_impl<F32>(a), transpose_matrix_impl<F16>(a))
// tiled_transpose_mhsa: out[j][i] = in[i][j] for the N x M matrix of transp_args [ref: pulp_mhsa_fp32.c:2111-2160]
TL_EXPORT void tiled_transpose_mhsa(void *a, void *, int) { transpose_matrix_impl<F32>(a); }
TL_EXPORT void tiled_transpose_mhsa_fp16(void *a, void *, int) { transpose_matrix_impl<F16>(a); }
TL_PAIR(transpose, transpose_fp16, transpose_impl<F32>(a), transpose_impl<F16>(a))
TL_PAIR(copy, copy_fp16, copy_impl<F32>(a), copy_impl<F16>(a))
TL_PAIR(set_to_value, set_to_value_fp16, setval_impl<F32>(a), setval_impl<F16>(a))
TL_PAIR(vect_sum, vect_sum_fp16, vsum_impl<F32>(a), vsum_impl<F16>(a))
TL_PAIR(array_broadcast_sum_fp32, array_broadcast_sum_fp16, bcast_impl<F32>(a), bcast_impl<F16>(a))
TL_PAIR(pad_tensor, pad_tensor_fp16, pad_impl<F32>(a), pad_impl<F16>(a))
TL_PAIR(pulp_scalar_mul_fp32_cl, pulp_scalar_mul_fp16_cl, smul_impl<F32>(a), smul_impl<F16>(a))
TL_PAIR(mm_bias_add_transposed, mm_bias_add_transposed_fp16, biasadd_impl<F32>(a), biasadd_impl<F16>(a))
TL_EXPORT void HWC_to_CHW(void *a) { layout_impl<float, layout_args>(a, 1); }
TL_EXPORT void CHW_to_HWC(void *a) { layout_impl<float, layout_args>(a, 0); }
TL_EXPORT void HWC_to_CHW_fp16(void *a) { layout_impl<__half, layout_args_fp16>(a, 1); }
TL_EXPORT void CHW_to_HWC_fp16(void *a) { layout_impl<__half, layout_args_fp16>(a, 0); }

TL_EXPORT void pulp_row_max_fp32_cl(void *args)
{
    auto *a = (max_args *)args;
    TL_REQUIRE(a->H > 0 && a->W > 0, "pulp_row_max: H=%d W=%d", a->H, a->W);
    Scope sc;
    const float *in = sc.in(a->input, (size_t)a->H * a->W); float *mx = sc.inout(a->maxes, (size_t)a->H);
    if (sc.ok()) row_max<float>(in, mx, a->H, a->W);
}
TL_EXPORT void pulp_exp_sum_fp32_cl(void *args)
{
    auto *a = (exp_sum_args *)args;
    TL_REQUIRE(a->H > 0 && a->W > 0, "pulp_exp_sum: H=%d W=%d", a->H, a->W);
    Scope sc;
    const size_t n = (size_t)a->H * a->W;
    const float *in = sc.in(a->input, n), *mx = sc.in(a->maxes, (size_t)a->H);
    float *out = sc.out(a->output, n), *sm = sc.inout(a->sums, (size_t)a->H);
    if (sc.ok()) exp_sum<float>(in, out, mx, sm, a->H, a->W);
}
TL_EXPORT void pulp_row_div_fp32_cl(void *args)
{
    auto *a = (row_div_args *)args;
    TL_REQUIRE(a->H > 0 && a->W > 0, "pulp_row_div: H=%d W=%d", a->H, a->W);
    Scope sc;
    float *io = sc.inout(a->input, (size_t)a->H * a->W); const float *sm = sc.in(a->sums, (size_t)a->H);
    if (sc.ok()) row_div<float>(io, sm, a->H, a->W);
}
TL_EXPORT void pulp_mean_std_fp32_cl(void *args)
{
    auto *a = (mean_std_args *)args;
    TL_REQUIRE(a->dim > 0, "pulp_mean_std: dim=%d", a->dim);
    Scope sc;
    const float *x = sc.in(a->input, (size_t)a->dim);
    float *m = sc.out(a->mean, 1), *v = sc.out(a->var, 1), *s = sc.out(a->std, 1);
    if (sc.ok()) mean_std<float>(x, m, v, s, a->dim, a->epsilon);
}
TL_EXPORT void cast_fp16_tensor_to_fp32(void *args)
{
    auto a = *(cast_16t32_args *)args;
    if (a.size <= 0) return;
    Scope sc;
    const __half *s = sc.in(a.source, (size_t)a.size); float *d = sc.out(a.destination, (size_t)a.size);
    if (sc.ok()) cast_h2f(s, d, a.size);
}
TL_EXPORT void cast_fp32_tensor_to_fp16(void *args)
{
    auto a = *(cast_32t16_args *)args;
    if (a.size <= 0) return;
    Scope sc;
    const float *s = sc.in(a.source, (size_t)a.size); __half *d = sc.out(a.destination, (size_t)a.size);
    if (sc.ok()) cast_f2h(s, d, a.size);
}

// Host-side scalars with the reference's bit tricks [ref: lib/sources/pulp_train_utils_fp32.c:1223-1247]
TL_EXPORT float fastexp_gist(float x)
{
    volatile float t = GIST_A * x;      // keep multiply and add separately rounded
    x = t + GIST_B;
    if (x < GIST_C || x > GIST_D) x = (x < GIST_C) ? 0.0f : (float)GIST_D;
    uint32_t n = (uint32_t)x;
    float r; memcpy(&r, &n, sizeof r);
    return r;
}
TL_EXPORT float q_rsqrt(float number)
{
    int32_t i; float y = number;
    const float x2 = number * 0.5f;
    memcpy(&i, &y, sizeof i);
    i = 0x5f3759df - (i >> 1);
    memcpy(&y, &i, sizeof y);
    return y * (1.5f - (x2 * y * y));
}
// [ref: lib/sources/pulp_train_utils_fp32.c:25-37] host arrays only
TL_EXPORT int verify_tensor(float *tensor_out, float *tensor_ref, int size, float tolerance)
{
    int error_flag = 0;
    for (int i = 0; i < size; i++) {
        if (fabsf(tensor_out[i] - tensor_ref[i]) > tolerance) {
            if (!error_flag) printf("\n");
            printf("Error at index: %d   (Ideal = %.16f  vs  Actual = %.16f)\n", i, tensor_ref[i], tensor_out[i]);
            error_flag = 1;
        }
    }
    return error_flag;
}

// ---- table of library workers for pi_cl_team_fork
typedef void (*worker_t)(void *);
static const worker_t g_workers[] = {
    dw_kernel_forward, dw_kernel_weight_grad, dw_kernel_input_grad, dw_kernel_forward_fp16, dw_kernel_weight_grad_fp16, dw_kernel_input_grad_fp16,
    pulp_L1Loss, pulp_L1Loss_backward, pulp_L1Loss_fp16, pulp_L1Loss_backward_fp16, pulp_berHuLoss, pulp_berHuLoss_backward,
    pulp_berHuLoss_fp16, pulp_berHuLoss_backward_fp16, pulp_maxpool_fp32_fw_cl, pulp_maxpool_fp32_bw_cl, pulp_maxpool_fp16_fw_cl,
    pulp_maxpool_fp16_bw_cl, pulp_nonorm_fp32_fw_cl, pulp_nonorm_fp16_fw_cl, weighted_scaling_fp32_cl, weighted_scaling_fp16_cl,
    sum_of_squares_fp32_cl, sum_of_squares_fp16_cl, pulp_swiglu_fp32_cl, pulp_swiglu_fp16_cl, pulp_max_fp32_cl, pulp_max_fp16_cl,
    pulp_div_fp32_cl, pulp_div_fp16_cl, pulp_shift_sum_fp32_cl, vector_exp_sum_fp32_cl, vector_exp_sum_fp16_cl,
    pulp_sm_bw_op_1, pulp_sm_bw_op_1_fp16, pulp_sm_bw_op_2, pulp_sm_bw_op_2_fp16, pulp_row_max_fp16_cl, pulp_exp_sum_fp16_cl,
    pulp_row_div_fp16_cl, pulp_mean_std_fp16_cl, sigmoid_core_fw_fp16, sigmoid_core_bw_fp16, leakyrelu_core_fw_fp16, leakyrelu_core_bw_fp16,
    pulp_instnorm_parallelized_fp16_fw_cl, pulp_instnorm_parallelized_fp16_bw_input_grads_cl, pulp_instnorm_parallelized_fp16_bw_param_grads_cl,
#define X(name) name,
    TL_MM_VARIANTS(X)
#undef X
    mm_add, mm_fp16, mm_M_fp16, mm_manager, mm_manager_fp16,
    pulp_im2row_fp32, pulp_im2row_fp16, pulp_im2col_fp32, pulp_im2col_fp16, pulp_blocktransp_fp32, pulp_blocktransp_fp16,
    pulp_conv2d_fp32_fw_cl, pulp_conv2d_fp16_fw_cl, pulp_conv2d_fp32_bw_cl, pulp_conv2d_fp16_bw_cl,
    pulp_conv2d_fp32_bw_param_grads_cl, pulp_conv2d_fp16_bw_param_grads_cl, pulp_conv2d_fp32_bw_input_grads_cl, pulp_conv2d_fp16_bw_input_grads_cl,
    naive_conv2d_fw_kernel_CHW, naive_conv2d_param_grad_kernel_CHW, naive_conv2d_in_grad_kernel_CHW,
    naive_conv2d_fw_kernel_CHW_fp16, naive_conv2d_param_grad_kernel_CHW_fp16, naive_conv2d_in_grad_kernel_CHW_fp16,
    naive_conv2d_fw_kernel_CHW_k3x3_s2_p1, naive_conv2d_param_grad_kernel_CHW_k3x3_s2_p1, naive_conv2d_in_grad_kernel_CHW_k3x3_s2_p1,
    naive_conv2d_fw_kernel_CHW_k5x5_s2_p1, naive_conv2d_param_grad_kernel_CHW_k5x5_s2_p1, naive_conv2d_in_grad_kernel_CHW_k5x5_s2_p1,
    naive_conv2d_fw_kernel_CHW_k3x3_s2_p1_fp16, naive_conv2d_param_grad_kernel_CHW_k3x3_s2_p1_fp16, naive_conv2d_in_grad_kernel_CHW_k3x3_s2_p1_fp16,
    naive_conv2d_fw_kernel_CHW_k5x5_s2_p1_fp16, naive_conv2d_param_grad_kernel_CHW_k5x5_s2_p1_fp16, naive_conv2d_in_grad_kernel_CHW_k5x5_s2_p1_fp16,
    pulp_linear_fp32_fw_cl_kernel, pulp_linear_fp16_fw_cl_kernel, pulp_linear_fp32_bw_param_grads_cl_kernel, pulp_linear_fp16_bw_param_grads_cl_kernel,
    im2col_conv2d_fw_kernel, im2col_conv2d_fw_kernel_fp16, im2col_conv2d_param_grad_kernel, im2col_conv2d_param_grad_kernel_fp16,
    mm_fp16_SIMD_2x4, mm_fp16_SIMD_4x8, mm_fp16_unroll_8x1, mm_fp16_unroll_4x1, mm_fp16_unroll_2x1, mm_M_fp16_SIMD_2x4, mm_M_fp16_SIMD_4x8,
    mv_fp16_SIMD_2x1, mv_fp16_SIMD_4x1, mv_fp16_SIMD_8x1, HWC_to_CHW_fp16, CHW_to_HWC_fp16,
    pulp_conv_pw_fp32_fw_cl, pulp_conv_pw_fp16_fw_cl, pulp_conv_pw_fp32_bw_cl, pulp_conv_pw_fp16_bw_cl,
    pulp_conv_pw_fp32_bw_param_grads_cl, pulp_conv_pw_fp16_bw_param_grads_cl, pulp_conv_pw_fp32_bw_input_grads_cl, pulp_conv_pw_fp16_bw_input_grads_cl,
    pulp_conv_dw_fp32_fw_cl, pulp_conv_dw_fp16_fw_cl, pulp_conv_dw_fp32_bw_cl, pulp_conv_dw_fp16_bw_cl,
    pulp_conv_dw_fp32_bw_param_grads_cl, pulp_conv_dw_fp16_bw_param_grads_cl, pulp_conv_dw_fp32_bw_input_grads_cl, pulp_conv_dw_fp16_bw_input_grads_cl,
    pulp_linear_fp32_fw_cl, pulp_linear_fp16_fw_cl, pulp_linear_fp32_bw_cl, pulp_linear_fp16_bw_cl,
    pulp_linear_fp32_bw_param_grads_cl, pulp_linear_fp16_bw_param_grads_cl, pulp_linear_fp32_bw_input_grads_cl, pulp_linear_fp16_bw_input_grads_cl,
    pulp_mhsa_fp32_fw_cl, pulp_mhsa_fp16_fw_cl, pulp_mhsa_fp32_bw_cl, pulp_mhsa_fp16_bw_cl,
    pulp_mhsa_mobilebert_inference_fp32_fw_cl, pulp_mhsa_mobilebert_inference_fp16_fw_cl,
    pulp_mhsa_mobilebert_inference_fp32_bw_cl, pulp_mhsa_mobilebert_inference_fp16_bw_cl,
    pulp_relu_fp32_fw_cl, pulp_relu_fp16_fw_cl, pulp_relu_fp32_bw_cl, pulp_relu_fp16_bw_cl, relu_core_fw_fp32, relu_core_fw_fp16, relu_core_bw_fp32, relu_core_bw_fp16,
    pulp_sigmoid_fp32_fw_cl, pulp_sigmoid_fp16_fw_cl, pulp_sigmoid_fp32_bw_cl, pulp_sigmoid_fp16_bw_cl, sigmoid_core_fw_fp32, sigmoid_core_bw_fp32,
    pulp_gelu_tanh_approx_fp32_fw_cl, pulp_gelu_fp16_fw_cl,
    pulp_leakyrelu_fp32_fw_cl, pulp_leakyrelu_fp32_bw_cl, leakyrelu_core_fw_fp32, leakyrelu_core_bw_fp32, pulp_leakyrelu_fp16_fw_cl, pulp_leakyrelu_fp16_bw_cl,
    pulp_softmax_fp32_fw_cl, pulp_softmax_fp16_fw_cl, pulp_softmax_fp32_bw_cl, pulp_softmax_fp16_bw_cl,
    pulp_instnorm_fp32_fw_cl, pulp_instnorm_fp16_fw_cl, pulp_instnorm_fp32_bw_cl, pulp_instnorm_fp16_bw_cl,
    pulp_instnorm_fp32_bw_param_grads_cl, pulp_instnorm_fp16_bw_param_grads_cl, pulp_instnorm_fp32_bw_input_grads_cl, pulp_instnorm_fp16_bw_input_grads_cl,
    pulp_instnorm_parallelized_fp32_fw_cl, pulp_instnorm_parallelized_fp32_bw_input_grads_cl, pulp_instnorm_parallelized_fp32_bw_param_grads_cl,
    pulp_batch_norm_fp32_fw_cl, pulp_batch_norm_parallelized_fp32_fw_cl, pulp_layerNorm_fp32_fw_cl,
    pulp_MSELoss, pulp_MSELoss_fp16, pulp_MSELoss_backward, pulp_MSELoss_backward_fp16,
    pulp_CrossEntropyLoss, pulp_CrossEntropyLoss_fp16, pulp_CrossEntropyLoss_backward, pulp_CrossEntropyLoss_backward_fp16,
    pulp_gradient_descent_fp32, pulp_gradient_descent_fp16,
    pulp_residualconn_fp32_fw, pulp_residualconn_fp16_fw, pulp_sumnode_fp32_bw, pulp_sumnode_fp16_bw, pulp_residualconn_fp32_bw, pulp_residualconn_fp16_bw,
    pulp_avgpool_fp32_fw_cl, pulp_avgpool_fp16_fw_cl, pulp_avgpool_fp32_bw_cl, pulp_avgpool_fp16_bw_cl,
    transpose_matrix, transpose_matrix_fp16, transpose, transpose_fp16, copy, copy_fp16, set_to_value, set_to_value_fp16,
    vect_sum, vect_sum_fp16, array_broadcast_sum_fp32, array_broadcast_sum_fp16, pad_tensor, pad_tensor_fp16,
    pulp_scalar_mul_fp32_cl, pulp_scalar_mul_fp16_cl, mm_bias_add_transposed, mm_bias_add_transposed_fp16, HWC_to_CHW, CHW_to_HWC,
    pulp_row_max_fp32_cl, pulp_exp_sum_fp32_cl, pulp_row_div_fp32_cl, pulp_mean_std_fp32_cl, cast_fp16_tensor_to_fp32, cast_fp32_tensor_to_fp16,
};
extern "C" bool tl_is_library_worker(void (*fn)(void *))
{
    for (size_t i = 0; i < sizeof(g_workers) / sizeof(g_workers[0]); i++)
        if (g_workers[i] == fn) return true;
    return false;
}
