/*
 * resnet8_streams.c - see resnet8_streams.h.  User-level code of the PULP-TrainLib API only.
 */
#include "pulp_train.h"
#include "resnet8_streams.h"

#ifndef NUM_CORES
#define NUM_CORES 1
#endif

/* ------------------------------------------------------------------ per-stream iteration
 * With libtrainlib_b200 one call handles all streams (trainlib_set_streams).  With the reference
 * library each call is repeated per stream on blobs shifted to that stream, and weight gradients
 * are added up in stream order. */
static int g_n = 1;
#ifdef NET_REFERENCE
static float *g_acc;                                   /* scratch for one stream's weight gradient */
static size_t g_acc_floats;
static struct blob shift(const struct blob *b, int s, int shift_data)
{
    struct blob r = *b;
    if (shift_data) { if (r.data) r.data += (size_t)s * b->dim; if (r.diff) r.diff += (size_t)s * b->dim; }
    return r;
}
static void accumulate(float *dst, const float *src, int n, int first) { for (int i = 0; i < n; i++) dst[i] = first ? src[i] : dst[i] + src[i]; }
#endif

static void conv_fw(struct Conv2D_args *a)
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) { struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1); struct Conv2D_args t = *a; t.input = &in; t.output = &out; pulp_conv2d_fp32_fw_cl(&t); }
#else
    pulp_conv2d_fp32_fw_cl(a);
#endif
}
static void conv_wg(struct Conv2D_args *a)
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) {
        struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1), w = *a->coeff; struct Conv2D_args t = *a;
        w.diff = g_acc; t.input = &in; t.output = &out; t.coeff = &w;
        pulp_conv2d_fp32_bw_param_grads_cl(&t);
        accumulate(a->coeff->diff, g_acc, a->coeff->dim, s == 0);
    }
#else
    pulp_conv2d_fp32_bw_param_grads_cl(a);
#endif
}
static void conv_ig(struct Conv2D_args *a)
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) { struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1); struct Conv2D_args t = *a; t.input = &in; t.output = &out; pulp_conv2d_fp32_bw_input_grads_cl(&t); }
#else
    pulp_conv2d_fp32_bw_input_grads_cl(a);
#endif
}
static void norm_fw(struct InstNorm_args *a)
{
#ifdef NET_REFERENCE
    const int C = a->input->C;
    for (int s = 0; s < g_n; s++) {
        struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1); struct InstNorm_args t = *a;
        t.input = &in; t.output = &out; t.running_mean += (size_t)s * C; t.running_var += (size_t)s * C; t.running_stdev += (size_t)s * C;
        pulp_instnorm_fp32_fw_cl(&t);
    }
#else
    pulp_instnorm_fp32_fw_cl(a);
#endif
}
static void norm_bw(struct InstNorm_args *a)
{
#ifdef NET_REFERENCE
    const int C = a->input->C;
    for (int s = 0; s < g_n; s++) {
        struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1), co = *a->coeff; struct InstNorm_args t = *a;
        co.diff = g_acc;
        t.input = &in; t.output = &out; t.coeff = &co; t.running_mean += (size_t)s * C; t.running_var += (size_t)s * C; t.running_stdev += (size_t)s * C;
        pulp_instnorm_fp32_bw_cl(&t);
        accumulate(a->coeff->diff, g_acc, 2 * C, s == 0);
    }
#else
    pulp_instnorm_fp32_bw_cl(a);
#endif
}
#ifndef NET_REFERENCE
/* The library can run a norm, the residual sum behind it and the ReLU in one pass over the activation (same values as the
   three calls); resnet8_set_fusion(0) goes back to the separate calls. */
static int g_fuse = 1;
void resnet8_set_fusion(int on) { g_fuse = on != 0; }
static void norm_act_fw(struct InstNorm_args *a, struct blob *skip, int relu)
{
    struct trainlib_instnorm_act_args f; f.norm = a; f.skip = skip; f.relu = relu; f.diff2 = NULL;
    trainlib_instnorm_act_fp32_fw_cl(&f);
}
static void norm_relu_bw(struct InstNorm_args *a, float *diff2)
{
    struct trainlib_instnorm_act_args f; f.norm = a; f.skip = NULL; f.relu = 1; f.diff2 = diff2;
    trainlib_instnorm_act_fp32_bw_cl(&f);
}
static void conv_ig_add(struct Conv2D_args *a) { trainlib_conv2d_fp32_bw_input_grads_acc_cl(a); }
#else
enum { g_fuse = 0 };
void resnet8_set_fusion(int on) { (void)on; }
static void norm_act_fw(struct InstNorm_args *a, struct blob *skip, int relu) { (void)a; (void)skip; (void)relu; }
static void norm_relu_bw(struct InstNorm_args *a, float *diff2) { (void)a; (void)diff2; }
static void conv_ig_add(struct Conv2D_args *a) { (void)a; }
#endif
static void relu_fw(struct act_args *a)
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) { struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1); struct act_args t = *a; t.input = &in; t.output = &out; pulp_relu_fp32_fw_cl(&t); }
#else
    pulp_relu_fp32_fw_cl(a);
#endif
}
static void relu_bw(struct act_args *a)
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) { struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1); struct act_args t = *a; t.input = &in; t.output = &out; pulp_relu_fp32_bw_cl(&t); }
#else
    pulp_relu_fp32_bw_cl(a);
#endif
}
static void skip_call(struct SkipConn_args *a, void (*fn)(void *))
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) {
        struct blob sk = shift(a->skip, s, 1), lo = shift(a->lout, s, 1), out = shift(a->output, s, 1); struct SkipConn_args t = *a;
        t.skip = &sk; t.lout = &lo; t.output = &out; fn(&t);
    }
#else
    fn(a);
#endif
}
static void pool_call(struct pool_args *a, void (*fn)(void *))
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) { struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1); struct pool_args t = *a; t.input = &in; t.output = &out; pi_cl_team_fork(NUM_CORES, fn, &t); }
#else
    pi_cl_team_fork(NUM_CORES, fn, a);
#endif
}
static void linear_fw(struct Linear_args *a)
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) {
        struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1); struct Linear_args t = *a; t.input = &in; t.output = &out;
        pulp_linear_fp32_fw_cl(&t);
        for (int o = 0; o < out.dim; o++) out.data[o] += a->bias->data[o];        /* the fp32 reference forward never adds the bias */
    }
#else
    pulp_linear_fp32_fw_cl(a);
#endif
}
static void linear_bw(struct Linear_args *a)
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) {
        struct blob in = shift(a->input, s, 1), out = shift(a->output, s, 1), w = *a->coeff, b = *a->bias; struct Linear_args t = *a;
        w.diff = g_acc; b.diff = g_acc + a->coeff->dim;
        t.input = &in; t.output = &out; t.coeff = &w; t.bias = &b;
        pulp_linear_fp32_bw_cl(&t);
        accumulate(a->coeff->diff, g_acc, a->coeff->dim, s == 0);
        accumulate(a->bias->diff, g_acc + a->coeff->dim, a->bias->dim, s == 0);
    }
#else
    pulp_linear_fp32_bw_cl(a);
#endif
}
static void loss_call(struct loss_args *a, void (*fn)(void *))
{
#ifdef NET_REFERENCE
    for (int s = 0; s < g_n; s++) { struct blob out = shift(a->output, s, 1); struct loss_args t = *a; t.output = &out; t.target += (size_t)s * out.dim; t.wr_loss += s; fn(&t); }
#else
    fn(a);
#endif
}

/* ------------------------------------------------------------------ the network */
enum { N_CONV = 9, N_NORM = 7, N_ACT = 7 };
enum { C0, C1, C2, C3, C4, P2, C5, C6, P3 };           /* conv indices */

typedef struct { int cin, hin, cout, k, stride, pad; } conv_spec;
static const conv_spec SPEC[N_CONV] = {
    {3, 32, 16, 3, 1, 1},    /* C0 stem */
    {16, 32, 16, 3, 1, 1},   /* C1 */
    {16, 32, 16, 3, 1, 1},   /* C2 */
    {16, 32, 32, 3, 2, 1},   /* C3 downsample */
    {32, 16, 32, 3, 1, 1},   /* C4 */
    {16, 32, 32, 1, 2, 0},   /* P2 projection shortcut */
    {32, 16, 64, 3, 2, 1},   /* C5 downsample */
    {64, 8, 64, 3, 1, 1},    /* C6 */
    {32, 16, 64, 1, 2, 0},   /* P3 projection shortcut */
};
static int conv_hout(const conv_spec *c) { return (c->hin - c->k + 2 * c->pad) / c->stride + 1; }
static const int NORM_OF_CONV[N_NORM] = {C0, C1, C2, C3, C4, C5, C6};

static struct blob b_x, b_conv[N_CONV], b_norm[N_NORM], b_sum[3], b_tmp[2], b_gap, b_z;
static struct blob w_conv[N_CONV], w_norm[N_NORM], w_fc, w_fcb, b_nobias;
static struct Conv2D_args a_conv[N_CONV];
static struct InstNorm_args a_norm[N_NORM];
static struct act_args a_relu_n[N_NORM], a_relu_s[3];
static struct SkipConn_args a_res[3], a_skipgrad[3];
static struct pool_args a_pool;
static struct Linear_args a_fc;
static struct loss_args a_loss;
static float dummy1[1];
static size_t p_off[2 * N_CONV + 8], p_cnt[2 * N_CONV + 8];
static int p_n;
static float *g_params, *g_grads;
static float *g_img, *g_lab, *g_loss;                  /* resident copies used by resnet8_forward_host */
static float *g_img2, *g_lab2;                         /* second copy: uploads alternate between the two */
static int g_host_slot = -1;                           /* copy read by the step in flight (-1: caller-owned device batch) */

static size_t conv_w_count(int i) { return (size_t)SPEC[i].cout * SPEC[i].cin * SPEC[i].k * SPEC[i].k; }

static void layout_params(void)
{
    size_t off = 0; p_n = 0;
    for (int i = 0; i < N_CONV; i++) {
        p_off[p_n] = off; p_cnt[p_n] = conv_w_count(i); off += p_cnt[p_n++];
        for (int j = 0; j < N_NORM; j++) if (NORM_OF_CONV[j] == i) { p_off[p_n] = off; p_cnt[p_n] = 2 * (size_t)SPEC[i].cout; off += p_cnt[p_n++]; }
    }
    p_off[p_n] = off; p_cnt[p_n] = 64 * RESNET8_CLASSES; off += p_cnt[p_n++];
    p_off[p_n] = off; p_cnt[p_n] = RESNET8_CLASSES; off += p_cnt[p_n++];
}
size_t resnet8_param_count(void) { layout_params(); return p_off[p_n - 1] + p_cnt[p_n - 1]; }
int resnet8_param_blobs(void) { layout_params(); return p_n; }
size_t resnet8_param_offset(int i, size_t *count) { layout_params(); if (count) *count = p_cnt[i]; return p_off[i]; }

double resnet8_flops_per_stream(void)
{
    double f = 0;
    for (int i = 0; i < N_CONV; i++) {
        double ho = conv_hout(&SPEC[i]);
        double one = 2.0 * SPEC[i].cout * SPEC[i].cin * SPEC[i].k * SPEC[i].k * ho * ho;
        f += (i == C0) ? 2 * one : 3 * one;              /* the stem has no input gradient */
    }
    return f + 3 * 2.0 * 64 * RESNET8_CLASSES;
}

/* activation floats per stream, in allocation order */
static size_t act_floats(int i) { int ho = conv_hout(&SPEC[i]); return (size_t)SPEC[i].cout * ho * ho; }
size_t resnet8_workspace_floats(int n)
{
    size_t per = 0;
    for (int i = 0; i < N_CONV; i++) per += 2 * act_floats(i);                 /* conv outputs: data + diff */
    for (int j = 0; j < N_NORM; j++) per += 2 * act_floats(NORM_OF_CONV[j]) + 3 * (size_t)SPEC[NORM_OF_CONV[j]].cout;   /* norm outputs + statistics */
    per += 2 * (act_floats(C2) + act_floats(C4) + act_floats(C6));             /* residual sums */
    per += act_floats(C2) + act_floats(C4);                                     /* shortcut input-gradient temporaries */
    per += 2 * 64 + 2 * RESNET8_CLASSES;                                        /* pooled features, logits */
    per += 2 * (RESNET8_IMAGE_FLOATS + RESNET8_CLASSES) + 1;                    /* two resident copies of a host batch (images, labels), losses */
    return per * (size_t)n + 64;
}

static unsigned lcg(unsigned *s) { *s = *s * 1664525u + 1013904223u; return *s; }
static float gauss(unsigned *s)
{
    float u1 = ((lcg(s) >> 8) + 1) * (1.0f / 16777217.0f), u2 = (lcg(s) >> 8) * (1.0f / 16777216.0f);
    return sqrtf(-2.0f * logf(u1)) * cosf(6.28318530718f * u2);
}
void resnet8_init_params(float *p, unsigned seed)
{
    layout_params();
    unsigned s = seed * 2654435761u + 12345u;
    int idx = 0;
    for (int i = 0; i < N_CONV; i++) {
        float sd = sqrtf(2.0f / (SPEC[i].cin * SPEC[i].k * SPEC[i].k));
        for (size_t e = 0; e < p_cnt[idx]; e++) p[p_off[idx] + e] = sd * gauss(&s);
        idx++;
        for (int j = 0; j < N_NORM; j++) if (NORM_OF_CONV[j] == i) {
            for (int c = 0; c < SPEC[i].cout; c++) { p[p_off[idx] + c] = 1.0f; p[p_off[idx] + SPEC[i].cout + c] = 0.0f; }
            idx++;
        }
    }
    for (size_t e = 0; e < p_cnt[idx]; e++) p[p_off[idx] + e] = sqrtf(1.0f / 64) * gauss(&s);
    idx++;
    for (size_t e = 0; e < p_cnt[idx]; e++) p[p_off[idx] + e] = 0.0f;
}

static float *take(float **ws, size_t count) { float *r = *ws; *ws += count; return r; }
static void mkblob(struct blob *b, float *data, float *diff, int C, int H, int W) { b->data = data; b->diff = diff; b->C = C; b->H = H; b->W = W; b->dim = C * H * W; }

int resnet8_bind(int n, float *params, float *grads, float *ws)
{
    if (n < 1 || !params || !grads || !ws) return 1;
    layout_params();
    g_n = n; g_params = params; g_grads = grads;
#ifndef NET_REFERENCE
    trainlib_set_streams(n);
#else
    g_acc_floats = 64 * 64 * 9 + 64;
    g_acc = (float *)malloc(sizeof(float) * g_acc_floats);
#endif
    const size_t N = (size_t)n;
    mkblob(&b_x, NULL, NULL, 3, 32, 32);
    mkblob(&b_nobias, dummy1, dummy1, 1, 1, 1);
    int idx = 0;
    /* parameters */
    for (int i = 0; i < N_CONV; i++) {
        mkblob(&w_conv[i], params + p_off[idx], grads + p_off[idx], SPEC[i].cin, SPEC[i].k, SPEC[i].k); w_conv[i].dim = (int)p_cnt[idx]; idx++;
        for (int j = 0; j < N_NORM; j++) if (NORM_OF_CONV[j] == i) { mkblob(&w_norm[j], params + p_off[idx], grads + p_off[idx], 2 * SPEC[i].cout, 1, 1); idx++; }
    }
    mkblob(&w_fc, params + p_off[idx], grads + p_off[idx], 1, RESNET8_CLASSES, 64); idx++;
    mkblob(&w_fcb, params + p_off[idx], grads + p_off[idx], 1, 1, RESNET8_CLASSES);
    /* activations: conv outputs */
    for (int i = 0; i < N_CONV; i++) { int ho = conv_hout(&SPEC[i]); float *d = take(&ws, N * act_floats(i)), *g = take(&ws, N * act_floats(i)); mkblob(&b_conv[i], d, g, SPEC[i].cout, ho, ho); }
    /* residual sums (ReLU applied in place) */
    const int sum_of[3] = {C2, C4, C6};
    for (int r = 0; r < 3; r++) { int i = sum_of[r], ho = conv_hout(&SPEC[i]); float *d = take(&ws, N * act_floats(i)), *g = take(&ws, N * act_floats(i)); mkblob(&b_sum[r], d, g, SPEC[i].cout, ho, ho); }
    /* norm outputs (ReLU in place).  The norm that feeds a residual sum shares its gradient with the sum. */
    for (int j = 0; j < N_NORM; j++) {
        int i = NORM_OF_CONV[j], ho = conv_hout(&SPEC[i]);
        float *d = take(&ws, N * act_floats(i)), *g = take(&ws, N * act_floats(i));
        if (i == C2) g = b_sum[0].diff; else if (i == C4) g = b_sum[1].diff; else if (i == C6) g = b_sum[2].diff;
        mkblob(&b_norm[j], d, g, SPEC[i].cout, ho, ho);
        a_norm[j].input = &b_conv[i]; a_norm[j].output = &b_norm[j]; a_norm[j].coeff = &w_norm[j];
        a_norm[j].running_mean = take(&ws, N * SPEC[i].cout); a_norm[j].running_var = take(&ws, N * SPEC[i].cout); a_norm[j].running_stdev = take(&ws, N * SPEC[i].cout);
        a_norm[j].freeze_running_params = 0; a_norm[j].skip_wg_grad = 0; a_norm[j].skip_in_grad = 0;
        a_relu_n[j].input = &b_norm[j]; a_relu_n[j].output = &b_norm[j]; a_relu_n[j].H = 1; a_relu_n[j].W = b_norm[j].dim;
    }
    /* projection shortcuts share their output gradient with the sum they feed */
    b_conv[P2].diff = b_sum[1].diff; b_conv[P3].diff = b_sum[2].diff;
    mkblob(&b_tmp[0], NULL, take(&ws, N * act_floats(C2)), 16, 32, 32);      /* dX of P2 before it is added to sum 1 */
    mkblob(&b_tmp[1], NULL, take(&ws, N * act_floats(C4)), 32, 16, 16);      /* dX of P3 before it is added to sum 2 */
    { float *d = take(&ws, N * 64), *g = take(&ws, N * 64); mkblob(&b_gap, d, g, 64, 1, 1); }
    { float *d = take(&ws, N * RESNET8_CLASSES), *g = take(&ws, N * RESNET8_CLASSES); mkblob(&b_z, d, g, 1, 1, RESNET8_CLASSES); }
    g_img = take(&ws, N * RESNET8_IMAGE_FLOATS); g_lab = take(&ws, N * RESNET8_CLASSES); g_loss = take(&ws, N);
    g_img2 = take(&ws, N * RESNET8_IMAGE_FLOATS); g_lab2 = take(&ws, N * RESNET8_CLASSES);

    /* conv wiring: input blob of every conv */
    struct blob *conv_in[N_CONV] = {&b_x, &b_norm[0], &b_norm[1], &b_sum[0], &b_norm[3], &b_sum[0], &b_sum[1], &b_norm[5], &b_sum[1]};
    for (int i = 0; i < N_CONV; i++) {
        struct Conv2D_args *a = &a_conv[i];
        a->input = conv_in[i]; a->coeff = &w_conv[i]; a->bias = &b_nobias; a->output = &b_conv[i];
        a->Lpad = a->Rpad = a->Upad = a->Dpad = SPEC[i].pad; a->stride_h = a->stride_w = SPEC[i].stride;
        a->i2c_buffer = dummy1; a->bt_buffer = dummy1; a->skip_wg_grad = 0; a->skip_in_grad = (i == C0); a->HWC = 0;
        a->opt_matmul_type_fw = a->opt_matmul_type_wg = a->opt_matmul_type_ig = 0;
        a->USE_BIASES = 0; a->USE_IM2COL = 0; a->USE_DMA_IM2COL = 0;
    }
    /* residual sums: stage 1 adds the stage input, stages 2/3 add the projection */
    struct blob *skip_of[3] = {&b_norm[0], &b_conv[P2], &b_conv[P3]};
    struct blob *lout_of[3] = {&b_norm[2], &b_norm[4], &b_norm[6]};
    for (int r = 0; r < 3; r++) {
        a_res[r].skip = skip_of[r]; a_res[r].lout = lout_of[r]; a_res[r].output = &b_sum[r]; a_res[r].skip_in_grad = 0;
        a_relu_s[r].input = &b_sum[r]; a_relu_s[r].output = &b_sum[r]; a_relu_s[r].H = 1; a_relu_s[r].W = b_sum[r].dim;
    }
    /* gradient joins: norm0.diff += sum1.diff ; sum1.diff += dX(P2) ; sum2.diff += dX(P3) */
    a_skipgrad[0].skip = &b_norm[0]; a_skipgrad[0].lout = &b_norm[0]; a_skipgrad[0].output = &b_sum[0]; a_skipgrad[0].skip_in_grad = 0;
    a_skipgrad[1].skip = &b_sum[0]; a_skipgrad[1].lout = &b_sum[0]; a_skipgrad[1].output = &b_tmp[0]; a_skipgrad[1].skip_in_grad = 0;
    a_skipgrad[2].skip = &b_sum[1]; a_skipgrad[2].lout = &b_sum[1]; a_skipgrad[2].output = &b_tmp[1]; a_skipgrad[2].skip_in_grad = 0;

    a_pool.input = &b_sum[2]; a_pool.output = &b_gap; a_pool.Hker = 8; a_pool.Wker = 8; a_pool.Hstride = 1; a_pool.Wstride = 1;
    a_fc.input = &b_gap; a_fc.coeff = &w_fc; a_fc.bias = &w_fcb; a_fc.output = &b_z; a_fc.skip_wg_grad = 0; a_fc.skip_in_grad = 0;
    a_fc.opt_matmul_type_fw = a_fc.opt_matmul_type_wg = a_fc.opt_matmul_type_ig = 0; a_fc.use_biases = 1;
    a_loss.output = &b_z;
    return 0;
}

float *resnet8_logits(void) { return b_z.data; }

static void stage(int conv_a, int norm_a, int conv_b, int norm_b, int proj, int r)
{
    if (g_fuse) {
        conv_fw(&a_conv[conv_a]); norm_act_fw(&a_norm[norm_a], NULL, 1);
        if (proj >= 0) conv_fw(&a_conv[proj]);
        conv_fw(&a_conv[conv_b]);
        /* the sum goes where the separate calls leave it: the norm writes relu(norm + skip) straight into the sum's blob */
        struct InstNorm_args t = a_norm[norm_b]; t.output = a_res[r].output;
        norm_act_fw(&t, a_res[r].skip, 1);
        return;
    }
    conv_fw(&a_conv[conv_a]); norm_fw(&a_norm[norm_a]); relu_fw(&a_relu_n[norm_a]);
    conv_fw(&a_conv[conv_b]); norm_fw(&a_norm[norm_b]);
    if (proj >= 0) conv_fw(&a_conv[proj]);
    skip_call(&a_res[r], pulp_residualconn_fp32_fw);
    relu_fw(&a_relu_s[r]);
}

void resnet8_forward(const float *images, const float *labels, float *loss)
{
    b_x.data = (float *)images;
    conv_fw(&a_conv[C0]);
    if (g_fuse) norm_act_fw(&a_norm[0], NULL, 1); else { norm_fw(&a_norm[0]); relu_fw(&a_relu_n[0]); }
    stage(C1, 1, C2, 2, -1, 0);
    stage(C3, 3, C4, 4, P2, 1);
    stage(C5, 5, C6, 6, P3, 2);
    pool_call(&a_pool, pulp_avgpool_fp32_fw_cl);
    linear_fw(&a_fc);
    a_loss.target = (float *)labels; a_loss.wr_loss = loss;
    loss_call(&a_loss, pulp_CrossEntropyLoss);
}

void resnet8_forward_host(const float *host_images, const float *host_labels, float *host_loss)
{
#ifdef NET_REFERENCE
    resnet8_forward(host_images, host_labels, host_loss);
#else
    /* two resident copies of the batch, used in turn: the upload of this step runs beside the backward pass and the
       update of the previous step, which are still queued when this function is entered */
    static int slot = 0;
    float *img = slot ? g_img2 : g_img, *lab = slot ? g_lab2 : g_lab;
    g_host_slot = slot;
    trainlib_memcpy_h2d_overlapped(img, host_images, sizeof(float) * (size_t)g_n * RESNET8_IMAGE_FLOATS, slot);
    trainlib_memcpy_h2d_overlapped(lab, host_labels, sizeof(float) * (size_t)g_n * RESNET8_CLASSES, slot);
    resnet8_forward(img, lab, g_loss);
    trainlib_mark_consumed(slot);                  /* resnet8_backward marks it again: it reads the images and labels too */
    trainlib_memcpy_d2h(host_loss, g_loss, sizeof(float) * (size_t)g_n);
    slot ^= 1;
#endif
}

static void conv_bw(int i) { conv_wg(&a_conv[i]); if (!a_conv[i].skip_in_grad) conv_ig(&a_conv[i]); }

static void stage_bw(int conv_a, int norm_a, int conv_b, int norm_b, int proj, int r)
{
    relu_bw(&a_relu_s[r]);                         /* sum.diff masked in place; norm_b and the shortcut share it */
    norm_bw(&a_norm[norm_b]); conv_bw(conv_b);
    if (g_fuse) norm_relu_bw(&a_norm[norm_a], NULL); else { relu_bw(&a_relu_n[norm_a]); norm_bw(&a_norm[norm_a]); }
    conv_bw(conv_a);                               /* writes the stage input's gradient */
    if (proj >= 0 && g_fuse) {
        conv_wg(&a_conv[proj]);
        conv_ig_add(&a_conv[proj]);                /* the shortcut's dX is added to the stage input's gradient in place */
    } else if (proj >= 0) {
        struct blob *in = a_conv[proj].input; float *keep = in->diff;
        conv_wg(&a_conv[proj]);
        in->diff = b_tmp[r - 1].diff;              /* shortcut dX goes to a temporary ... */
        conv_ig(&a_conv[proj]);
        in->diff = keep;
        skip_call(&a_skipgrad[r], pulp_sumnode_fp32_bw);   /* ... and is added to the stage input's gradient */
    } else if (!g_fuse) {                          /* fused: the stem's norm backward reads both gradients itself */
        skip_call(&a_skipgrad[0], pulp_sumnode_fp32_bw);   /* identity shortcut: norm0.diff += sum1.diff */
    }
}

void resnet8_backward(void)
{
#ifndef NET_REFERENCE
    /* the two dozen fixed-order sums of partial gradients run as one launch at the end of the pass (same values) */
    if (g_fuse) trainlib_set_deferred_reductions(1);
#endif
    loss_call(&a_loss, pulp_CrossEntropyLoss_backward);
    linear_bw(&a_fc);
    pool_call(&a_pool, pulp_avgpool_fp32_bw_cl);
    stage_bw(C5, 5, C6, 6, P3, 2);
    stage_bw(C3, 3, C4, 4, P2, 1);
    stage_bw(C1, 1, C2, 2, -1, 0);
    if (g_fuse) norm_relu_bw(&a_norm[0], b_sum[0].diff); else { relu_bw(&a_relu_n[0]); norm_bw(&a_norm[0]); }
    conv_bw(C0);
#ifndef NET_REFERENCE
    if (g_fuse) trainlib_set_deferred_reductions(0);   /* runs the pending sums: the gradient buffer is complete on return */
    if (g_host_slot >= 0) { trainlib_mark_consumed(g_host_slot); g_host_slot = -1; }   /* last reader of that batch copy */
#endif
}

void resnet8_update(float lr)
{
    struct optim_args o;
    struct blob flat;
    /* all parameters are one flat tensor, so one SGD call updates the whole network */
    flat.data = g_params; flat.diff = g_grads; flat.dim = (int)resnet8_param_count(); flat.C = 1; flat.H = 1; flat.W = flat.dim;
    o.weights = &flat; o.biases = &flat; o.learning_rate = lr; o.weight_decay_lambda = 0; o.use_biases = 0;
    pi_cl_team_fork(NUM_CORES, pulp_gradient_descent_fp32, &o);
}
