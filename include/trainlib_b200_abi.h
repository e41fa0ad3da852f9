/*
 * trainlib_b200_abi.h - the C ABI that libtrainlib_b200.so exports for the
 * matmul-centred training step of PULP-TrainLib.
 *
 * Every struct below is layout-identical (field order, types, names) to the struct
 * of the same name in the reference library, so that C code written against the
 * reference headers links against this library unchanged.  Every function has the
 * reference's `void f(void *args)` shape.  The reference declaration each item
 * replaces is cited as  [ref: <file under lib/include or lib/sources>:<line>].
 *
 * Semantics that differ from the reference on purpose (the reference computes a
 * wrong or undefined result there) are marked "DEVIATION".
 *
 * Tensors are row-major; activations are CHW unless a struct carries HWC = 1.
 * Pointers may be host or device addresses, see trainlib_b200.h (memory modes).
 */
#ifndef TRAINLIB_B200_ABI_H
#define TRAINLIB_B200_ABI_H

#include "pmsis.h"   /* pi_cl_dma_cmd_t of the tiled-attention arguments, as pulp_mhsa_fp32.h includes it */

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ scalar types */
/* [ref: pulp_train_defines.h:32-33] `fp16` is float16alt on PULP.  Here it is IEEE
 * binary16 storage; all fp16 kernels accumulate in fp32 on the GPU. */
#ifndef TRAINLIB_FP16_TYPE
#define TRAINLIB_FP16_TYPE _Float16
#endif
#ifndef TRAINLIB_NO_FP16_TYPEDEF
typedef TRAINLIB_FP16_TYPE fp16;
#endif

/* [ref: pulp_train_defines.h:51-65] selectors carried by mm_manager_args */
#define LAYER_CONV2D   0
#define LAYER_DW_CONV  1
#define LAYER_PW_CONV  2
#define LAYER_LINEAR   3
#define STEP_FW        0
#define STEP_WGT_GRAD  1
#define STEP_IN_GRAD   2

/* [ref: pulp_train_defines.h:85-93] Schraudolph-exp constants used by softmax */
#define GIST_A  12102203.17133801f
#define GIST_B  1064986823.010288f
#define GIST_C  8388608
#define GIST_D  2139095040
/* [ref: pulp_train_defines.h:104] variance floor of the instance norm */
#define EPSILON 1e-10

#ifndef ABS
#define ABS(x) ((x) > 0 ? (x) : (-(x)))
#endif

/* ================================================================== fp32 structs */

/* [ref: pulp_train_utils_fp32.h:37-44] tensor handle: values, gradient, flat size, W/H/C */
struct blob { float *data; float *diff; int dim; int W; int H; int C; };

/* [ref: pulp_train_utils_fp32.h:63-77] */
struct im2col_args {
    struct blob *input; struct blob *c; struct blob *output; float *pBuffer;
    int Lpad; int Rpad; int Upad; int Dpad; int mod; int stride_w; int stride_h; int HWC; int USE_DMA;
};
/* [ref: pulp_train_utils_fp32.h:92-100] 2-D (N,M) or n_dim-D transpose */
struct transp_args { float *in_matrix; float *out_matrix; int N; int M; int *dim; int *transposed_axes; int n_dim; };
/* [ref: pulp_train_utils_fp32.h:110-115] */
struct layout_args { struct blob *tensor; float *transp_buffer; int transpose_data; int transpose_grad; };
/* [ref: pulp_train_utils_fp32.h:127-135] */
struct blocktransp_args { float *weights; float *bt_weights; int Cin; int Cout; int Hk; int Wk; int HWC; };
/* [ref: pulp_train_utils_fp32.h:144-148] */
struct copy_args { float *from; float *to; int size; };
/* [ref: pulp_train_utils_fp32.h:157-161] */
struct set_to_value_args { float *to; float value; int size; };
/* [ref: pulp_train_utils_fp32.h:171-176] */
struct vect_sum_args { float *op_1; float *op_2; float *dest; int size; };
/* [ref: pulp_train_utils_fp32.h:190-198] */
struct array_broadcast_sum_fp32_args {
    float *op_1; float *op_2; float *dest; int *op_1_dims; int *op_2_dims; int op_1_dims_len; int op_2_dims_len;
};
/* [ref: pulp_train_utils_fp32.h:207-211] */
struct cast_16t32_args { fp16 *source; float *destination; int size; };
/* [ref: pulp_train_utils_fp32.h:227-238] */
struct pad_args { float *source; float *dest; int C; int H; int W; int T_RPAD; int T_LPAD; int T_UPAD; int T_DPAD; int HWC_lay; };
/* [ref: pulp_train_utils_fp32.h:268-297] GEMM descriptor: C[N x M] = A[N x K] * B, B is
 * [K x M] (trans_B = 0) or [M x K] (trans_B = 1); the conv fields feed the naive kernels. */
struct matMul_args {
    float *__restrict__ A; float *__restrict__ B; float *__restrict__ C;
    int N; int M; int K; int trans_B;
    int H; int W; int pW; int pH; int pCin; int pCout;
    int stride_h; int stride_w; int Lpad; int Rpad; int Upad; int Dpad;
    float *__restrict__ bias; int bias_dim; int USE_BIASES; int bias_transposed; int HWC;
};
/* [ref: pulp_train_utils_fp32.h:310-318] */
struct broadcastMatMul_args_fp32 {
    float *__restrict__ A; float *__restrict__ B; float *__restrict__ C;
    int *__restrict__ A_dims; int *__restrict__ B_dims; int A_dims_len; int B_dims_len;
};
/* [ref: pulp_train_utils_fp32.h:337-347] */
struct kernel_DW_args {
    struct blob *input; struct blob *weights; struct blob *output;
    int stride_h; int stride_w; int Lpad; int Rpad; int Upad; int Dpad;
};
struct matMul_DW_args;   /* named but never defined by the reference either */
/* [ref: pulp_train_utils_fp32.h:360-366] */
struct mm_manager_args {
    struct matMul_args *mm_args; struct matMul_DW_args *mm_dw_args; int layer_type; int step_type; int matmul_type;
};
/* [ref: pulp_train_utils_fp32.h:375-379] */
struct tanh_args { float *input; int dim; float *output; };
/* [ref: pulp_train_utils_fp32.h:388-392] */
struct update_weight_args { float *accum; float *grad; int dim; };
/* [ref: pulp_train_utils_fp32.h:402-407] */
struct max_args { float *input; int H; int W; float *maxes; };
/* [ref: pulp_train_utils_fp32.h:419-426] */
struct exp_sum_args { float *input; float *output; int H; int W; float *maxes; float *sums; };
/* [ref: pulp_train_utils_fp32.h:438-445] */
struct shift_sum_args { float *input; float *sums; float *output; int dim; int dim2; float *maxes; };
/* [ref: pulp_train_utils_fp32.h:454-458] */
struct div_args { float *input; float n; int dim; };
/* [ref: pulp_train_utils_fp32.h:468-473] */
struct row_div_args { float *input; int H; int W; float *sums; };
/* [ref: pulp_train_utils_fp32.h:482-486] */
struct scalar_mul_args { float *input; float scalar; int dim; };
/* [ref: pulp_train_utils_fp32.h:498-505] */
struct mean_std_args { float *input; float *mean; float *var; float *std; float epsilon; int dim; };
/* [ref: pulp_train_utils_fp32.h:516-522] */
struct vector_exp_sum_args { float *input; float *sums; float *output; int dim; float max; };
/* [ref: pulp_train_utils_fp32.h:533-539] */
struct sm_bw_op_1_args { float *A; float *B; float *S; int H; int W; };
/* [ref: pulp_train_utils_fp32.h:551-558] */
struct sm_bw_op_2_args { float *A; float *B; float *S; float *output; int H; int W; };
/* [ref: pulp_train_utils_fp32.h:569-575] */
struct mm_bias_add_args { float *mat; float *bias; int H; int W; int t; };
/* [ref: pulp_train_utils_fp32.h:586-592] */
struct reduce_mean_args_fp32 { float *input; float *output; int *dims; int dims_len; int reduce_axis; };

/* [ref: pulp_conv2d_fp32.h:50-72] */
struct Conv2D_args {
    struct blob *input; struct blob *coeff; struct blob *bias; struct blob *output;
    int Lpad; int Rpad; int Upad; int Dpad; int stride_h; int stride_w;
    float *i2c_buffer; float *bt_buffer;
    int skip_wg_grad; int skip_in_grad; int HWC;
    int opt_matmul_type_fw; int opt_matmul_type_wg; int opt_matmul_type_ig;
    int USE_BIASES; int USE_IM2COL; int USE_DMA_IM2COL;
};
/* [ref: pulp_linear_fp32.h:39-50] */
struct Linear_args {
    struct blob *input; struct blob *coeff; struct blob *bias; struct blob *output;
    int skip_wg_grad; int skip_in_grad;
    int opt_matmul_type_fw; int opt_matmul_type_wg; int opt_matmul_type_ig; int use_biases;
};
/* [ref: pulp_conv_pw_fp32.h:39-50] */
struct PointWise_Conv_args {
    struct blob *input; struct blob *coeff; struct blob *output; float *transpose_buffer;
    int skip_wg_grad; int skip_in_grad;
    int opt_matmul_type_fw; int opt_matmul_type_wg; int opt_matmul_type_ig; int HWC;
};
/* [ref: pulp_conv_dw_fp32.h:43-60] */
struct DepthWise_Conv_args {
    struct blob *input; struct blob *coeff; struct blob *output;
    int stride_h; int stride_w; int Lpad; int Rpad; int Upad; int Dpad;
    int skip_wg_grad; int skip_in_grad; int HWC;
};
/* [ref: pulp_mhsa_fp32.h:52-83] input/output are E x L (transposed), projection weights
 * E x F, q/k/v/attention_map F x L, softmax_buffer n_heads x L x L. */
struct Mhsa_args {
    struct blob *input; struct blob *input_bn; int n_heads;
    int opt_matmul_type_fw; int opt_matmul_type_wg; int opt_matmul_type_ig;
    struct blob *output;
    struct blob *coeff_in_q; struct blob *coeff_in_k; struct blob *coeff_in_v;
    struct blob *bias_in_q; struct blob *bias_in_k; struct blob *bias_in_v;
    struct blob *coeff_out; struct blob *bias_out;
    struct blob *q; struct blob *k; struct blob *v; struct blob *attention_map;
    float *temp_buffer; float *grad;
    struct blob *head_buffer; struct blob *softmax_buffer;
    float *global_max; float *partial_exp_sum; float *maxes; float *sums;
};
/* [ref: pulp_mhsa_fp32.h:91-122] tile sizes of the L1-tiled attention; the tiles are a memory plan for the cluster's
 * scratchpad and change no result, so this library reads none of them */
struct Tiled_Matmul_Mhsa_args {
    struct matMul_args *mm_args; struct mm_manager_args *man_args; float *BUFF;
    int tile_h; int tile_w; int tile_dim; int tile_h_p; int tile_w_p; int tile_dim_p; int tile_h_sm; int tile_w_sm; int tile_dim_sm;
    int tile_h_tr; int tile_w_tr; int tile_dim_tr; int tile_h_attv; int tile_w_attv; int tile_dim_attv;
    int tile_h_out_tr; int tile_w_out_tr; int tile_dim_out_tr;
    pi_cl_dma_cmd_t *cmd_store; pi_cl_dma_cmd_t *cmd_load;
};
/* [ref: pulp_act_fp32.h:27-32] */
struct act_args { struct blob *input; struct blob *output; int H; int W; };
/* [ref: pulp_act_fp32.h:40-44] */
struct leakyrelu_args { struct blob *input; struct blob *output; float negative_slope; };
/* [ref: pulp_act_fp32.h:53-66] */
struct softmax_args {
    float *input_data; float *input_diff; float *output_data; float *output_diff;
    int H; int W; int L; int n_heads;
    float *global_max; float *partial_exp_sum; float *maxes; float *sums;
};
/* [ref: pulp_instnorm_fp32.h:38-48] coeff->data = [gamma(C), beta(C)] */
struct InstNorm_args {
    struct blob *input; struct blob *output; struct blob *coeff;
    float *running_mean; float *running_var; float *running_stdev;
    int freeze_running_params; int skip_wg_grad; int skip_in_grad;
};
/* [ref: pulp_batchnorm_fp32.h:40-66] */
struct BatchNorm_args_fp32 {
    struct blob *input; struct blob *output; struct blob *coeff; struct blob *bias;
    int batch_size;
    float *running_mean; float *running_var; float *running_stdev;
    int freeze_running_params; int skip_wg_grad; int skip_in_grad;
    float *weight_data; float *bias_data; float *eps;
    int B; int C; int H; int W;
};
/* [ref: pulp_layernorm_fp32.h:26-34] */
struct LayerNorm_args_fp32 { float *x; float *weight; float *bias; float *output; float *eps; int size; int step_size; };
/* [ref: pulp_losses_fp32.h:32-36] */
struct loss_args { struct blob *output; float *target; float *wr_loss; };
/* [ref: pulp_optimizers_fp32.h:34-40] */
struct optim_args { struct blob *weights; struct blob *biases; float learning_rate; float weight_decay_lambda; int use_biases; };
/* [ref: pulp_residual_fp32.h:50-55] */
struct SkipConn_args { struct blob *skip; struct blob *lout; struct blob *output; int skip_in_grad; };
/* [ref: pulp_pooling_fp32.h:34-41] */
struct pool_args { struct blob *input; struct blob *output; int Hker; int Wker; int Hstride; int Wstride; };
/* [ref: pulp_losses_fp32.h:45-50] */
struct berHu_loss_args { struct blob *output; float *target; float *wr_loss; float alpha; };
/* [ref: pulp_nonorm_fp32.h:35-40] */
struct Nonorm_args { struct blob *input; struct blob *coeff; struct blob *bias; struct blob *output; };
/* [ref: pulp_rmsnorm_fp32.h:17-31] */
struct weighted_scaling_args { float *out; float *in; float *w; float scaling_factor; unsigned int size; };
struct sum_of_squares_args { float *out; float *in; unsigned int size; };
/* [ref: pulp_act_fp32.h:76-81] */
struct swiglu_args { float *in1; float *in2; float *out; int dim; };

/* ================================================================== fp16 structs */
/* Field-for-field twins of the above on `fp16` storage. */

/* [ref: pulp_train_utils_fp16.h:38-45] */
struct blob_fp16 { fp16 *data; fp16 *diff; int dim; int W; int H; int C; };
/* [ref: pulp_train_utils_fp16.h:64-78] */
struct im2col_args_fp16 {
    struct blob_fp16 *input; struct blob_fp16 *c; struct blob_fp16 *output; fp16 *pBuffer;
    int Lpad; int Rpad; int Upad; int Dpad; int mod; int stride_w; int stride_h; int HWC; int USE_DMA;
};
/* [ref: pulp_train_utils_fp16.h:93-101] */
struct transp_args_fp16 { fp16 *in_matrix; fp16 *out_matrix; int N; int M; int *dim; int *transposed_axes; int n_dim; };
/* [ref: pulp_train_utils_fp16.h:115-123] */
struct array_broadcast_sum_fp16_args {
    fp16 *op_1; fp16 *op_2; fp16 *dest; int *op_1_dims; int *op_2_dims; int op_1_dims_len; int op_2_dims_len;
};
/* [ref: pulp_train_utils_fp16.h:252-262] */
struct broadcastMatMul_args_fp16 {
    fp16 *__restrict__ A; fp16 *__restrict__ B; fp16 *__restrict__ C;
    int *__restrict__ A_dims; int *__restrict__ B_dims; int A_dims_len; int B_dims_len;
};
/* [ref: pulp_train_utils_fp16.h:133-138] */
struct layout_args_fp16 { struct blob_fp16 *tensor; fp16 *transp_buffer; int transpose_data; int transpose_grad; };
/* [ref: pulp_train_utils_fp16.h:150-158] */
struct blocktransp_args_fp16 { fp16 *weights; fp16 *bt_weights; int Cin; int Cout; int Hk; int Wk; int HWC; };
/* [ref: pulp_train_utils_fp16.h:167-171] */
struct copy_args_fp16 { fp16 *from; fp16 *to; int size; };
/* [ref: pulp_train_utils_fp16.h:180-184] */
struct set_to_value_args_fp16 { fp16 *to; fp16 value; int size; };
/* [ref: pulp_train_utils_fp16.h:194-199] */
struct vect_sum_args_fp16 { fp16 *op_1; fp16 *op_2; fp16 *dest; int size; };
/* [ref: pulp_train_utils_fp16.h:208-212] */
struct cast_32t16_args { float *source; fp16 *destination; int size; };
/* [ref: pulp_train_utils_fp16.h:228-239] */
struct pad_args_fp16 { fp16 *source; fp16 *dest; int C; int H; int W; int T_RPAD; int T_LPAD; int T_UPAD; int T_DPAD; int HWC_lay; };
/* [ref: pulp_train_utils_fp16.h:292-321] */
struct matMul_args_fp16 {
    fp16 *__restrict__ A; fp16 *__restrict__ B; fp16 *__restrict__ C;
    int N; int M; int K; int trans_B;
    int H; int W; int pW; int pH; int pCin; int pCout;
    int stride_h; int stride_w; int Lpad; int Rpad; int Upad; int Dpad;
    fp16 *__restrict__ bias; int bias_dim; int USE_BIASES; int bias_transposed; int HWC;
};
struct matMul_DW_args_fp16;
/* [ref: pulp_train_utils_fp16.h:345-351] */
struct mm_manager_args_fp16 {
    struct matMul_args_fp16 *mm_args; struct matMul_DW_args_fp16 *mm_dw_args; int layer_type; int step_type; int matmul_type;
};
/* [ref: pulp_train_utils_fp16.h:411-418] */
struct exp_sum_args_fp16 { fp16 *input; fp16 *output; int H; int W; fp16 *maxes; fp16 *sums; };
/* [ref: pulp_train_utils_fp16.h:454-458] */
struct scalar_mul_args_fp16 { fp16 *input; fp16 scalar; int dim; };
/* [ref: pulp_train_utils_fp16.h:524-530] */
struct mm_bias_add_args_fp16 { fp16 *mat; fp16 *bias; int H; int W; int t; };

/* [ref: pulp_conv2d_fp16.h:51-73] */
struct Conv2D_args_fp16 {
    struct blob_fp16 *input; struct blob_fp16 *coeff; struct blob_fp16 *bias; struct blob_fp16 *output;
    int Lpad; int Rpad; int Upad; int Dpad; int stride_h; int stride_w;
    fp16 *i2c_buffer; fp16 *bt_buffer;
    int skip_wg_grad; int skip_in_grad; int HWC;
    int opt_matmul_type_fw; int opt_matmul_type_wg; int opt_matmul_type_ig;
    int USE_BIASES; int USE_IM2COL; int USE_DMA_IM2COL;
};
/* [ref: pulp_linear_fp16.h:39-50] */
struct Linear_args_fp16 {
    struct blob_fp16 *input; struct blob_fp16 *coeff; struct blob_fp16 *bias; struct blob_fp16 *output;
    int skip_wg_grad; int skip_in_grad;
    int opt_matmul_type_fw; int opt_matmul_type_wg; int opt_matmul_type_ig; int use_biases;
};
/* [ref: pulp_conv_pw_fp16.h:40-51] */
struct PointWise_Conv_args_fp16 {
    struct blob_fp16 *input; struct blob_fp16 *coeff; struct blob_fp16 *output; fp16 *transpose_buffer;
    int skip_wg_grad; int skip_in_grad;
    int opt_matmul_type_fw; int opt_matmul_type_wg; int opt_matmul_type_ig; int HWC;
};
/* [ref: pulp_conv_dw_fp16.h:40-51] note: no stride fields, unlike the fp32 twin */
struct DepthWise_Conv_args_fp16 {
    struct blob_fp16 *input; struct blob_fp16 *coeff; struct blob_fp16 *output;
    int Lpad; int Rpad; int Upad; int Dpad;
    int skip_wg_grad; int skip_in_grad; int HWC;
};
/* [ref: pulp_mhsa_fp16.h:56-87] */
struct Mhsa_args_fp16 {
    struct blob_fp16 *input; struct blob_fp16 *input_bn; int n_heads;
    int opt_matmul_type_fw; int opt_matmul_type_wg; int opt_matmul_type_ig;
    struct blob_fp16 *output;
    struct blob_fp16 *coeff_in_q; struct blob_fp16 *coeff_in_k; struct blob_fp16 *coeff_in_v;
    struct blob_fp16 *bias_in_q; struct blob_fp16 *bias_in_k; struct blob_fp16 *bias_in_v;
    struct blob_fp16 *coeff_out; struct blob_fp16 *bias_out;
    struct blob_fp16 *q; struct blob_fp16 *k; struct blob_fp16 *v; struct blob_fp16 *attention_map;
    fp16 *temp_buffer; fp16 *grad;
    struct blob_fp16 *head_buffer; struct blob_fp16 *softmax_buffer;
    fp16 *global_max; fp16 *partial_exp_sum; fp16 *maxes; fp16 *sums;
};
/* [ref: pulp_mhsa_fp16.h:90-114] */
struct Tiled_Matmul_Mhsa_args_fp16 {
    struct matMul_args_fp16 *mm_args; struct mm_manager_args_fp16 *man_args; fp16 *BUFF;
    int tile_h; int tile_w; int tile_dim; int tile_h_p; int tile_w_p; int tile_dim_p; int tile_h_sm; int tile_w_sm; int tile_dim_sm;
    int tile_h_tr; int tile_w_tr; int tile_dim_tr; int tile_h_attv; int tile_w_attv; int tile_dim_attv;
    int tile_h_out_tr; int tile_w_out_tr; int tile_dim_out_tr;
    pi_cl_dma_cmd_t *cmd_store; pi_cl_dma_cmd_t *cmd_load;
};
/* [ref: pulp_act_fp16.h:28-33] */
struct act_args_fp16 { struct blob_fp16 *input; struct blob_fp16 *output; int H; int W; };
/* [ref: pulp_act_fp16.h:41-45] */
struct leakyrelu_args_fp16 { struct blob_fp16 *input; struct blob_fp16 *output; fp16 negative_slope; };
/* [ref: pulp_act_fp16.h:54-67] */
struct softmax_args_fp16 {
    fp16 *input_data; fp16 *input_diff; fp16 *output_data; fp16 *output_diff;
    int H; int W; int L; int n_heads;
    fp16 *global_max; fp16 *partial_exp_sum; fp16 *maxes; fp16 *sums;
};
/* [ref: pulp_instnorm_fp16.h:38-48] */
struct InstNorm_args_fp16 {
    struct blob_fp16 *input; struct blob_fp16 *output; struct blob_fp16 *coeff;
    fp16 *running_mean; fp16 *running_var; fp16 *running_stdev;
    int freeze_running_params; int skip_wg_grad; int skip_in_grad;
};
/* [ref: pulp_losses_fp16.h:33-37] */
struct loss_args_fp16 { struct blob_fp16 *output; fp16 *target; fp16 *wr_loss; };
/* [ref: pulp_optimizers_fp16.h:35-41] */
struct optim_args_fp16 { struct blob_fp16 *weights; struct blob_fp16 *biases; fp16 learning_rate; fp16 weight_decay_lambda; int use_biases; };
/* [ref: pulp_residual_fp16.h:50-55] */
struct SkipConn_args_fp16 { struct blob_fp16 *skip; struct blob_fp16 *lout; struct blob_fp16 *output; int skip_in_grad; };
/* [ref: pulp_pooling_fp16.h:34-41] */
struct pool_args_fp16 { struct blob_fp16 *input; struct blob_fp16 *output; int Hker; int Wker; int Hstride; int Wstride; };
/* [ref: pulp_losses_fp16.h:46-51] */
struct berHu_loss_args_fp16 { struct blob_fp16 *output; fp16 *target; fp16 *wr_loss; fp16 alpha; };
/* [ref: pulp_nonorm_fp16.h:36-41] */
struct Nonorm_args_fp16 { struct blob_fp16 *input; struct blob_fp16 *coeff; struct blob_fp16 *bias; struct blob_fp16 *output; };
/* [ref: pulp_rmsnorm_fp16.h:4-16] */
struct weighted_scaling_args_fp16 { fp16 *out; fp16 *in; fp16 *w; fp16 scaling_factor; unsigned int size; };
struct sum_of_squares_args_fp16 { fp16 *out; fp16 *in; unsigned int size; };
/* [ref: pulp_act_fp16.h:195-200] */
struct swiglu_args_fp16 { fp16 *in1; fp16 *in2; fp16 *out; int dim; };
/* [ref: pulp_train_utils_fp16.h:387-393, 427-432, 441-445, 470-477, 488-513, 786-792] */
struct max_args_fp16 { fp16 *input; int H; int W; fp16 *maxes; int dim; };
struct row_div_args_fp16 { fp16 *input; int H; int W; fp16 *sums; };
struct div_args_fp16 { fp16 *input; fp16 n; int dim; };
struct mean_std_args_fp16 { fp16 *input; fp16 *mean; fp16 *var; fp16 *std; fp16 epsilon; int dim; };
struct sm_bw_op_1_args_fp16 { fp16 *A; fp16 *B; fp16 *S; int H; int W; };
struct sm_bw_op_2_args_fp16 { fp16 *A; fp16 *B; fp16 *S; fp16 *output; int H; int W; };
struct vector_exp_sum_args_fp16 { fp16 *input; fp16 *sums; fp16 *output; int dim; fp16 max; };

/* ================================================================== fp32 entry points */

/* ---- matmul family [ref: pulp_matmul_fp32.h:52-246; sources pulp_matmul_fp32.c:190-3697].
 * All variants compute the same C = A*B (one fp32 accumulator per output, k ascending) and
 * differ only in loop unrolling on PULP; here they are one GPU GEMM.  Argument: struct matMul_args. */
void mm_broadcast_fp32(void *broadcastMatMul_args_fp32);   /* NumPy-style batched product  [ref: pulp_matmul_fp32.c:29] */
void mm(void *matMul_args);
void mm_add(void *matMul_args);          /* C += A*B  [ref: pulp_matmul_fp32.c:267] */
void mm_M(void *matMul_args);
void mm_u2(void *matMul_args);
void mm_unroll_1x2(void *matMul_args);  void mm_unroll_1x4(void *matMul_args);  void mm_unroll_1x8(void *matMul_args);
void mm_unroll_2x1(void *matMul_args);  void mm_unroll_4x1(void *matMul_args);  void mm_unroll_8x1(void *matMul_args);
void mm_unroll_2x2(void *matMul_args);  void mm_unroll_2x4(void *matMul_args);  void mm_unroll_4x2(void *matMul_args);
void mm_unroll_4x4(void *matMul_args);
void mm_M_u2(void *matMul_args);        /* DEVIATION: the reference's trans_B branch is wrong (pulp_matmul_fp32.c:2122) */
void mm_M_unroll_2x1(void *matMul_args); void mm_M_unroll_4x1(void *matMul_args); void mm_M_unroll_8x1(void *matMul_args);
void mm_M_unroll_1x2(void *matMul_args); void mm_M_unroll_1x4(void *matMul_args); void mm_M_unroll_1x8(void *matMul_args);
void mm_M_unroll_2x2(void *matMul_args); void mm_M_unroll_4x2(void *matMul_args); void mm_M_unroll_2x4(void *matMul_args);
void mm_M_unroll_4x4(void *matMul_args);
/* [ref: pulp_train_utils_fp32.h:706, source pulp_train_utils_fp32.c:1330-1683] argument:
 * struct mm_manager_args.  matmul_type is accepted and ignored; an unknown layer_type prints
 * the reference's message and returns; the bias add after the product follows :1671-1682. */
void mm_manager(void *mm_manager_args);

/* ---- im2col helpers [ref: pulp_im2col_fp32.h:30,38,53; sources pulp_im2col_fp32.c:29,668,1020] */
void pulp_im2row_fp32(void *im2col_args);
void pulp_im2col_fp32(void *im2col_args);
void pulp_blocktransp_fp32(void *blocktransp_args);

/* ---- Conv2D [ref: pulp_conv2d_fp32.h:84-120; sources pulp_conv2d_fp32.c:27,225,240,454]
 * One implicit-GEMM kernel serves USE_IM2COL = 0 and 1; i2c_buffer / bt_buffer are never
 * touched.  DEVIATION: with padding, the weight and input gradients are the mathematically
 * correct ones (what the reference's naive kernels compute), not the im2col path's. */
void pulp_conv2d_fp32_fw_cl(void *Conv2D_args);
void pulp_conv2d_fp32_bw_cl(void *Conv2D_args);
void pulp_conv2d_fp32_bw_param_grads_cl(void *Conv2D_args);
void pulp_conv2d_fp32_bw_input_grads_cl(void *Conv2D_args);
/* naive kernels on struct matMul_args [ref: pulp_conv_naive_fp32.h:63-109; pulp_conv_naive_fp32.c:198,302,410] */
void naive_conv2d_fw_kernel_CHW(void *matMul_args);
void naive_conv2d_param_grad_kernel_CHW(void *matMul_args);
void naive_conv2d_in_grad_kernel_CHW(void *matMul_args);
/* the fixed-geometry forms: kernel 3x3 or 5x5, stride 2, padding 1 whatever the struct's fields say
 * [ref: pulp_conv_naive_fp32.h:112-170; pulp_conv_naive_fp32.c:520,581,643] */
void naive_conv2d_fw_kernel_CHW_k3x3_s2_p1(void *matMul_args);
void naive_conv2d_param_grad_kernel_CHW_k3x3_s2_p1(void *matMul_args);
void naive_conv2d_in_grad_kernel_CHW_k3x3_s2_p1(void *matMul_args);
void naive_conv2d_fw_kernel_CHW_k5x5_s2_p1(void *matMul_args);
void naive_conv2d_param_grad_kernel_CHW_k5x5_s2_p1(void *matMul_args);
void naive_conv2d_in_grad_kernel_CHW_k5x5_s2_p1(void *matMul_args);
/* workers the layer functions fork with a mm_manager_args: the product of mm_args, then (forward, USE_BIASES = 1) the bias of
 * row co added to C[co][0 .. M) [ref: pulp_conv2d_fp32.h:185,194; pulp_conv2d_fp32.c:669-800].  DEVIATION: the weight-gradient
 * worker leaves the bias gradient to pulp_conv2d_fp32_bw_param_grads_cl (the reference's loop there sums a tensor of the wrong shape). */
void im2col_conv2d_fw_kernel(void *mm_manager_args);
void im2col_conv2d_param_grad_kernel(void *mm_manager_args);

/* ---- pointwise conv [ref: pulp_conv_pw_fp32.h:62-95; pulp_conv_pw_fp32.c:27,104,121,233]
 * DEVIATION: input grad is correct for C_in != C_out (reference swaps N/M, :278-279). */
void pulp_conv_pw_fp32_fw_cl(void *PointWise_Conv_args);
void pulp_conv_pw_fp32_bw_cl(void *PointWise_Conv_args);
void pulp_conv_pw_fp32_bw_param_grads_cl(void *PointWise_Conv_args);
void pulp_conv_pw_fp32_bw_input_grads_cl(void *PointWise_Conv_args);

/* ---- depthwise conv [ref: pulp_conv_dw_fp32.h:72-111; pulp_conv_dw_fp32.c:27-86] */
void pulp_conv_dw_fp32_fw_cl(void *DepthWise_Conv_args);
void pulp_conv_dw_fp32_bw_cl(void *DepthWise_Conv_args);
void pulp_conv_dw_fp32_bw_param_grads_cl(void *DepthWise_Conv_args);
void pulp_conv_dw_fp32_bw_input_grads_cl(void *DepthWise_Conv_args);

/* ---- Linear [ref: pulp_linear_fp32.h:62-118; pulp_linear_fp32.c:25,70,85,142]
 * DEVIATION: with use_biases = 1 forward adds the bias (the fp32 reference skips it). */
void pulp_linear_fp32_fw_cl(void *Linear_args);
void pulp_linear_fp32_bw_cl(void *Linear_args);
void pulp_linear_fp32_bw_param_grads_cl(void *Linear_args);
void pulp_linear_fp32_bw_input_grads_cl(void *Linear_args);
/* workers forked with a mm_manager_args [ref: pulp_linear_fp32.h:120,130; pulp_linear_fp32.c:199-267]: the product of mm_args;
 * the weight-gradient worker also copies the output gradient A[0 .. N) into mm_args->bias when USE_BIASES = 1 */
void pulp_linear_fp32_fw_cl_kernel(void *mm_manager_args);
void pulp_linear_fp32_bw_param_grads_cl_kernel(void *mm_manager_args);

/* ---- multi-head self-attention [ref: pulp_mhsa_fp32.h:127-131; pulp_mhsa_fp32.c:20,648]
 * DEVIATION: backward uses the corrected transpose of V (reference :930 is wrong for L != H). */
void pulp_mhsa_fp32_fw_cl(void *Mhsa_args);
void pulp_mhsa_fp32_bw_cl(void *Mhsa_args);
/* Attention of the MobileBERT encoder block [ref: pulp_mhsa_fp32.h:147-156; pulp_mhsa_fp32.c:1749,2037,2111,2162,2413].
 * Token-major activations: input L x E (H = L, W = E), input_bn L x Kb, output L x No; coeff_in_q / coeff_in_k are
 * F x Kb, coeff_in_v is F x E, coeff_out is No x F, every projection adds its bias (as the reference does when built
 * with -DOPTIMIZE, which is how its tests build it).  The inference entry points take F = Kb = No = input_bn->W as the
 * reference does; the tiled entry point reads F, Kb and No from the H / W fields of the coefficient blobs.  q, k, v,
 * attention_map (F x L) and softmax_buffer (heads x L x L) are written as in the training path.
 * DEVIATION (backward): the reference's backward does not compile and reads output.diff as E x L although its forward
 * writes the output as L x No; here it is the gradient of the forward in the forward's layouts: coefficient gradients
 * in the coefficients' layouts, input.diff += the gradient through v, input_bn.diff += the gradient through q and k
 * (into input.diff instead when input_bn has no diff buffer and Kb = E, which is where the reference adds all three).
 * tiled_matmul_mhsa is the product (+ bias) of its matMul_args, tiled_transpose_mhsa the N x M transpose of its
 * transp_args; `projection` only selects tile sizes and is ignored. */
void pulp_mhsa_mobilebert_inference_fp32_fw_cl(void *Mhsa_args);
void pulp_mhsa_mobilebert_inference_fp32_bw_cl(void *Mhsa_args);
void tiled_mhsa_fp32(void *Mhsa_args, void *Tiled_Matmul_Mhsa_args);
void tiled_matmul_mhsa(void *matMul_args, void *Tiled_Matmul_Mhsa_args, int projection);
void tiled_transpose_mhsa(void *transp_args, void *Tiled_Matmul_Mhsa_args, int projection);

/* ---- activations and softmax [ref: pulp_act_fp32.h:89-289; pulp_act_fp32.c:25-392,714] */
void pulp_sigmoid_fp32_fw_cl(void *act_args);   void pulp_sigmoid_fp32_bw_cl(void *act_args);
void sigmoid_core_fw_fp32(void *act_args);      void sigmoid_core_bw_fp32(void *act_args);
void pulp_relu_fp32_fw_cl(void *act_args);      void pulp_relu_fp32_bw_cl(void *act_args);
void relu_core_fw_fp32(void *act_args);         void relu_core_bw_fp32(void *act_args);
void pulp_leakyrelu_fp32_fw_cl(void *leakyrelu_args); void pulp_leakyrelu_fp32_bw_cl(void *leakyrelu_args);
void leakyrelu_core_fw_fp32(void *leakyrelu_args);    void leakyrelu_core_bw_fp32(void *leakyrelu_args);
void pulp_softmax_fp32_fw_cl(void *softmax_args);
void pulp_softmax_fp32_bw_cl(void *softmax_args);
void pulp_gelu_tanh_approx_fp32_fw_cl(void *act_args);

/* ---- norms [ref: pulp_instnorm_fp32.h:57-87, pulp_batchnorm_fp32.h:74-80, pulp_layernorm_fp32.h:40] */
void pulp_instnorm_fp32_fw_cl(void *InstNorm_args);
void pulp_instnorm_fp32_bw_cl(void *InstNorm_args);
void pulp_instnorm_fp32_bw_param_grads_cl(void *InstNorm_args);
void pulp_instnorm_fp32_bw_input_grads_cl(void *InstNorm_args);
void pulp_instnorm_parallelized_fp32_fw_cl(void *InstNorm_args);
void pulp_instnorm_parallelized_fp32_bw_input_grads_cl(void *InstNorm_args);
void pulp_instnorm_parallelized_fp32_bw_param_grads_cl(void *InstNorm_args);
void pulp_batch_norm_fp32_fw_cl(void *BatchNorm_args_fp32);
void pulp_batch_norm_parallelized_fp32_fw_cl(void *BatchNorm_args_fp32);
void pulp_layerNorm_fp32_fw_cl(void *LayerNorm_args_fp32);

/* ---- losses [ref: pulp_losses_fp32.h:62-100; pulp_losses_fp32.c:26,91,214,254] */
void pulp_CrossEntropyLoss(void *loss_args);
void pulp_CrossEntropyLoss_backward(void *loss_args);
void pulp_MSELoss(void *loss_args);
void pulp_MSELoss_backward(void *loss_args);

/* ---- optimizer [ref: pulp_optimizers_fp32.h:50; pulp_optimizers_fp32.c:26] */
void pulp_gradient_descent_fp32(void *optim_args);

/* ---- residual [ref: pulp_residual_fp32.h:68-91; pulp_residual_fp32.c:27,59,92] */
void pulp_residualconn_fp32_fw(void *SkipConn_args);
void pulp_sumnode_fp32_bw(void *SkipConn_args);
void pulp_residualconn_fp32_bw(void *SkipConn_args);

/* ---- pooling [ref: pulp_pooling_fp32.h:52-58; pulp_pooling_fp32.c:24,69] */
void pulp_avgpool_fp32_fw_cl(void *pool_args);
void pulp_avgpool_fp32_bw_cl(void *pool_args);

/* ---- tensor helpers [ref: pulp_train_utils_fp32.h:609-852; pulp_train_utils_fp32.c:39-1329] (bit-exact) */
void transpose_matrix(void *transp_args);
void transpose(void *transp_args);
void copy(void *copy_args);
void set_to_value(void *set_to_value_args);
void vect_sum(void *vect_sum_args);
void array_broadcast_sum_fp32(void *array_broadcast_sum_fp32_args);
void HWC_to_CHW(void *layout_args);
void CHW_to_HWC(void *layout_args);
void pad_tensor(void *pad_args);        /* DEVIATION: correct zero padding for any pad (reference :957 only for 1) */
void pulp_scalar_mul_fp32_cl(void *scalar_mul_args);
void mm_bias_add_transposed(void *mm_bias_add_args);
void pulp_row_max_fp32_cl(void *max_args);
void pulp_exp_sum_fp32_cl(void *exp_sum_args);
void pulp_row_div_fp32_cl(void *row_div_args);
void pulp_mean_std_fp32_cl(void *mean_std_args);
void cast_fp16_tensor_to_fp32(void *cast_16t32_args);
float fastexp_gist(float x);            /* host-side scalar, same bit trick as the kernels use */
float q_rsqrt(float number);            /* DEVIATION: 32-bit integer pun (reference puns through `long`) */
int verify_tensor(float *tensor_out, float *tensor_ref, int size, float tolerance);

/* ================================================================== fp16 entry points */
/* Same contracts on fp16 storage with fp32 accumulation. */

/* [ref: pulp_matmul_fp16.h:49-136; pulp_matmul_fp16.c:191,273] argument: struct matMul_args_fp16 */
void mm_broadcast_fp16(void *broadcastMatMul_args_fp16);   /* [ref: pulp_matmul_fp16.c:30] */
void mm_fp16(void *matMul_args_fp16);
void mm_M_fp16(void *matMul_args_fp16);
/* the variants mm_manager_fp16 selects by matmul_type and tests fork by name [ref: pulp_matmul_fp16.h:56-134]: one product
 * (fp32 accumulation) behind every name; the mv_* forms are the M = 1 case */
void mm_fp16_SIMD_2x4(void *matMul_args_fp16);
void mm_fp16_SIMD_4x8(void *matMul_args_fp16);
void mm_fp16_unroll_8x1(void *matMul_args_fp16);
void mm_fp16_unroll_4x1(void *matMul_args_fp16);
void mm_fp16_unroll_2x1(void *matMul_args_fp16);
void mm_M_fp16_SIMD_2x4(void *matMul_args_fp16);
void mm_M_fp16_SIMD_4x8(void *matMul_args_fp16);
void mv_fp16_SIMD_2x1(void *matMul_args_fp16);
void mv_fp16_SIMD_4x1(void *matMul_args_fp16);
void mv_fp16_SIMD_8x1(void *matMul_args_fp16);
/* [ref: pulp_conv_naive_fp16.h; pulp_conv_naive_fp16.c] naive kernels and fixed-geometry forms on struct matMul_args_fp16 */
void naive_conv2d_fw_kernel_CHW_fp16(void *matMul_args_fp16);
void naive_conv2d_param_grad_kernel_CHW_fp16(void *matMul_args_fp16);
void naive_conv2d_in_grad_kernel_CHW_fp16(void *matMul_args_fp16);
void naive_conv2d_fw_kernel_CHW_k3x3_s2_p1_fp16(void *matMul_args_fp16);
void naive_conv2d_param_grad_kernel_CHW_k3x3_s2_p1_fp16(void *matMul_args_fp16);
void naive_conv2d_in_grad_kernel_CHW_k3x3_s2_p1_fp16(void *matMul_args_fp16);
void naive_conv2d_fw_kernel_CHW_k5x5_s2_p1_fp16(void *matMul_args_fp16);
void naive_conv2d_param_grad_kernel_CHW_k5x5_s2_p1_fp16(void *matMul_args_fp16);
void naive_conv2d_in_grad_kernel_CHW_k5x5_s2_p1_fp16(void *matMul_args_fp16);
/* forked workers [ref: pulp_conv2d_fp16.h; pulp_linear_fp16.h] */
void im2col_conv2d_fw_kernel_fp16(void *mm_manager_args_fp16);
void im2col_conv2d_param_grad_kernel_fp16(void *mm_manager_args_fp16);
void pulp_linear_fp16_fw_cl_kernel(void *mm_manager_args_fp16);
void pulp_linear_fp16_bw_param_grads_cl_kernel(void *mm_manager_args_fp16);
/* layout change of an fp16 blob [ref: pulp_train_utils_fp16.h:619,626] */
void HWC_to_CHW_fp16(void *layout_args_fp16);
void CHW_to_HWC_fp16(void *layout_args_fp16);
/* [ref: pulp_train_utils_fp16.h:661; pulp_train_utils_fp16.c:1258] */
void mm_manager_fp16(void *mm_manager_args_fp16);
/* [ref: pulp_im2col_fp16.h:30,38,53] */
void pulp_im2row_fp16(void *im2col_args_fp16);
void pulp_im2col_fp16(void *im2col_args_fp16);
void pulp_blocktransp_fp16(void *blocktransp_args_fp16);
/* [ref: pulp_conv2d_fp16.h:85-121; pulp_conv2d_fp16.c:27,225,240,458] */
void pulp_conv2d_fp16_fw_cl(void *Conv2D_args_fp16);
void pulp_conv2d_fp16_bw_cl(void *Conv2D_args_fp16);
void pulp_conv2d_fp16_bw_param_grads_cl(void *Conv2D_args_fp16);
void pulp_conv2d_fp16_bw_input_grads_cl(void *Conv2D_args_fp16);
/* [ref: pulp_conv_pw_fp16.h:63-96] */
void pulp_conv_pw_fp16_fw_cl(void *PointWise_Conv_args_fp16);
void pulp_conv_pw_fp16_bw_cl(void *PointWise_Conv_args_fp16);
void pulp_conv_pw_fp16_bw_param_grads_cl(void *PointWise_Conv_args_fp16);
void pulp_conv_pw_fp16_bw_input_grads_cl(void *PointWise_Conv_args_fp16);
/* [ref: pulp_conv_dw_fp16.h:63-102] stride is always 1 (the struct has no stride fields) */
void pulp_conv_dw_fp16_fw_cl(void *DepthWise_Conv_args_fp16);
void pulp_conv_dw_fp16_bw_cl(void *DepthWise_Conv_args_fp16);
void pulp_conv_dw_fp16_bw_param_grads_cl(void *DepthWise_Conv_args_fp16);
void pulp_conv_dw_fp16_bw_input_grads_cl(void *DepthWise_Conv_args_fp16);
/* [ref: pulp_linear_fp16.h:62-118; pulp_linear_fp16.c:25,70,85,149] */
void pulp_linear_fp16_fw_cl(void *Linear_args_fp16);
void pulp_linear_fp16_bw_cl(void *Linear_args_fp16);
void pulp_linear_fp16_bw_param_grads_cl(void *Linear_args_fp16);
void pulp_linear_fp16_bw_input_grads_cl(void *Linear_args_fp16);
/* [ref: pulp_mhsa_fp16.h:164-165; pulp_mhsa_fp16.c:20,645] */
void pulp_mhsa_fp16_fw_cl(void *Mhsa_args_fp16);
void pulp_mhsa_fp16_bw_cl(void *Mhsa_args_fp16);
/* [ref: pulp_mhsa_fp16.h:184-192; pulp_mhsa_fp16.c:1731] fp16 twins of the MobileBERT attention entry points (the
 * backward is this library's addition: the reference has no fp16 one) */
void pulp_mhsa_mobilebert_inference_fp16_fw_cl(void *Mhsa_args_fp16);
void pulp_mhsa_mobilebert_inference_fp16_bw_cl(void *Mhsa_args_fp16);
void tiled_mhsa_fp16(void *Mhsa_args_fp16, void *Tiled_Matmul_Mhsa_args_fp16);
void tiled_matmul_mhsa_fp16(void *matMul_args_fp16, void *Tiled_Matmul_Mhsa_args_fp16, int projection);
void tiled_transpose_mhsa_fp16(void *transp_args_fp16, void *Tiled_Matmul_Mhsa_args_fp16, int projection);
/* [ref: pulp_act_fp16.h:90-204; pulp_act_fp16.c:185,226,359] */
void pulp_relu_fp16_fw_cl(void *act_args_fp16);       void pulp_relu_fp16_bw_cl(void *act_args_fp16);
void relu_core_fw_fp16(void *act_args_fp16);          void relu_core_bw_fp16(void *act_args_fp16);
void pulp_leakyrelu_fp16_fw_cl(void *leakyrelu_args_fp16); void pulp_leakyrelu_fp16_bw_cl(void *leakyrelu_args_fp16);
void pulp_sigmoid_fp16_fw_cl(void *act_args_fp16);    void pulp_sigmoid_fp16_bw_cl(void *act_args_fp16);
void pulp_softmax_fp16_fw_cl(void *softmax_args_fp16);
void pulp_softmax_fp16_bw_cl(void *softmax_args_fp16);
void pulp_gelu_fp16_fw_cl(void *act_args_fp16);
/* [ref: pulp_instnorm_fp16.h:57-87] */
void pulp_instnorm_fp16_fw_cl(void *InstNorm_args_fp16);
void pulp_instnorm_fp16_bw_cl(void *InstNorm_args_fp16);
void pulp_instnorm_fp16_bw_param_grads_cl(void *InstNorm_args_fp16);
void pulp_instnorm_fp16_bw_input_grads_cl(void *InstNorm_args_fp16);
/* [ref: pulp_losses_fp16.h:63-101; pulp_losses_fp16.c:26,88,212,252] */
void pulp_CrossEntropyLoss_fp16(void *loss_args_fp16);
void pulp_CrossEntropyLoss_backward_fp16(void *loss_args_fp16);
void pulp_MSELoss_fp16(void *loss_args_fp16);
void pulp_MSELoss_backward_fp16(void *loss_args_fp16);
/* [ref: pulp_optimizers_fp16.h:51; pulp_optimizers_fp16.c:26] */
void pulp_gradient_descent_fp16(void *optim_args_fp16);
/* [ref: pulp_residual_fp16.h:68-91; pulp_residual_fp16.c:30,67,100] */
void pulp_residualconn_fp16_fw(void *SkipConn_args_fp16);
void pulp_sumnode_fp16_bw(void *SkipConn_args_fp16);
void pulp_residualconn_fp16_bw(void *SkipConn_args_fp16);
/* [ref: pulp_pooling_fp16.h:52-58; pulp_pooling_fp16.c:24,69] */
void pulp_avgpool_fp16_fw_cl(void *pool_args_fp16);
void pulp_avgpool_fp16_bw_cl(void *pool_args_fp16);
/* [ref: pulp_train_utils_fp16.h:560-803] */
void transpose_matrix_fp16(void *transp_args_fp16);
void transpose_fp16(void *transp_args_fp16);
void copy_fp16(void *copy_args_fp16);
void set_to_value_fp16(void *set_to_value_args_fp16);
void vect_sum_fp16(void *vect_sum_args_fp16);
void array_broadcast_sum_fp16(void *array_broadcast_sum_fp16_args);
void pad_tensor_fp16(void *pad_args_fp16);
void cast_fp32_tensor_to_fp16(void *cast_32t16_args);
void pulp_scalar_mul_fp16_cl(void *scalar_mul_args_fp16);
void mm_bias_add_transposed_fp16(void *mm_bias_add_args_fp16);

/* ---- the depthwise workers behind pulp_conv_dw_* [ref: pulp_conv_naive_fp32.h:27-45; pulp_conv_naive_fp32.c:29-330;
 * pulp_conv_naive_fp16.h:27-45].  The fp32 ones read stride and padding from kernel_DW_args; the fp16 struct has only
 * the three blobs (stride 1, no padding).  weight_grad writes weights.diff, input_grad writes input.diff. */
struct kernel_DW_args_fp16 { struct blob_fp16 *input; struct blob_fp16 *weights; struct blob_fp16 *output; };
void dw_kernel_forward(void *kernel_DW_args);           void dw_kernel_forward_fp16(void *kernel_DW_args_fp16);
void dw_kernel_weight_grad(void *kernel_DW_args);       void dw_kernel_weight_grad_fp16(void *kernel_DW_args_fp16);
void dw_kernel_input_grad(void *kernel_DW_args);        void dw_kernel_input_grad_fp16(void *kernel_DW_args_fp16);

/* ---- the rest of the element-wise family [ref: pulp_losses_fp32.h:79-121, pulp_pooling_fp32.h:64-70, pulp_nonorm_fp32.h:53,
 * pulp_rmsnorm_fp32.h:33-49, pulp_act_fp32.h:274-281; the fp16 twins in the _fp16 headers].  Losses and pooling work on
 * every stream in streams mode like their MSE / average-pool siblings.  The "one value per core" outputs of the
 * reference's workers (maxes[core], sums[core], out[core]) have one entry here, index 0: this library is one core. */
void pulp_L1Loss(void *loss_args);                 void pulp_L1Loss_backward(void *loss_args);
void pulp_L1Loss_fp16(void *loss_args_fp16);       void pulp_L1Loss_backward_fp16(void *loss_args_fp16);
void pulp_berHuLoss(void *berHu_loss_args);        void pulp_berHuLoss_backward(void *berHu_loss_args);
void pulp_berHuLoss_fp16(void *berHu_loss_args_fp16);  void pulp_berHuLoss_backward_fp16(void *berHu_loss_args_fp16);
void pulp_maxpool_fp32_fw_cl(void *pool_args);     void pulp_maxpool_fp32_bw_cl(void *pool_args);
void pulp_maxpool_fp16_fw_cl(void *pool_args_fp16); void pulp_maxpool_fp16_bw_cl(void *pool_args_fp16);
void pulp_nonorm_fp32_fw_cl(void *Nonorm_args);    void pulp_nonorm_fp16_fw_cl(void *Nonorm_args_fp16);
void weighted_scaling_fp32_cl(void *weighted_scaling_args);  void weighted_scaling_fp16_cl(void *weighted_scaling_args_fp16);
void sum_of_squares_fp32_cl(void *sum_of_squares_args);      void sum_of_squares_fp16_cl(void *sum_of_squares_args_fp16);
void rmsnorm_parallelized_fp32(float *o, float *x, float *weight, float *buffer_n_cores, int size);
void rmsnorm_parallelized_fp16(fp16 *o, fp16 *x, fp16 *weight, fp16 *buffer_n_cores, int size);
void pulp_swiglu_fp32_cl(void *swiglu_args);       void pulp_swiglu_fp16_cl(void *swiglu_args_fp16);
void pulp_vector_softmax_fp32(float *out, float *in, float *buffer_n_cores, unsigned int size);
void pulp_vector_softmax_fp16(fp16 *out, fp16 *in, fp16 *buffer_n_cores, unsigned int size);
/* pieces of the reference's softmax [ref: pulp_train_utils_fp32.h:707-834; pulp_train_utils_fp16.h:399-760] */
void pulp_max_fp32_cl(void *max_args);             void pulp_max_fp16_cl(void *max_args_fp16);
void pulp_div_fp32_cl(void *div_args);             void pulp_div_fp16_cl(void *div_args_fp16);
void pulp_shift_sum_fp32_cl(void *shift_sum_args);
void vector_exp_sum_fp32_cl(void *vector_exp_sum_args);  void vector_exp_sum_fp16_cl(void *vector_exp_sum_args_fp16);
void pulp_sm_bw_op_1(void *sm_bw_op_1_args);       void pulp_sm_bw_op_1_fp16(void *sm_bw_op_1_args_fp16);
void pulp_sm_bw_op_2(void *sm_bw_op_2_args);       void pulp_sm_bw_op_2_fp16(void *sm_bw_op_2_args_fp16);
void pulp_row_max_fp16_cl(void *max_args_fp16);    void pulp_exp_sum_fp16_cl(void *exp_sum_args_fp16);
void pulp_row_div_fp16_cl(void *row_div_args_fp16); void pulp_mean_std_fp16_cl(void *mean_std_args_fp16);
/* fp16 twins of the forkable activation workers and of the parallelised instance norm
 * [ref: pulp_act_fp16.h; pulp_instnorm_fp16.h] */
void sigmoid_core_fw_fp16(void *act_args_fp16);    void sigmoid_core_bw_fp16(void *act_args_fp16);
void leakyrelu_core_fw_fp16(void *leakyrelu_args_fp16);  void leakyrelu_core_bw_fp16(void *leakyrelu_args_fp16);
void pulp_instnorm_parallelized_fp16_fw_cl(void *InstNorm_args_fp16);
void pulp_instnorm_parallelized_fp16_bw_input_grads_cl(void *InstNorm_args_fp16);
void pulp_instnorm_parallelized_fp16_bw_param_grads_cl(void *InstNorm_args_fp16);

#ifdef __cplusplus
}
#endif
#endif /* TRAINLIB_B200_ABI_H */
