/*
 * resnet8_streams.h - the batched training workload: a small ResNet (conv3x3 stem of 16 channels,
 * three residual stages of 16/32/64 channels with stride-2 downsampling and 1x1 projection
 * shortcuts, a norm and ReLU after every 3x3 conv, global average pool, Linear 64 -> 10,
 * CrossEntropy) trained on n independent batch-1 streams whose weight gradients are summed.
 *
 * The network is ordinary user code of the PULP-TrainLib API (struct blob, Conv2D_args,
 * InstNorm_args, ... and the pulp_*_cl calls), in the style of the code TrainLib_Deployer
 * generates.  The same source builds against libtrainlib_b200.so (streams mode: one call per
 * layer covers all streams) and, with -DNET_REFERENCE, against the reference library, where
 * every call is repeated per stream.
 */
#ifndef RESNET8_STREAMS_H
#define RESNET8_STREAMS_H
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

#define RESNET8_CLASSES 10
#define RESNET8_IMAGE_FLOATS (3 * 32 * 32)

size_t resnet8_param_count(void);                 /* floats in the flat parameter (and gradient) buffer */
size_t resnet8_workspace_floats(int n_streams);   /* floats of activation / gradient workspace */
/* He-style seeded initialisation of a host copy of the parameters (norm gamma = 1, beta = 0). */
void   resnet8_init_params(float *host_params, unsigned seed);
/* Wire the network onto caller-owned buffers (host or device pointers).  Returns 0 on success. */
int    resnet8_bind(int n_streams, float *params, float *grads, float *workspace);
/* images [n][3][32][32], labels one-hot [n][10]; loss [n] receives the per-stream CrossEntropy. */
void   resnet8_forward(const float *images, const float *labels, float *loss);
/* Same step for callers whose batch lives in host memory: the images and labels are copied into
 * the workspace once (they are read by the forward, the loss backward and the stem's weight
 * gradient), the losses are copied back. */
void   resnet8_forward_host(const float *host_images, const float *host_labels, float *host_loss);
void   resnet8_backward(void);                    /* fills the flat gradient buffer (sum over streams) */
void   resnet8_update(float lr);                  /* SGD on every parameter blob */
float *resnet8_logits(void);                      /* [n][10], inside the workspace */
int    resnet8_param_blobs(void);                 /* number of parameter tensors */
size_t resnet8_param_offset(int i, size_t *count);/* offset/size of parameter tensor i in the flat buffer */
void   resnet8_set_fusion(int on);                /* 1 (default): norm + residual sum + ReLU as one library call; 0: separate calls */
double resnet8_flops_per_stream(void);            /* FW + WG + IG multiply-add FLOPs of the convs and the Linear */

#ifdef __cplusplus
}
#endif
#endif
