/*
 * tinycnn_b200.h -- C ABI of the B200 (sm_100a) training hot path for tiny-dnn.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, and returns
 * an int status: 0 = ok, non-zero = error (text via b200_last_error()).  The C++
 * host shim turns a non-zero status into `throw nn_error(...)`, the reference's
 * only error convention (tiny_dnn/util/nn_error.h:19-27).
 *
 * Pointer convention: unless a parameter is documented as HOST memory, every
 * float/uint8/int32 buffer is DEVICE memory on the context's GPU.  The
 * `*_host` entry points take HOST buffers, stage them through the context's
 * device arena and copy results back; they are what the reference-side
 * OpKernel branches call (tensor_t rows are host vectors).
 *
 * Tensor layouts are the reference's own: a batch is `B` rows, each row planar
 * CHW, index (H*c + y)*W + x (tiny_dnn/util/util.h:168-173), rows stored back to
 * back.  Convolution weights are [(in_c*o + inc)][ky][kx]
 * (tiny_dnn/core/kernels/conv2d_op_internal.h:41); fully-connected weights are
 * row-major [in][out] (tiny_dnn/core/kernels/fully_connected_op_internal.h:28).
 *
 * Gradient convention: the reference keeps one dW/db row per sample and sums
 * the rows later (tiny_dnn/node.h:89-103).  The device path produces the batch
 * SUM directly (no 1/B factor: tiny_dnn/layers/layer.h:663-673 scales by 1.0).
 */
#ifndef TINYCNN_B200_H_
#define TINYCNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define B200_API
#else
#define B200_API __attribute__((visibility("default")))
#endif

/* ------------------------------------------------------------------------- */
/* Runtime                                                                     */
/* ------------------------------------------------------------------------- */

typedef struct b200_ctx b200_ctx;

/* Library version, "major.minor". */
B200_API const char *b200_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
B200_API const char *b200_last_error(void);

/* Number of CUDA devices visible; 0 when there is no usable GPU. */
B200_API int b200_device_count(void);

/*
 * Create a context bound to `device`.  `stream` is a cudaStream_t the caller
 * owns (NULL = the context creates its own non-blocking stream).  All work of
 * the context is issued on that stream.  Replaces nothing in the reference
 * (it has no device context on this path; core/framework/device.fwd.h:38-112 is
 * the OpenCL-only analogue).
 */
B200_API int b200_ctx_create(int device, void *stream, b200_ctx **out);
B200_API int b200_ctx_destroy(b200_ctx *ctx);
B200_API int b200_ctx_set_stream(b200_ctx *ctx, void *stream);
B200_API void *b200_ctx_stream(b200_ctx *ctx);
B200_API int b200_ctx_sync(b200_ctx *ctx);

/*
 * Context options.  "fc_tensor_cores": 0 = fully-connected GEMMs always on the
 * fp32 FFMA kernels, 1 (default) = large ones on the tensor cores with the
 * 3xTF32 split (fp32-level accuracy), 2 = every GEMM the tensor-core kernel can
 * take.  "conv_tensor_cores": 0 = convolutions never on the tensor cores,
 * 1 (default) = stride-1 layers with at least 16 input and 16 output
 * channels, 2 = every pass the tensor-core kernels can take (stride 1,
 * dilation 1, windows up to 8x8, at most 256 channels either side).  Unknown names are an error.
 */
B200_API int b200_ctx_set_option(b200_ctx *ctx, const char *name, int value);

/* Raw device memory helpers for hosts that do not link the CUDA runtime. */
B200_API int b200_malloc(b200_ctx *ctx, size_t bytes, void **out);
B200_API int b200_free(b200_ctx *ctx, void *ptr);
B200_API int b200_memcpy_h2d(b200_ctx *ctx, void *dst, const void *src, size_t bytes);
B200_API int b200_memcpy_d2h(b200_ctx *ctx, void *dst, const void *src, size_t bytes);
B200_API int b200_memset(b200_ctx *ctx, void *dst, int value, size_t bytes);
/*
 * Page-locked host memory (cudaHostAlloc) for callers without the CUDA headers: the *_host entry
 * points and b200_net_fit_host copy asynchronously, and overlap uploads with compute, only from
 * such memory.  It replaces the std::vector<vec_t> staging of network::fit (network.h:911-926).
 */
B200_API int b200_host_alloc(size_t bytes, void **out);
B200_API int b200_host_free(void *ptr);

/* ------------------------------------------------------------------------- */
/* Convolution  (a1-a3)                                                        */
/* ------------------------------------------------------------------------- */

/*
 * Plain-C mirror of core::conv_params (tiny_dnn/core/params/conv_params.h:63-90).
 * `tbl` is a HOST array of in_c*out_c bytes in connection_table order
 * connected_[inc*out_c + o] (conv_params.h:52-54), or NULL for a full table.
 */
typedef struct b200_conv_desc {
  int32_t in_w, in_h, in_c;     /* params.in                                  */
  int32_t inp_w, inp_h;         /* params.in_padded (same: in + k - 1)        */
  int32_t out_w, out_h, out_c;  /* params.out                                 */
  int32_t k_w, k_h;             /* params.weight width/height                 */
  int32_t stride_w, stride_h;
  int32_t dil_w, dil_h;         /* forward only; backward ignores dilation as */
                                /* conv2d_op_internal.h:118-123,139-160 does  */
  int32_t has_bias;
  int32_t pad_same;             /* padding::same = 1, padding::valid = 0      */
  int32_t input_is_padded;      /* 1: `in`/`din` rows already have in_padded  */
                                /* geometry, as Conv2dOp::compute receives    */
                                /* them (convolutional_layer.h:283-299)       */
  int32_t algo;                 /* 0 auto, 1 general kernels, 2 tiled FFMA kernels, 3 tensor-core kernels */
  const uint8_t *tbl;           /* HOST, may be NULL                          */
} b200_conv_desc;

/*
 * Fill a descriptor the way convolutional_layer::conv_set_params does
 * (tiny_dnn/layers/convolutional_layer.h:404-438; conv_out_length
 * util/util.h:329-344).
 */
B200_API int b200_conv_desc_init(b200_conv_desc *d, int in_w, int in_h, int in_c,
                                 int k_w, int k_h, int out_c, int pad_same,
                                 int has_bias, int stride_w, int stride_h,
                                 int dil_w, int dil_h);

/*
 * out = conv(in, W) + bias.  Replaces kernels::conv2d_op_internal forward
 * (tiny_dnn/core/kernels/conv2d_op_internal.h:13-74) as dispatched by
 * Conv2dOp::compute (tiny_dnn/core/kernels/conv2d_op.h:23-51).  `out` is
 * overwritten.  in: B x (in_c*in_h*in_w) (or in_padded geometry when
 * input_is_padded); out: B x (out_c*out_h*out_w).
 */
B200_API int b200_conv2d_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in,
                             const float *W, const float *bias, float *out, int batch);

/*
 * din = dX, dW (+)= sum_n dW_n, db (+)= sum_n db_n.  Replaces the backward
 * kernels::conv2d_op_internal (conv2d_op_internal.h:78-181) as dispatched by
 * Conv2dGradOp::compute (tiny_dnn/core/kernels/conv2d_grad_op.h:22-50).  `din`
 * is overwritten (NULL skips dX); dW/db are overwritten when accumulate == 0
 * and added to when accumulate != 0 (the reference never clears them,
 * conv2d_op_internal.h:165,177).  db may be NULL when has_bias == 0.
 */
B200_API int b200_conv2d_bwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in,
                             const float *W, const float *dout, float *din, float *dW,
                             float *db, int accumulate, int batch);

/*
 * Measurement hook (no counterpart in the reference): average device time in
 * milliseconds of the MAIN kernel of one convolution pass -- pass 0 forward,
 * 1 dX, 2 dW -- over `reps` launches, timed with CUDA events on the context's
 * stream.  The operand copies and filter matrices a pass needs are prepared
 * once, outside the timed region; the small prepare / merge kernels are not
 * part of the figure (on the tiled FFMA path the filter re-layout kernel is,
 * because that launcher issues both).  `*on_tensor_cores` reports which kernel
 * family ran.  All pointers are DEVICE memory.
 */
B200_API int b200_conv2d_time_pass(b200_ctx *ctx, const b200_conv_desc *d, const float *in,
                                   const float *W, const float *dout, int batch, int pass, int reps,
                                   float *ms, int *on_tensor_cores);

/*
 * Weight gradient only -- dW (+)= sum_n dW_n, db (+)= sum_n db_n, the same
 * values b200_conv2d_bwd produces -- for callers that are not allowed to
 * allocate device memory at call time.  It has NO counterpart in the reference.
 *
 * Who needs it: a host that handed all of its HBM to its own pools at start-up
 * and has nothing left for cudaMalloc to find, or a latency-bound loop that
 * cannot take the device-wide synchronisation cudaMalloc/cudaFree imply.  The
 * other entry points grow a per-context scratch buffer on demand; this one
 * takes no context and never calls cudaMalloc, cudaFree or any allocating
 * routine.  Its scratch (the partial sums of the batch slices) is a fixed
 * 16 MiB array compiled into the library, which every GPU that loads the
 * library therefore carries until the process exits.
 *
 * Limits and rules:
 *  - `stream` is a cudaStream_t (NULL = the default stream); all pointers are
 *    DEVICE memory of the CURRENT device, which the caller selects beforehand.
 *  - stride 1, dilation 1, 3x3 or 5x5 windows, output width <= 64, no
 *    connection table (d->tbl must be NULL); anything else is refused with an
 *    error text, as is a filter tensor whose single partial row (out_c*in_c*k*k
 *    + out_c floats) exceeds the 4 Mi-float array.
 *  - The first call on each device looks up the array's device address; make
 *    that first call before any stream capture begins.  With lazy module loading
 *    (the default since CUDA 12.2) the library's device code, this array included,
 *    is only placed on a GPU when it is first used there, so that first call is
 *    also when the 16 MiB are taken: make it before the host hands the rest of
 *    the memory to its own pools (or run with CUDA_MODULE_LOADING=EAGER).
 *  - All calls share the one array and leave their partial sums in it.  No
 *    call depends on what an earlier call left behind (every element that is
 *    read is written first), but two calls whose kernels overlap in time on the
 *    same GPU -- different streams, different threads -- race on it.
 */
B200_API int b200_conv2d_dw_noalloc(void *stream, const b200_conv_desc *d, const float *in,
                                    const float *dout, float *dW, float *db, int accumulate,
                                    int batch);

/* HOST-buffer forms of the two calls above (what the OpKernel branches call). */
B200_API int b200_conv2d_fwd_host(b200_ctx *ctx, const b200_conv_desc *d, const float *in,
                                  const float *W, const float *bias, float *out, int batch);
B200_API int b200_conv2d_bwd_host(b200_ctx *ctx, const b200_conv_desc *d, const float *in,
                                  const float *W, const float *dout, float *din, float *dW,
                                  float *db, int accumulate, int batch);

/* ------------------------------------------------------------------------- */
/* Fully connected  (a4-a5)                                                    */
/* ------------------------------------------------------------------------- */

/*
 * out[n][i] = b[i] + sum_c W[c*out+i] * in[n][c].  Replaces
 * kernels::fully_connected_op_internal forward
 * (tiny_dnn/core/kernels/fully_connected_op_internal.h:15-36) as dispatched by
 * FullyConnectedOp::compute (tiny_dnn/core/kernels/fully_connected_op.h:25-64).
 * bias may be NULL (fully_params::has_bias_ == false).
 */
B200_API int b200_fc_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in,
                         const float *W, const float *bias, float *out, int batch);

/*
 * din[n][c] = dot(dout[n], W[c*out..]); dW[c*out+i] (+)= sum_n dout[n][i]*in[n][c];
 * db[i] (+)= sum_n dout[n][i].  Replaces the backward
 * kernels::fully_connected_op_internal (fully_connected_op_internal.h:38-71) as
 * dispatched by FullyConnectedGradOp::compute
 * (tiny_dnn/core/kernels/fully_connected_grad_op.h:22-52).  din may be NULL.
 */
B200_API int b200_fc_bwd(b200_ctx *ctx, int in_size, int out_size, const float *in,
                         const float *W, const float *dout, float *din, float *dW,
                         float *db, int accumulate, int batch);

B200_API int b200_fc_fwd_host(b200_ctx *ctx, int in_size, int out_size, const float *in,
                              const float *W, const float *bias, float *out, int batch);
B200_API int b200_fc_bwd_host(b200_ctx *ctx, int in_size, int out_size, const float *in,
                              const float *W, const float *dout, float *din, float *dW,
                              float *db, int accumulate, int batch);

/* ------------------------------------------------------------------------- */
/* Pooling  (a6-a7)                                                            */
/* ------------------------------------------------------------------------- */

/* Mirror of core::maxpool_params (tiny_dnn/core/params/maxpool_params.h:17-34). */
typedef struct b200_pool_desc {
  int32_t in_w, in_h, in_c;
  int32_t out_w, out_h;
  int32_t pool_w, pool_h;
  int32_t stride_w, stride_h;
} b200_pool_desc;

/* Output size per pool_out_length (tiny_dnn/util/util.h:346-363). */
B200_API int b200_pool_desc_init(b200_pool_desc *d, int in_w, int in_h, int in_c,
                                 int pool_w, int pool_h, int stride_w, int stride_h,
                                 int ceil_mode, int pad_same);

/*
 * Max pooling forward: strict `>` scan of the (border-clipped) window in
 * row-major order; `argmax` receives the winning in-row index (the reference's
 * params.out2inmax).  Replaces kernels::maxpool_op_internal
 * (tiny_dnn/core/kernels/maxpool_op_internal.h:16-39) as dispatched by
 * MaxPoolOp::compute (tiny_dnn/core/kernels/maxpool_op.h:23-61); window tables
 * tiny_dnn/layers/max_pooling_layer.h:195-235.
 */
B200_API int b200_maxpool_fwd(b200_ctx *ctx, const b200_pool_desc *d, const float *in,
                              float *out, int32_t *argmax, int batch);

/*
 * din[i] = (argmax[in2out(i)] == i) ? dout[in2out(i)] : 0 with in2out(i) the
 * LAST window covering i (0 when none does).  Replaces
 * kernels::maxpool_grad_op_internal (maxpool_op_internal.h:41-57) as dispatched
 * by MaxPoolGradOp::compute (tiny_dnn/core/kernels/maxpool_grad_op.h:22-47).
 */
B200_API int b200_maxpool_bwd(b200_ctx *ctx, const b200_pool_desc *d, const float *dout,
                              const int32_t *argmax, float *din, int batch);

B200_API int b200_maxpool_fwd_host(b200_ctx *ctx, const b200_pool_desc *d, const float *in,
                                   float *out, int32_t *argmax, int batch);
B200_API int b200_maxpool_bwd_host(b200_ctx *ctx, const b200_pool_desc *d, const float *dout,
                                   const int32_t *argmax, float *din, int batch);

/*
 * Average pooling with the reference's trainable per-channel scale and bias:
 * out = (sum window) * W[c] * 1/(pool_w*pool_h) + b[c].  Replaces
 * tiny_average_pooling_kernel (tiny_dnn/layers/average_pooling_layer.h:25-55).
 * W has pool_w*pool_h*in_c entries of which only the first in_c are used
 * (average_pooling_layer.h:231-233; partial_connected_layer.h:24-35).
 */
B200_API int b200_avgpool_fwd(b200_ctx *ctx, const b200_pool_desc *d, const float *in,
                              const float *W, const float *bias, float *out, int batch);

/*
 * din = W[c]*scale*dout[first window covering i]; dW[c] (+)= scale*sum in*dout;
 * db[c] (+)= sum dout.  Replaces tiny_average_pooling_back_kernel
 * (average_pooling_layer.h:58-106).  dW has pool_w*pool_h*in_c entries; entries
 * >= in_c receive 0.
 */
B200_API int b200_avgpool_bwd(b200_ctx *ctx, const b200_pool_desc *d, const float *in,
                              const float *W, const float *dout, float *din, float *dW,
                              float *db, int accumulate, int batch);

B200_API int b200_avgpool_fwd_host(b200_ctx *ctx, const b200_pool_desc *d, const float *in,
                                   const float *W, const float *bias, float *out, int batch);
B200_API int b200_avgpool_bwd_host(b200_ctx *ctx, const b200_pool_desc *d, const float *in,
                                   const float *W, const float *dout, float *din, float *dW,
                                   float *db, int accumulate, int batch);

/* ------------------------------------------------------------------------- */
/* Activations and loss gradients  (a8-a9)                                     */
/* ------------------------------------------------------------------------- */

enum {
  B200_ACT_NONE = 0,
  B200_ACT_RELU = 1,
  B200_ACT_TANH = 2,
  B200_ACT_SOFTMAX = 3,
  B200_ACT_SIGMOID = 4,    /* tiny_dnn/activations/sigmoid_layer.h:24-39                        */
  B200_ACT_LEAKY_RELU = 5, /* leaky_relu_layer.h:74-90; parameter = epsilon (0.01 by default)    */
  B200_ACT_ELU = 6         /* elu_layer.h:38-57; parameter = alpha (1 by default)                */
};

/*
 * y = f(x) row by row (`dim` elements per row).  Replaces
 * relu_layer/tanh_layer/softmax_layer::forward_activation
 * (tiny_dnn/activations/relu_layer.h:25-29, tanh_layer.h:24-28,
 * softmax_layer.h:24-34) under activation_layer::forward_propagation
 * (tiny_dnn/activations/activation_layer.h:74-79).
 */
B200_API int b200_act_fwd(b200_ctx *ctx, int kind, const float *x, float *y, int dim, int batch);

/*
 * dx from (y, dy): relu dy*(y>0), tanh dy*(1-y*y), softmax
 * dx_j = sum_k dy_k*(k==j ? y_j(1-y_j) : -y_k*y_j).  Replaces the
 * backward_activation members (relu_layer.h:31-39, tanh_layer.h:30-38,
 * softmax_layer.h:36-55).
 */
B200_API int b200_act_bwd(b200_ctx *ctx, int kind, const float *y, const float *dy, float *dx,
                          int dim, int batch);

/*
 * The same two calls for the activations that carry a constructor parameter:
 * sigmoid y = 1/(1+exp(-x)), dx = dy*y*(1-y) (parameter unused); leaky relu
 * y = x > 0 ? x : epsilon*x, dx = dy*(y > 0 ? 1 : epsilon)
 * (leaky_relu_layer.h:74-90, `epsilon_`); elu y = x < 0 ? alpha*(exp(x)-1) : x,
 * dx = dy*(y > 0 ? 1 : alpha + y) (elu_layer.h:38-57, `alpha_`).  The
 * parameterless calls above run these kinds with the reference's default
 * parameters (0.01, 1).
 */
B200_API int b200_act_param_fwd(b200_ctx *ctx, int kind, float param, const float *x, float *y,
                                int dim, int batch);
B200_API int b200_act_param_bwd(b200_ctx *ctx, int kind, float param, const float *y,
                                const float *dy, float *dx, int dim, int batch);
B200_API int b200_act_param_fwd_host(b200_ctx *ctx, int kind, float param, const float *x,
                                     float *y, int dim, int batch);
B200_API int b200_act_param_bwd_host(b200_ctx *ctx, int kind, float param, const float *y,
                                     const float *dy, float *dx, int dim, int batch);

B200_API int b200_act_fwd_host(b200_ctx *ctx, int kind, const float *x, float *y, int dim,
                               int batch);
B200_API int b200_act_bwd_host(b200_ctx *ctx, int kind, const float *y, const float *dy,
                               float *dx, int dim, int batch);

enum { B200_LOSS_MSE = 0, B200_LOSS_CROSS_ENTROPY = 1, B200_LOSS_CROSS_ENTROPY_MULTICLASS = 2 };

/* ------------------------------------------------------------------------- */
/* Layers between the hot operators: batch normalization, dropout, LRN         */
/* ------------------------------------------------------------------------- */

/*
 * batch_normalization_layer::forward_propagation
 * (tiny_dnn/layers/batch_normalization_layer.h:136-168) on rows of
 * `channels` x `spatial` values.  train != 0 (net_phase::train): `mean` and
 * `variance` receive this mini-batch's moments (moments(),
 * tiny_dnn/util/math_functions.h:25-96: mean = sum / (batch*spatial),
 * variance = sum (x-mean)^2 / max(1, batch*spatial - 1)); train == 0: they
 * are read (the layer's moving averages).  `stddev` always receives
 * sqrt(variance + eps), and y = (x - mean) / stddev.  The sums are formed by
 * a fixed tree, not in the reference's sample-by-sample order: results agree
 * with the reference to rounding, not bit for bit.
 */
B200_API int b200_batchnorm_fwd(b200_ctx *ctx, int channels, int spatial, float eps, const float *x,
                                float *mean, float *variance, float *stddev, float *y, int batch,
                                int train);
/*
 * batch_normalization_layer::back_propagation (:94-134):
 * dx = (dy - mean(dy) - mean(dy*y) * y) / stddev, the means per channel over
 * batch x spatial; `stddev` as the forward pass left it.
 */
B200_API int b200_batchnorm_bwd(b200_ctx *ctx, int channels, int spatial, const float *y,
                                const float *dy, const float *stddev, float *dx, int batch);
/* batch_normalization_layer::post_update (:174-180):
 * mean = momentum*mean + (1-momentum)*mean_cur, the same for the variance. */
B200_API int b200_batchnorm_post_update(b200_ctx *ctx, int channels, float momentum, float *mean,
                                        float *variance, const float *mean_cur,
                                        const float *var_cur);
B200_API int b200_batchnorm_fwd_host(b200_ctx *ctx, int channels, int spatial, float eps,
                                     const float *x, float *mean, float *variance, float *stddev,
                                     float *y, int batch, int train);
B200_API int b200_batchnorm_bwd_host(b200_ctx *ctx, int channels, int spatial, const float *y,
                                     const float *dy, const float *stddev, float *dx, int batch);

/*
 * dropout_layer in the train phase with the mask the caller drew
 * (tiny_dnn/layers/dropout_layer.h:95-115: the reference draws it from its
 * host generator inside a parallel loop, so only a mask handed over can
 * reproduce a run): out = mask * scale * in with scale = 1 / (1 - rate).
 * The backward pass (:66-84) is the same call on dy with scale = 1 -- the
 * reference does not scale the gradient.  `n` values, one mask byte each.
 */
B200_API int b200_dropout(b200_ctx *ctx, const float *in, const uint8_t *mask, float scale,
                          float *out, long long n);
B200_API int b200_dropout_host(b200_ctx *ctx, const float *in, const uint8_t *mask, float scale,
                               float *out, long long n);

/*
 * lrn_layer::forward_propagation, norm_region::across_channels
 * (tiny_dnn/layers/lrn_layer.h:82-143): out = in * (1 + alpha/size * S)^-beta
 * with S the running sum of squares over a window of `size` channels, updated
 * in the reference's order.  The reference has no backward pass for this
 * layer (:96-104 throws "not implemented") and no within-channel form
 * (:145-149 throws), so neither exists here.
 */
B200_API int b200_lrn_fwd(b200_ctx *ctx, const float *in, float *out, int channels, int area, int size,
                          float alpha, float beta, int batch);
B200_API int b200_lrn_fwd_host(b200_ctx *ctx, const float *in, float *out, int channels, int area,
                               int size, float alpha, float beta, int batch);

/*
 * Per-sample loss gradient dE/dy: mse 2/dim*(y-t), cross_entropy
 * (y-t)/(y*(1-y)), multiclass -t/y.  Replaces mse::df / cross_entropy::df /
 * cross_entropy_multiclass::df and the mini-batch loop gradient<E>
 * (tiny_dnn/lossfunctions/loss_function.h:28-36,120-128,143-150,190-218).
 */
B200_API int b200_loss_grad(b200_ctx *ctx, int kind, const float *y, const float *t, float *dy,
                            int dim, int batch);

/*
 * Sum over the batch of E::f(y_n, t_n) (loss_function.h:17-26,107-118,132-141),
 * written to one device float.  The reference exposes it as network::get_loss.
 */
B200_API int b200_loss_value(b200_ctx *ctx, int kind, const float *y, const float *t,
                             float *loss_sum, int dim, int batch);

/* ------------------------------------------------------------------------- */
/* Gradient merge + optimizer  (a10-a11)                                       */
/* ------------------------------------------------------------------------- */

/* every optimizer of tiny_dnn/optimizers/optimizer.h: adagrad :57-71, adam :103-137,
 * momentum :201-218, RMSprop :79-95, adamax :145-175, gradient_descent :182-193,
 * nesterov_momentum :227-245 */
enum {
  B200_OPT_ADAGRAD = 0,
  B200_OPT_ADAM = 1,
  B200_OPT_MOMENTUM = 2,
  B200_OPT_RMSPROP = 3,
  B200_OPT_ADAMAX = 4,
  B200_OPT_GRADIENT_DESCENT = 5,
  B200_OPT_NESTEROV_MOMENTUM = 6
};

/* Public hyper-parameters of the reference optimizers. */
typedef struct b200_opt_hyper {
  float alpha;   /* learning rate (all)                                  */
  float b1, b2;  /* adam / adamax decay terms                            */
  float b1_t;    /* adam / adamax b1^t for THIS update call (per tensor) */
  float b2_t;    /* adam b2^t for THIS update call                       */
  float mu;      /* momentum, nesterov_momentum; RMSprop's decay term    */
  float lambda;  /* weight decay of the three SGD forms                  */
  float eps;     /* 1e-8 in the reference (private member)               */
} b200_opt_hyper;

/*
 * dst[i] = sum_{r<rows} grads[r*len + i], summed in row order like
 * edge::merge_grads (tiny_dnn/node.h:89-103).  rows may be 1.
 */
B200_API int b200_merge_grads(b200_ctx *ctx, const float *grads, int rows, size_t len,
                              float *dst);

/*
 * One optimizer::update call on one parameter tensor
 * (adagrad optimizer.h:60-66, adam :112-127, momentum :205-213, RMSprop :82-89,
 * adamax :153-166, gradient_descent :185-188, nesterov_momentum :233-240).  state0 is g
 * (adagrad, RMSprop), mt (adam, adamax) or dWprev (momentum, nesterov_momentum); state1 is
 * vt (adam) or ut (adamax); gradient_descent keeps none.  The caller advances b1_t / b2_t
 * after each call as adam::update and adamax::update do (:125-126, :165).  adamax's step
 * size alpha / (1.0 - b1_t) is formed in double precision, as the reference's literal does.
 */
B200_API int b200_opt_update(b200_ctx *ctx, int kind, const b200_opt_hyper *h, const float *dW,
                             float *W, float *state0, float *state1, size_t len);

/*
 * merge_grads fused with the update: dW_i = sum_r grads[r*stride + i] is formed
 * in registers and consumed by the optimizer formula; `merged` (may be NULL)
 * receives the sum.  Replaces the body of layer::update_weight for one
 * trainable edge (tiny_dnn/layers/layer.h:663-682).
 */
B200_API int b200_merge_update(b200_ctx *ctx, int kind, const b200_opt_hyper *h,
                               const float *grads, int rows, size_t stride, float *merged,
                               float *W, float *state0, float *state1, size_t len);

/* ------------------------------------------------------------------------- */
/* Quantized forward  (a12-a14)                                                */
/* ------------------------------------------------------------------------- */

/*
 * uint8 quantized convolution forward, bit-exact with
 * tiny_quantized_conv2d_kernel (tiny_dnn/core/kernels/tiny_quantized_conv2d_kernel.h:20-148)
 * run per sample by tiny_backend::conv2d_q (tiny_dnn/core/backend_tiny.h:97-112):
 * per-sample input range, filter range taken from the element subset the
 * reference scans (:40-55), int32 accumulate, shrink-range requantize
 * (tiny_quantization_kernel.h:145-186,230-254), dequantize to float.
 * `in` has in_padded geometry when pad_same (the layer pads first).
 */
B200_API int b200_qconv2d_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in,
                              const float *W, const float *bias, float *out, int batch);

/*
 * uint8 quantized fully-connected forward, bit-exact with
 * tiny_quantized_fully_connected_kernel
 * (tiny_dnn/core/kernels/tiny_quantized_fully_connected_kernel.h:22-128) run per
 * sample as tiny_backend::fully_q would (backend_tiny.h:300-319).
 */
B200_API int b200_qfc_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in,
                          const float *W, const float *bias, float *out, int batch);

/*
 * The forms for quantized layers chained without dequantizing in between
 * (tiny_backend::conv2d_eq / fully_eq, tiny_dnn/core/backend_tiny.h:115-135,321-345, over
 * the nine- / eleven-argument overloads of tiny_quantized_conv2d_kernel
 * (tiny_quantized_conv2d_kernel.h:353-466) and tiny_quantized_fully_connected_kernel
 * (tiny_quantized_fully_connected_kernel.h:269-370)): `in`, `W` and `bias` hold uint8 values
 * in floats, `in_r` (2 floats per sample), `W_r`, `b_r` (2 floats each) their ranges; `out`
 * receives the requantized uint8 values in floats and `out_r` (2 floats per sample) their
 * range.  Bit for bit with the reference kernels, including the convolution's bias term
 * formed in float.  The convolution input rows are the PADDED rows, as for b200_qconv2d_fwd.
 * In the reference nothing constructs a layer with the six inputs that select these forms,
 * so only a caller of the backend interface reaches them.
 */
B200_API int b200_qconv2d_eq_fwd(b200_ctx *ctx, const b200_conv_desc *d, const float *in,
                                 const float *W, const float *bias, const float *in_r,
                                 const float *W_r, const float *b_r, float *out, float *out_r,
                                 int batch);
B200_API int b200_qfc_eq_fwd(b200_ctx *ctx, int in_size, int out_size, const float *in,
                             const float *W, const float *bias, const float *in_r,
                             const float *W_r, const float *b_r, float *out, float *out_r,
                             int batch);
B200_API int b200_qconv2d_eq_fwd_host(b200_ctx *ctx, const b200_conv_desc *d, const float *in,
                                      const float *W, const float *bias, const float *in_r,
                                      const float *W_r, const float *b_r, float *out,
                                      float *out_r, int batch);
B200_API int b200_qfc_eq_fwd_host(b200_ctx *ctx, int in_size, int out_size, const float *in,
                                  const float *W, const float *bias, const float *in_r,
                                  const float *W_r, const float *b_r, float *out, float *out_r,
                                  int batch);

B200_API int b200_qconv2d_fwd_host(b200_ctx *ctx, const b200_conv_desc *d, const float *in,
                                   const float *W, const float *bias, float *out, int batch);
B200_API int b200_qfc_fwd_host(b200_ctx *ctx, int in_size, int out_size, const float *in,
                               const float *W, const float *bias, float *out, int batch);

/* ------------------------------------------------------------------------- */
/* Device-resident training step (driver of a1-a11)                            */
/* ------------------------------------------------------------------------- */

enum {
  B200_LAYER_CONV = 1,
  B200_LAYER_FC = 2,
  B200_LAYER_MAXPOOL = 3,
  B200_LAYER_AVGPOOL = 4,
  B200_LAYER_RELU = 5,
  B200_LAYER_TANH = 6,
  B200_LAYER_SOFTMAX = 7,
  B200_LAYER_SIGMOID = 8,
  B200_LAYER_LEAKY_RELU = 9, /* act_param = epsilon */
  B200_LAYER_ELU = 10,       /* act_param = alpha   */
  B200_LAYER_BATCHNORM = 11  /* bn_* fields         */
};

/* One layer of a network<sequential> (tiny_dnn/nodes.h:268-360). */
typedef struct b200_layer_spec {
  int32_t kind;
  b200_conv_desc conv;   /* B200_LAYER_CONV                                   */
  b200_pool_desc pool;   /* B200_LAYER_MAXPOOL / B200_LAYER_AVGPOOL           */
  int32_t fc_in, fc_out, fc_has_bias; /* B200_LAYER_FC                        */
  float act_param;       /* B200_LAYER_LEAKY_RELU / B200_LAYER_ELU            */
  /* B200_LAYER_BATCHNORM: batch_normalization_layer(in_spatial_size, in_channels, epsilon,
   * momentum) (tiny_dnn/layers/batch_normalization_layer.h:59-72) */
  int32_t bn_channels, bn_spatial;
  float bn_eps, bn_momentum;
} b200_layer_spec;

typedef struct b200_net b200_net;

/*
 * Build a device-resident twin of a sequential network.  Parameters live in one
 * flat buffer in network order (layer order; W before b: layer.h:663-678), and
 * so do the batch-summed gradients (the all-reduce bucket) and optimizer state.
 */
B200_API int b200_net_create(b200_ctx *ctx, const b200_layer_spec *layers, int n_layers,
                             int max_batch, b200_net **out);
B200_API int b200_net_destroy(b200_net *net);

B200_API size_t b200_net_param_count(const b200_net *net);
B200_API int b200_net_tensor_count(const b200_net *net);
/* offset/length of trainable tensor `i` inside the flat parameter buffer. */
B200_API int b200_net_tensor_info(const b200_net *net, int i, size_t *offset, size_t *len);
B200_API int b200_net_in_dim(const b200_net *net);
B200_API int b200_net_out_dim(const b200_net *net);

/* HOST <-> device copies of the flat parameter buffer. */
B200_API int b200_net_set_params(b200_net *net, const float *host_params);
B200_API int b200_net_get_params(b200_net *net, float *host_params);
/* HOST copy of the flat batch-summed gradient bucket of the last backward. */
B200_API int b200_net_get_grads(b200_net *net, float *host_grads);

/* Device pointers for callers that own the collective (NCCL all-reduce). */
B200_API float *b200_net_params_ptr(b200_net *net);
B200_API float *b200_net_grads_ptr(b200_net *net);
B200_API float *b200_net_output_ptr(b200_net *net);
/* Device pointer to the output of layer `i` / its gradient dE/d out, [batch][dim] CHW rows
 * (tests).  A layer whose activation was folded into its producer has no output of its own
 * (NULL).  The gradient of a convolution whose backward kernels all read the pixel-major copy
 * is kept in that form only, and this buffer is then not written; set the environment variable
 * B200_NET_KEEP_GRADS=1 before b200_net_create to have every gradient here as well. */
B200_API float *b200_net_layer_out_ptr(b200_net *net, int i);
B200_API float *b200_net_layer_grad_ptr(b200_net *net, int i);

/*
 * network::set_netphase (tiny_dnn/network.h:438-442): train != 0 is net_phase::train (batch
 * normalization layers use the mini-batch's moments and, after every update, move their averages
 * toward them), 0 is net_phase::test (they use the moving averages).  A new net is in the train
 * phase, as a new layer object is.  Only batch normalization layers look at it.
 */
B200_API int b200_net_set_phase(b200_net *net, int train);

/*
 * The gradient with respect to the network's INPUT (prev_delta of the first layer).  The
 * reference's backward pass computes it for every layer (layers/layer.h back_propagation) and
 * network::fit never reads it; a new net computes it as well (b200_net_layer_grad_ptr(net, -1)).
 * on = 0 drops the first layer's dX kernel from the following steps -- the weights come out bit
 * for bit the same -- and rebuilds the captured graphs.
 */
B200_API int b200_net_set_input_grad(b200_net *net, int on);
/*
 * The moving averages of batch normalization layer `layer` (index into the layer list):
 * mean_ and variance_ of the reference object, `channels` floats each, host memory.
 * set != 0 writes them to the device, 0 reads them back.
 */
B200_API int b200_net_bn_stats(b200_net *net, int layer, float *mean, float *variance, int set);

/* network::fprop (tiny_dnn/network.h:911-926 -> nodes.h:288-303). */
B200_API int b200_net_forward(b200_net *net, const float *x, int batch);
/*
 * gradient<E>(out, t) then network::bprop (loss_function.h:190-218,
 * nodes.h:276-286); leaves the batch-summed gradients in the bucket.
 */
B200_API int b200_net_backward(b200_net *net, const float *t, int loss_kind);

/* Reset optimizer state (optimizer::reset, optimizer.h:36-38 -- b1_t/b2_t are
 * NOT reset by the reference; `reset_powers` != 0 restarts them for a new
 * optimizer object). */
B200_API int b200_net_opt_reset(b200_net *net, int reset_powers);

/*
 * nodes::update_weights (nodes.h:103-107): one optimizer update per trainable
 * tensor in network order, Adam's powers advancing once per TENSOR
 * (optimizer.h:125-126).  `h->b1_t/b2_t` are ignored; the net keeps its own.
 */
B200_API int b200_net_update(b200_net *net, int opt_kind, const b200_opt_hyper *h);

/* forward + backward + update in one call; device x/t.  Uses a captured CUDA
 * graph after the first call for a given (x, t, batch, loss, optimizer). */
B200_API int b200_net_train_step(b200_net *net, const float *x, const float *t, int batch,
                                 int loss_kind, int opt_kind, const b200_opt_hyper *h);

/*
 * forward + backward only (captured like the whole step): what a data-parallel
 * rank runs before the gradient bucket is all-reduced and b200_net_update is
 * called.
 */
B200_API int b200_net_forward_backward(b200_net *net, const float *x, const float *t, int batch,
                                       int loss_kind);

/*
 * Data-parallel replicas (one process per GPU, the mini-batch sharded over them): the
 * device form of edge::merge_grads (network.h:880-906) across GPUs.  Every rank provides
 * a zero-filled buffer of b200_net_peer_reduce_bytes() bytes that all ranks have mapped
 * (peer / symmetric memory) and passes the `world` base addresses, as mapped in its own
 * process, to b200_net_peer_reduce_init.  From then on b200_net_train_step sums the
 * gradient bucket over the ranks inside its captured graph: the gradients of every layer
 * but the first one with parameters are pushed into every rank's buffer over NVLink from a
 * side branch as soon as the backward pass has produced them, and summed there (bounded wait
 * for the other ranks' pushes, the `world` copies added in rank order); after the backward
 * pass one kernel per GPU sends the first layer's gradients -- as 8-byte words {value, step
 * number} that need neither fence nor counter when there are at most 65 536 of them -- waits
 * (bounded) for the other ranks' and adds them in rank order, so the replicas stay
 * bit-identical.  No 1/world
 * factor.  Every rank must call the step the same number of times.
 *
 * `timeout_ms` bounds every wait for another rank (0 = 10 s).  A wait that runs out sets the
 * context's error word (b200_ctx_sync then returns an error naming code 7) and the update
 * of that step changes nothing on this rank; the other ranks may have finished the step, so
 * the replicas differ from then on and the buffers' arrival counters are out of step: a
 * timeout is terminal for this group of ranks (rebuild the nets, reload a checkpoint).
 *
 * b200_net_peer_reduce is the reduction alone (after b200_net_forward_backward, before
 * b200_net_update).  b200_net_peer_push / b200_net_peer_sum are its two halves -- push the
 * whole bucket to every rank without waiting; wait for every rank's push and sum -- for a
 * caller that runs several ranks of one GPU one after the other (tests): kernels that wait
 * for one another must never be separate launches on one GPU, so there every rank pushes
 * before any rank sums.
 */
B200_API size_t b200_net_peer_reduce_bytes(b200_net *net, int world);
B200_API int b200_net_peer_reduce_init(b200_net *net, int rank, int world,
                                       const unsigned long long *buffers, int timeout_ms);
B200_API int b200_net_peer_reduce(b200_net *net);
B200_API int b200_net_peer_push(b200_net *net);
B200_API int b200_net_peer_sum(b200_net *net);

/*
 * The rendezvous of those exchange buffers between the processes of one box, for a host
 * that has no framework to do it (a multi-process C++ launcher around network::fit):
 * b200_peer_buffer_create allocates `bytes` of zero-filled device memory on the context's
 * GPU and writes an opaque B200_PEER_HANDLE_BYTES-byte handle that the caller sends to the
 * other processes by any means (a pipe, a file, MPI, a torch.distributed object gather);
 * b200_peer_buffer_open maps the buffer behind another process's handle into this process
 * (peer access between the two GPUs is enabled on first use) and returns its address here.
 * The addresses -- the own buffer at index `rank` -- are what b200_net_peer_reduce_init
 * takes.  b200_peer_buffer_close unmaps an opened buffer; b200_peer_buffer_destroy frees a
 * created one, after every other process has closed it.  A handle is only meaningful on
 * the box and during the life of the process that created it.
 */
#define B200_PEER_HANDLE_BYTES 64
B200_API int b200_peer_buffer_create(b200_ctx *ctx, size_t bytes, void **dev,
                                     unsigned char handle[B200_PEER_HANDLE_BYTES]);
B200_API int b200_peer_buffer_open(b200_ctx *ctx, const unsigned char handle[B200_PEER_HANDLE_BYTES],
                                   void **dev);
B200_API int b200_peer_buffer_close(b200_ctx *ctx, void *dev);
B200_API int b200_peer_buffer_destroy(b200_ctx *ctx, void *dev);

/*
 * The same step from HOST buffers (what network::train_onebatch does,
 * network.h:911-926): x/t are copied to the device, the step runs, and the
 * network output of the forward pass (batch x out_dim floats) is copied back
 * to `out_host` when it is not NULL.  Pinned host memory makes the copies
 * asynchronous; the call returns after the output has arrived.
 */
B200_API int b200_net_train_step_host(b200_net *net, const float *x_host, const float *t_host,
                                      int batch, int loss_kind, int opt_kind,
                                      const b200_opt_hyper *h, float *out_host);

/*
 * network::fit over HOST arrays (tiny_dnn/network.h:840-879): `epochs` passes
 * over n_samples rows of x_host [n_samples][in_dim] / t_host [n_samples][out_dim]
 * in mini-batches of `batch`, one training step each.  A last mini-batch with fewer
 * samples runs as the reference runs it (network.h:883-926): the new samples replace the
 * first rows of the batch buffers and the step still covers all `batch` rows, the rest
 * being the previous step's; exactly one left-over sample is a one-sample step.  (So
 * n_samples must be at least `batch`, or 1.)  The upload of the next mini-batch runs
 * on a second stream while the current step computes (pinned host memory makes
 * that overlap real).  With `out_host` [n_samples][out_dim] not NULL the
 * forward output of every step's NEW samples is copied back to their rows (the last
 * epoch's values remain).  Returns after everything has finished.
 */
B200_API int b200_net_fit_host(b200_net *net, const float *x_host, const float *t_host,
                               long long n_samples, int batch, int epochs, int loss_kind,
                               int opt_kind, const b200_opt_hyper *h, float *out_host);

/*
 * The same, returning as soon as the steps are queued: for a host that prepares its rows in
 * runs (tiny-dnn keeps one heap vector per sample; the fit hook packs them into page-locked
 * memory while the device trains on the rows packed before) and wants the device to go from
 * one run to the next without draining.  The arrays of every queued call must stay valid and
 * unchanged, and `out_host` unread, until b200_net_fit_host_wait has returned.
 */
B200_API int b200_net_fit_host_enqueue(b200_net *net, const float *x_host, const float *t_host,
                               long long n_samples, int batch, int epochs, int loss_kind,
                               int opt_kind, const b200_opt_hyper *h, float *out_host);
B200_API int b200_net_fit_host_wait(b200_net *net);

/* ------------------------------------------------------------------------- */
/* The callers' data formats: raw dataset bytes to device batches              */
/* ------------------------------------------------------------------------- */

enum { B200_IMAGE_CIFAR10 = 0, B200_IMAGE_MNIST = 1 };

/*
 * How uint8 pixels become the floats of the first layer's input rows.  `mode` selects the
 * reference parser whose arithmetic is reproduced bit for bit:
 *   B200_IMAGE_CIFAR10  parse_cifar10 (tiny_dnn/io/cifar10_parser.h:26-86):
 *                       scale_min + (scale_max - scale_min) * c / 255
 *   B200_IMAGE_MNIST    parse_mnist_images (tiny_dnn/io/mnist_parser.h:43-68,130-157):
 *                       (c / 255) * (scale_max - scale_min) + scale_min
 * Images are planar [channels][height][width] bytes (a CIFAR-10 record without its label byte, the
 * pixels of an idx3 file); the output rows are [channels][height + 2*y_padding][width +
 * 2*x_padding] floats with the border filled with scale_min, as both parsers do.
 */
typedef struct b200_image_desc {
  int32_t mode;
  int32_t channels, height, width;
  int32_t x_padding, y_padding;
  float scale_min, scale_max;
} b200_image_desc;

/* n images of DEVICE bytes -> n DEVICE float rows. */
B200_API int b200_images_u8_to_float(b200_ctx *ctx, const b200_image_desc *d, const uint8_t *src,
                                     long long n, float *dst);
/*
 * n DEVICE class labels -> n DEVICE target rows of out_dim floats: target_min everywhere,
 * target_max at the label (nodes::label2vec, tiny_dnn/nodes.h:180-189; the two values are the
 * output range of the network's last layer, nodes.h:147-156).
 */
B200_API int b200_labels_to_targets(b200_ctx *ctx, const uint8_t *labels, long long n, int out_dim,
                                    float target_min, float target_max, float *dst);
/*
 * network::train (network.h:268-307) from the dataset's own bytes: like b200_net_fit_host, but
 * every mini-batch is uploaded as uint8 images + uint8 labels (HOST memory, page-locked for
 * overlap) and converted on the device by the two functions above before its step.  The net's
 * input size must equal the padded image size and its output size must exceed every label.
 */
B200_API int b200_net_fit_u8_host(b200_net *net, const b200_image_desc *d, const uint8_t *images_host,
                                  const uint8_t *labels_host, long long n_samples, int batch, int epochs,
                                  float target_min, float target_max, int loss_kind, int opt_kind,
                                  const b200_opt_hyper *h, float *out_host);

/* Adam powers currently held by the net: what the next update of the FIRST tensor will use,
 * i.e. the b1_t / b2_t members of the reference's adam object at that moment (optimizer.h:129-133). */
B200_API int b200_net_adam_powers(const b200_net *net, float *b1_t, float *b2_t);

/*
 * Hand-off of the optimizer between the host objects of the reference and the device
 * (network::save / load move the weights, network.h:676-728; the optimizer's state lives in
 * stateful_optimizer::E_, optimizer.h:34-48, and in adam's public b1_t / b2_t).
 * State buffer 0 is adagrad's g, adam's mt, momentum's dWprev; buffer 1 is adam's vt.  Both are
 * flat in network parameter order, like b200_net_get_params.  b200_net_set_adam_powers makes the
 * next step continue from an adam object whose powers currently are (b1_t, b2_t); a fresh object
 * has (b1, b2), which is also what a net starts from when this is never called.
 */
B200_API int b200_net_get_opt_state(b200_net *net, int which, float *host_state);
B200_API int b200_net_set_opt_state(b200_net *net, int which, const float *host_state);
B200_API int b200_net_set_adam_powers(b200_net *net, float b1, float b2, float b1_t, float b2_t);

/* Number of kernels this library launched on the calling process so far. */
B200_API unsigned long long b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* TINYCNN_B200_H_ */
