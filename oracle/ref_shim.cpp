// ref_shim.cpp -- extern "C" doors into the UNMODIFIED reference (tiny-dnn),
// compiled from its own headers where they lie (never copied into this
// repository) into oracle/_ref/libtinydnn_ref.so by oracle/build_oracle.py.
//
// TEST INFRASTRUCTURE ONLY: it pins oracle.c (the C restatement) against the
// real implementation, generates the golden fixtures, and serves as the timed
// CPU baseline.  Every entry point drives the reference through its own layer
// classes / free functions with engine REF_ENGINE (backend_t::internal unless
// the build says otherwise).
//
// Flat-array conventions match oracle.c (B rows back to back, reference
// layouts), so a test can call ref_X and orc_X with the same arguments.
#include <chrono>
#ifdef _OPENMP
#include <omp.h>
#endif
#include <cstring>
#include <memory>
#include <vector>

#include "tiny_dnn/tiny_dnn.h"
#include "tinycnn_b200.h"

using namespace tiny_dnn;

#define REF_API extern "C" __attribute__((visibility("default")))

// Engine every layer is constructed with.  The default build is the parity
// target, backend_t::internal; oracle/build_oracle.py compiles this file a
// second time with -DREF_ENGINE=core::backend_t::avx (and the reference's AVX
// macros) into a separate library that is only ever TIMED, as the reference's
// fastest shipped CPU path for 5x5 convolutions (conv2d_op_avx.h:451-468).
#ifndef REF_ENGINE
#define REF_ENGINE core::backend_t::internal
#endif

namespace {

tensor_t to_tensor(const float *p, size_t rows, size_t len) {
  tensor_t t(rows, vec_t(len));
  if (p)
    for (size_t r = 0; r < rows; ++r) std::copy(p + r * len, p + (r + 1) * len, t[r].begin());
  return t;
}
void from_tensor(const tensor_t &t, float *p, size_t len) {
  if (!p) return;
  for (size_t r = 0; r < t.size(); ++r) std::copy(t[r].begin(), t[r].begin() + len, p + r * len);
}

core::connection_table make_table(const b200_conv_desc *d) {
  if (!d->tbl) return core::connection_table();
  std::vector<char> tmp(d->tbl, d->tbl + (size_t)d->in_c * d->out_c);
  std::unique_ptr<bool[]> ar(new bool[tmp.size()]);
  for (size_t i = 0; i < tmp.size(); ++i) ar[i] = tmp[i] != 0;
  // rows = in channels, cols = out channels (examples/mnist/train.cpp:44-51)
  return core::connection_table(ar.get(), d->in_c, d->out_c);
}

std::unique_ptr<convolutional_layer> make_conv(const b200_conv_desc *d) {
  return std::unique_ptr<convolutional_layer>(new convolutional_layer(
    d->in_w, d->in_h, d->k_w, d->k_h, d->in_c, d->out_c, make_table(d),
    d->pad_same ? padding::same : padding::valid, d->has_bias != 0, d->stride_w, d->stride_h,
    d->dil_w, d->dil_h, REF_ENGINE));
}

}  // namespace

#define REF_STR2(x) #x
#define REF_STR(x) REF_STR2(x)
REF_API const char *ref_version() { return "tiny-dnn reference, " REF_STR(REF_ENGINE); }

REF_API int ref_openmp_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// Thread count of the OpenMP runtime inside this library.  A launcher may have
// exported OMP_NUM_THREADS=1 (torch.distributed.run does); the timed baseline
// asks for the host's cores explicitly instead of inheriting that.
REF_API int ref_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}

// ---------------------------------------------------------------- convolution
// convolutional_layer::forward_propagation with UNPADDED input rows.
REF_API int ref_conv2d_fwd(const b200_conv_desc *d, const float *in, const float *W,
                           const float *bias, float *out, int B) {
  auto l = make_conv(d);
  size_t in_len = (size_t)d->in_c * d->in_h * d->in_w;
  size_t out_len = (size_t)d->out_c * d->out_h * d->out_w;
  size_t lenW = (size_t)d->out_c * d->in_c * d->k_h * d->k_w;
  if (l->out_shape()[0].size() != out_len) return 1;
  tensor_t tin = to_tensor(in, B, in_len), tW = to_tensor(W, 1, lenW),
           tb = to_tensor(d->has_bias ? bias : nullptr, 1, d->out_c), tout(B, vec_t(out_len));
  // Conv2dOp::compute reads input(2) even when has_bias is false
  // (conv2d_op.h:29), so a bias tensor is always supplied.
  std::vector<tensor_t *> ins = {&tin, &tW, &tb};
  std::vector<tensor_t *> outs = {&tout};
  l->set_parallelize(true);
  l->forward_propagation(ins, outs);
  from_tensor(tout, out, out_len);
  return 0;
}

// forward then convolutional_layer::back_propagation.  din is unpadded;
// dW / db are per-sample rows (B x len) that START FROM ZERO.
REF_API int ref_conv2d_bwd(const b200_conv_desc *d, const float *in, const float *W,
                           const float *dout, float *din, float *dW_rows, float *db_rows, int B) {
  auto l = make_conv(d);
  size_t in_len = (size_t)d->in_c * d->in_h * d->in_w;
  size_t out_len = (size_t)d->out_c * d->out_h * d->out_w;
  size_t lenW = (size_t)d->out_c * d->in_c * d->k_h * d->k_w;
  tensor_t tin = to_tensor(in, B, in_len), tW = to_tensor(W, 1, lenW),
           tb = to_tensor(nullptr, 1, d->out_c), tout(B, vec_t(out_len));
  tensor_t gout = to_tensor(dout, B, out_len), gin(B, vec_t(in_len)), gW(B, vec_t(lenW)),
           gb(B, vec_t(d->out_c));
  // Conv2dGradOp::compute reads input_grad(2) unconditionally (conv2d_grad_op.h:29)
  std::vector<tensor_t *> ins = {&tin, &tW, &tb}, gins = {&gin, &gW, &gb};
  std::vector<tensor_t *> outs = {&tout}, gouts = {&gout};
  l->setup(false);
  l->set_sample_count(B);
  l->set_parallelize(true);
  l->forward_propagation(ins, outs);
  l->back_propagation(ins, outs, gouts, gins);
  from_tensor(gin, din, in_len);
  from_tensor(gW, dW_rows, lenW);
  if (d->has_bias) from_tensor(gb, db_rows, d->out_c);
  return 0;
}

// ---------------------------------------------------------------- fully connected
REF_API int ref_fc_fwd(int in_size, int out_size, const float *in, const float *W,
                       const float *bias, float *out, int B) {
  fully_connected_layer l(in_size, out_size, bias != nullptr, REF_ENGINE);
  tensor_t tin = to_tensor(in, B, in_size), tW = to_tensor(W, 1, (size_t)in_size * out_size),
           tb = to_tensor(bias, 1, out_size), tout(B, vec_t(out_size));
  std::vector<tensor_t *> ins = {&tin, &tW};
  if (bias) ins.push_back(&tb);
  std::vector<tensor_t *> outs = {&tout};
  l.set_parallelize(true);
  l.forward_propagation(ins, outs);
  from_tensor(tout, out, out_size);
  return 0;
}

REF_API int ref_fc_bwd(int in_size, int out_size, int has_bias, const float *in, const float *W,
                       const float *dout, float *din, float *dW_rows, float *db_rows, int B) {
  fully_connected_layer l(in_size, out_size, has_bias != 0, REF_ENGINE);
  size_t lenW = (size_t)in_size * out_size;
  tensor_t tin = to_tensor(in, B, in_size), tW = to_tensor(W, 1, lenW),
           tb = to_tensor(nullptr, 1, out_size), tout(B, vec_t(out_size));
  tensor_t gout = to_tensor(dout, B, out_size), gin(B, vec_t(in_size)), gW(B, vec_t(lenW)),
           gb(B, vec_t(out_size));
  std::vector<tensor_t *> ins = {&tin, &tW}, gins = {&gin, &gW};
  if (has_bias) {
    ins.push_back(&tb);
    gins.push_back(&gb);
  }
  std::vector<tensor_t *> outs = {&tout}, gouts = {&gout};
  l.set_parallelize(true);
  l.back_propagation(ins, outs, gouts, gins);
  from_tensor(gin, din, in_size);
  from_tensor(gW, dW_rows, lenW);
  if (has_bias) from_tensor(gb, db_rows, out_size);
  return 0;
}

// ---------------------------------------------------------------- pooling
namespace {
std::unique_ptr<max_pooling_layer> make_maxpool(const b200_pool_desc *d, int ceil_mode,
                                                int pad_same) {
  return std::unique_ptr<max_pooling_layer>(new max_pooling_layer(
    d->in_w, d->in_h, d->in_c, d->pool_w, d->pool_h, d->stride_w, d->stride_h, ceil_mode != 0,
    pad_same ? padding::same : padding::valid, REF_ENGINE));
}
}  // namespace

REF_API int ref_maxpool_fwd_bwd(const b200_pool_desc *d, int ceil_mode, int pad_same,
                                const float *in, float *out, const float *dout, float *din,
                                int B) {
  auto l = make_maxpool(d, ceil_mode, pad_same);
  size_t in_len = (size_t)d->in_c * d->in_h * d->in_w;
  size_t out_len = l->out_shape()[0].size();
  if (out_len != (size_t)d->in_c * d->out_h * d->out_w) return 1;
  tensor_t tin = to_tensor(in, B, in_len), tout(B, vec_t(out_len));
  std::vector<tensor_t *> ins = {&tin}, outs = {&tout};
  l->setup(false);
  l->set_sample_count(B);
  l->set_parallelize(true);
  l->forward_propagation(ins, outs);
  from_tensor(tout, out, out_len);
  if (dout && din) {
    tensor_t gout = to_tensor(dout, B, out_len), gin(B, vec_t(in_len));
    std::vector<tensor_t *> gouts = {&gout}, gins = {&gin};
    l->back_propagation(ins, outs, gouts, gins);
    from_tensor(gin, din, in_len);
  }
  return 0;
}

REF_API int ref_avgpool_fwd_bwd(const b200_pool_desc *d, const float *in, const float *W,
                                const float *bias, float *out, const float *dout, float *din,
                                float *dW_rows, float *db_rows, int B) {
  average_pooling_layer l(d->in_w, d->in_h, d->in_c, d->pool_w, d->pool_h, d->stride_w,
                          d->stride_h, false, padding::valid);
  size_t in_len = (size_t)d->in_c * d->in_h * d->in_w;
  size_t out_len = l.out_shape()[0].size();
  size_t wlen = (size_t)d->pool_w * d->pool_h * d->in_c;
  if (out_len != (size_t)d->in_c * d->out_h * d->out_w) return 1;
  if (l.in_shape()[1].size() != wlen) return 2;
  tensor_t tin = to_tensor(in, B, in_len), tW = to_tensor(W, 1, wlen),
           tb = to_tensor(bias, 1, d->in_c), tout(B, vec_t(out_len));
  std::vector<tensor_t *> ins = {&tin, &tW, &tb}, outs = {&tout};
  l.set_parallelize(true);
  l.forward_propagation(ins, outs);
  from_tensor(tout, out, out_len);
  if (dout && din) {
    tensor_t gout = to_tensor(dout, B, out_len), gin(B, vec_t(in_len)), gW(B, vec_t(wlen)),
             gb(B, vec_t(d->in_c));
    std::vector<tensor_t *> gouts = {&gout}, gins = {&gin, &gW, &gb};
    l.back_propagation(ins, outs, gouts, gins);
    from_tensor(gin, din, in_len);
    from_tensor(gW, dW_rows, wlen);
    from_tensor(gb, db_rows, d->in_c);
  }
  return 0;
}

// ---------------------------------------------------------------- activations / loss
namespace {
std::unique_ptr<activation_layer> make_act(int kind, size_t dim, float param) {
  if (kind == B200_ACT_RELU) return std::unique_ptr<activation_layer>(new relu_layer(dim));
  if (kind == B200_ACT_TANH) return std::unique_ptr<activation_layer>(new tanh_layer(dim));
  if (kind == B200_ACT_SIGMOID) return std::unique_ptr<activation_layer>(new sigmoid_layer(dim));
  if (kind == B200_ACT_LEAKY_RELU) return std::unique_ptr<activation_layer>(new leaky_relu_layer(dim, param));
  if (kind == B200_ACT_ELU) return std::unique_ptr<activation_layer>(new elu_layer(dim, param));
  return std::unique_ptr<activation_layer>(new softmax_layer(dim));
}
}  // namespace

REF_API int ref_act_param_fwd_bwd(int kind, float param, const float *x, float *y, const float *dy, float *dx,
                                  int dim, int B) {
  auto l = make_act(kind, dim, param);
  tensor_t tx = to_tensor(x, B, dim), ty(B, vec_t(dim));
  std::vector<tensor_t *> ins = {&tx}, outs = {&ty};
  l->forward_propagation(ins, outs);
  from_tensor(ty, y, dim);
  if (dy && dx) {
    tensor_t gy = to_tensor(dy, B, dim), gx(B, vec_t(dim));
    std::vector<tensor_t *> gouts = {&gy}, gins = {&gx};
    l->back_propagation(ins, outs, gouts, gins);
    from_tensor(gx, dx, dim);
  }
  return 0;
}

// batch_normalization_layer forward (train != 0: this batch's moments come back in mean / variance;
// else they are the layer's moving averages) and backward; stddev_ is private, so it is returned as
// sqrt(variance + eps) the way calc_stddev computes it
REF_API int ref_batchnorm_fwd_bwd(int C, int S, float eps, const float *x, float *mean, float *variance,
                                  float *stddev, float *y, const float *dy, float *dx, int B, int train) {
  batch_normalization_layer l(S, C, eps, float_t(0.999), train ? net_phase::train : net_phase::test);
  if (!train) {
    l.set_mean(vec_t(mean, mean + C));
    l.set_variance(vec_t(variance, variance + C));
  } else {
    l.update_immidiately(true);  // mean_ / variance_ = this batch's moments, readable through save()
  }
  tensor_t tx = to_tensor(x, B, (size_t)C * S), ty(B, vec_t((size_t)C * S));
  std::vector<tensor_t *> ins = {&tx}, outs = {&ty};
  l.forward_propagation(ins, outs);
  from_tensor(ty, y, (size_t)C * S);
  if (train) {
    std::ostringstream os;
    l.save(os, 9);
    std::istringstream is(os.str());
    for (int j = 0; j < C; ++j) is >> mean[j];
    for (int j = 0; j < C; ++j) is >> variance[j];
  }
  for (int j = 0; j < C; ++j) stddev[j] = std::sqrt(variance[j] + eps);
  if (dy && dx) {
    tensor_t gy = to_tensor(dy, B, (size_t)C * S), gx(B, vec_t((size_t)C * S));
    std::vector<tensor_t *> gouts = {&gy}, gins = {&gx};
    l.back_propagation(ins, outs, gouts, gins);
    from_tensor(gx, dx, (size_t)C * S);
  }
  return 0;
}

// lrn_layer forward, across channels
REF_API int ref_lrn_fwd(const float *in, float *out, int C, int w, int h, int size, float alpha, float beta, int B) {
  lrn_layer l(w, h, size, C, alpha, beta, norm_region::across_channels);
  tensor_t tx = to_tensor(in, B, (size_t)C * w * h), ty(B, vec_t((size_t)C * w * h));
  std::vector<tensor_t *> ins = {&tx}, outs = {&ty};
  l.forward_propagation(ins, outs);
  from_tensor(ty, out, (size_t)C * w * h);
  return 0;
}

// dropout_layer forward in the train phase: the mask it drew comes back with the output; then its
// backward pass on dy
REF_API int ref_dropout_fwd_bwd(int dim, float rate, const float *in, float *out, uint8_t *mask, const float *dy,
                                float *dx, int B) {
  dropout_layer l(dim, rate, net_phase::train);
  tensor_t tx = to_tensor(in, B, dim), ty(B, vec_t(dim));
  std::vector<tensor_t *> ins = {&tx}, outs = {&ty};
  l.forward_propagation(ins, outs);
  from_tensor(ty, out, dim);
  for (int n = 0; n < B; ++n) {
    const std::vector<uint8_t> &m = l.get_mask(n);
    std::copy(m.begin(), m.end(), mask + (size_t)n * dim);
  }
  tensor_t gy = to_tensor(dy, B, dim), gx(B, vec_t(dim));
  std::vector<tensor_t *> gouts = {&gy}, gins = {&gx};
  l.back_propagation(ins, outs, gouts, gins);
  from_tensor(gx, dx, dim);
  return 0;
}

// the layers' default constructor arguments
REF_API int ref_act_fwd_bwd(int kind, const float *x, float *y, const float *dy, float *dx, int dim, int B) {
  return ref_act_param_fwd_bwd(kind, kind == B200_ACT_LEAKY_RELU ? 0.01f : 1.f, x, y, dy, dx, dim, B);
}

REF_API int ref_loss_grad(int kind, const float *y, const float *t, float *dy, int dim, int B) {
  for (int n = 0; n < B; ++n) {
    vec_t vy(y + (size_t)n * dim, y + (size_t)(n + 1) * dim);
    vec_t vt(t + (size_t)n * dim, t + (size_t)(n + 1) * dim);
    vec_t g = kind == B200_LOSS_MSE              ? gradient<mse>(vy, vt)
              : kind == B200_LOSS_CROSS_ENTROPY ? gradient<cross_entropy>(vy, vt)
                                                : gradient<cross_entropy_multiclass>(vy, vt);
    std::copy(g.begin(), g.end(), dy + (size_t)n * dim);
  }
  return 0;
}

// ---------------------------------------------------------------- merge + optimizers
// `steps` consecutive optimizer::update calls with the same gradient on one
// tensor, exactly what test/test_optimizers.h does.
REF_API int ref_opt_steps(int kind, const b200_opt_hyper *h, const float *dW, float *W, size_t len,
                          int steps) {
  vec_t vW(W, W + len), vdW(dW, dW + len);
  if (kind == B200_OPT_ADAGRAD) {
    adagrad o;
    o.alpha = h->alpha;
    for (int s = 0; s < steps; ++s) o.update(vdW, vW, false);
  } else if (kind == B200_OPT_ADAM) {
    adam o;
    o.alpha = h->alpha;
    o.b1 = h->b1;
    o.b2 = h->b2;
    o.b1_t = h->b1_t;
    o.b2_t = h->b2_t;
    for (int s = 0; s < steps; ++s) o.update(vdW, vW, false);
  } else if (kind == B200_OPT_MOMENTUM) {
    momentum o;
    o.alpha = h->alpha;
    o.mu = h->mu;
    o.lambda = h->lambda;
    for (int s = 0; s < steps; ++s) o.update(vdW, vW, false);
  } else if (kind == B200_OPT_RMSPROP) {
    RMSprop o;
    o.alpha = h->alpha;
    o.mu = h->mu;
    for (int s = 0; s < steps; ++s) o.update(vdW, vW, false);
  } else if (kind == B200_OPT_ADAMAX) {
    adamax o;
    o.alpha = h->alpha;
    o.b1 = h->b1;
    o.b2 = h->b2;
    o.b1_t = h->b1_t;
    for (int s = 0; s < steps; ++s) o.update(vdW, vW, false);
  } else if (kind == B200_OPT_GRADIENT_DESCENT) {
    gradient_descent o;
    o.alpha = h->alpha;
    o.lambda = h->lambda;
    for (int s = 0; s < steps; ++s) o.update(vdW, vW, false);
  } else if (kind == B200_OPT_NESTEROV_MOMENTUM) {
    nesterov_momentum o;
    o.alpha = h->alpha;
    o.mu = h->mu;
    o.lambda = h->lambda;
    for (int s = 0; s < steps; ++s) o.update(vdW, vW, false);
  } else {
    return 1;
  }
  std::copy(vW.begin(), vW.end(), W);
  return 0;
}

// ---------------------------------------------------------------- quantization helpers
REF_API int64_t ref_f2q_unclamped(int bits, float input, float mn, float mx) {
  return bits == 8 ? core::kernels::float_to_quantized_unclamped<uint8_t>(input, mn, mx)
                   : core::kernels::float_to_quantized_unclamped<int32_t>(input, mn, mx);
}
REF_API int64_t ref_f2q(int bits, float input, float mn, float mx) {
  return bits == 8 ? (int64_t)core::kernels::float_to_quantized<uint8_t>(input, mn, mx)
                   : (int64_t)core::kernels::float_to_quantized<int32_t>(input, mn, mx);
}
REF_API float ref_q2f(int bits, int64_t q, float mn, float mx) {
  return bits == 8 ? core::kernels::quantized_to_float<uint8_t>((uint8_t)q, mn, mx)
                   : core::kernels::quantized_to_float<int32_t>((int32_t)q, mn, mx);
}
REF_API void ref_requantize_many_i32_u8(const int32_t *input, size_t count, float min_in,
                                        float max_in, float min_out, float max_out,
                                        uint8_t *output) {
  std::vector<int32_t> tmp(input, input + count);
  core::kernels::requantize_many_in_new_range<int32_t, uint8_t>(tmp.data(), count, min_in, max_in,
                                                                min_out, max_out, output);
}
REF_API void ref_quantize_down_and_shrink_range(const int32_t *input, size_t count, float min_in,
                                                float max_in, float *min_new, float *max_new,
                                                uint8_t *output) {
  std::vector<int32_t> tmp(input, input + count);
  std::vector<uint8_t> out(count);
  float_t mn, mx;
  core::kernels::quantize_down_and_shrink_range<int32_t, uint8_t>(tmp, min_in, max_in, &mn, &mx,
                                                                  &out);
  *min_new = mn;
  *max_new = mx;
  std::copy(out.begin(), out.end(), output);
}

// quantized_convolutional_layer::forward_propagation, UNPADDED input rows.
REF_API int ref_qconv2d_fwd(const b200_conv_desc *d, const float *in, const float *W,
                            const float *bias, float *out, int B) {
  quantized_convolutional_layer l(d->in_w, d->in_h, d->k_w, d->k_h, d->in_c, d->out_c,
                                  d->pad_same ? padding::same : padding::valid, d->has_bias != 0,
                                  d->stride_w, d->stride_h, REF_ENGINE);
  size_t in_len = (size_t)d->in_c * d->in_h * d->in_w;
  size_t out_len = l.out_shape()[0].size();
  if (out_len != (size_t)d->out_c * d->out_h * d->out_w) return 1;
  size_t lenW = (size_t)d->out_c * d->in_c * d->k_h * d->k_w;
  tensor_t tin = to_tensor(in, B, in_len), tW = to_tensor(W, 1, lenW),
           tb = to_tensor(d->has_bias ? bias : nullptr, 1, d->out_c), tout(B, vec_t(out_len));
  std::vector<tensor_t *> ins = {&tin, &tW, &tb}, outs = {&tout};
  l.set_parallelize(true);
  l.forward_propagation(ins, outs);
  from_tensor(tout, out, out_len);
  return 0;
}

// tiny_quantized_conv2d_kernel, the nine-argument overload for chained quantized layers
// (tiny_quantized_conv2d_kernel.h:353-466), once per sample as tiny_backend::conv2d_eq calls it
// (backend_tiny.h:115-135).  `in`: PADDED rows of uint8 values held in floats.
REF_API int ref_qconv2d_eq_fwd(const b200_conv_desc *d, const float *in, const float *W, const float *bias,
                               const float *in_r, const float *W_r, const float *b_r, float *out, float *out_r,
                               int B) {
  core::conv_params p;
  p.in = shape3d(d->in_w, d->in_h, d->in_c);
  p.in_padded = shape3d(d->inp_w, d->inp_h, d->in_c);
  p.out = shape3d(d->out_w, d->out_h, d->out_c);
  p.weight = shape3d(d->k_w, d->k_h, (size_t)d->in_c * d->out_c);
  p.has_bias = d->has_bias != 0;
  p.pad_type = d->pad_same ? padding::same : padding::valid;
  p.w_stride = d->stride_w;
  p.h_stride = d->stride_h;
  p.w_dilation = p.h_dilation = 1;
  p.tbl = make_table(d);
  const size_t in_len = p.in_padded.size(), out_len = p.out.size(), lenW = p.weight.size();
  vec_t vW(W, W + lenW), vb(d->out_c, 0.f), vWr(W_r, W_r + 2), vbr(b_r, b_r + 2);
  if (d->has_bias) vb.assign(bias, bias + d->out_c);
  for (int n = 0; n < B; ++n) {
    vec_t vin(in + (size_t)n * in_len, in + (size_t)(n + 1) * in_len), vinr(in_r + 2 * n, in_r + 2 * n + 2);
    vec_t va(out_len, 0.f), var(2, 0.f);
    core::kernels::tiny_quantized_conv2d_kernel(p, vin, vW, vb, vinr, vWr, vbr, va, var, true);
    std::copy(va.begin(), va.end(), out + (size_t)n * out_len);
    out_r[2 * n] = var[0];
    out_r[2 * n + 1] = var[1];
  }
  return 0;
}

// ---------------------------------------------------------------- whole network
namespace {

struct RefNet {
  network<sequential> net;
  std::vector<b200_layer_spec> specs;
  adagrad o_adagrad;
  adam o_adam;
  momentum o_momentum;
  RMSprop o_rmsprop;
  adamax o_adamax;
  gradient_descent o_sgd;
  nesterov_momentum o_nesterov;
  size_t in_dim = 0, out_dim = 0, n_params = 0;

  // the net's persistent optimizer object of a kind, with the caller's hyper-parameters
  optimizer *opt(int kind, const b200_opt_hyper *hy) {
    switch (kind) {
      case B200_OPT_ADAGRAD: o_adagrad.alpha = hy->alpha; return &o_adagrad;
      case B200_OPT_ADAM:
        o_adam.alpha = hy->alpha;
        o_adam.b1 = hy->b1;
        o_adam.b2 = hy->b2;
        return &o_adam;
      case B200_OPT_MOMENTUM:
        o_momentum.alpha = hy->alpha;
        o_momentum.mu = hy->mu;
        o_momentum.lambda = hy->lambda;
        return &o_momentum;
      case B200_OPT_RMSPROP:
        o_rmsprop.alpha = hy->alpha;
        o_rmsprop.mu = hy->mu;
        return &o_rmsprop;
      case B200_OPT_ADAMAX:
        o_adamax.alpha = hy->alpha;
        o_adamax.b1 = hy->b1;
        o_adamax.b2 = hy->b2;
        return &o_adamax;
      case B200_OPT_GRADIENT_DESCENT:
        o_sgd.alpha = hy->alpha;
        o_sgd.lambda = hy->lambda;
        return &o_sgd;
      case B200_OPT_NESTEROV_MOMENTUM:
        o_nesterov.alpha = hy->alpha;
        o_nesterov.mu = hy->mu;
        o_nesterov.lambda = hy->lambda;
        return &o_nesterov;
    }
    return nullptr;
  }
};

template <typename Opt>
void fit_loss(RefNet *r, Opt &o, int loss_kind, const std::vector<vec_t> &in, const std::vector<vec_t> &tgt, int batch,
              int epochs) {
  auto nop = []() {};
  if (loss_kind == B200_LOSS_MSE)
    r->net.fit<mse>(o, in, tgt, batch, epochs, nop, nop);
  else if (loss_kind == B200_LOSS_CROSS_ENTROPY)
    r->net.fit<cross_entropy>(o, in, tgt, batch, epochs, nop, nop);
  else
    r->net.fit<cross_entropy_multiclass>(o, in, tgt, batch, epochs, nop, nop);
}

void add_layer(RefNet *r, const b200_layer_spec &s, size_t prev_dim) {
  switch (s.kind) {
    case B200_LAYER_CONV: {
      const b200_conv_desc *d = &s.conv;
      r->net << convolutional_layer(d->in_w, d->in_h, d->k_w, d->k_h, d->in_c, d->out_c,
                                    make_table(d), d->pad_same ? padding::same : padding::valid,
                                    d->has_bias != 0, d->stride_w, d->stride_h, d->dil_w, d->dil_h,
                                    REF_ENGINE);
      break;
    }
    case B200_LAYER_FC:
      r->net << fully_connected_layer(s.fc_in, s.fc_out, s.fc_has_bias != 0,
                                      REF_ENGINE);
      break;
    case B200_LAYER_MAXPOOL:
      r->net << max_pooling_layer(s.pool.in_w, s.pool.in_h, s.pool.in_c, s.pool.pool_w,
                                  s.pool.pool_h, s.pool.stride_w, s.pool.stride_h, false,
                                  padding::valid, REF_ENGINE);
      break;
    case B200_LAYER_AVGPOOL:
      r->net << average_pooling_layer(s.pool.in_w, s.pool.in_h, s.pool.in_c, s.pool.pool_w,
                                      s.pool.pool_h, s.pool.stride_w, s.pool.stride_h, false,
                                      padding::valid);
      break;
    case B200_LAYER_RELU: r->net << relu_layer(prev_dim); break;
    case B200_LAYER_TANH: r->net << tanh_layer(prev_dim); break;
    case B200_LAYER_SOFTMAX: r->net << softmax_layer(prev_dim); break;
    case B200_LAYER_SIGMOID: r->net << sigmoid_layer(prev_dim); break;
    case B200_LAYER_LEAKY_RELU: r->net << leaky_relu_layer(prev_dim, s.act_param); break;
    case B200_LAYER_ELU: r->net << elu_layer(prev_dim, s.act_param); break;
    case B200_LAYER_BATCHNORM:
      r->net << batch_normalization_layer(s.bn_spatial, s.bn_channels, s.bn_eps, s.bn_momentum);
      break;
    default: throw nn_error("unknown layer kind");
  }
}

size_t spec_out_dim(const b200_layer_spec &s, size_t prev) {
  switch (s.kind) {
    case B200_LAYER_CONV: return (size_t)s.conv.out_c * s.conv.out_h * s.conv.out_w;
    case B200_LAYER_FC: return s.fc_out;
    case B200_LAYER_MAXPOOL:
    case B200_LAYER_AVGPOOL: return (size_t)s.pool.in_c * s.pool.out_h * s.pool.out_w;
    default: return prev;
  }
}

}  // namespace

REF_API void *ref_net_create(const b200_layer_spec *specs, int n_layers, unsigned seed) {
  try {
    RefNet *r = new RefNet();
    r->specs.assign(specs, specs + n_layers);
    size_t prev = 0;
    for (int i = 0; i < n_layers; ++i) {
      if (i == 0) {
        const b200_layer_spec &s = specs[0];
        r->in_dim = s.kind == B200_LAYER_CONV ? (size_t)s.conv.in_c * s.conv.in_h * s.conv.in_w
                    : s.kind == B200_LAYER_FC ? (size_t)s.fc_in
                                              : (size_t)s.pool.in_c * s.pool.in_h * s.pool.in_w;
      }
      add_layer(r, specs[i], prev);
      prev = spec_out_dim(specs[i], prev);
    }
    r->out_dim = prev;
    // deterministic weights: seed, then redraw every layer in order
    set_random_seed(seed);
    r->net.init_weight();
    for (size_t i = 0; i < r->net.depth(); ++i)
      for (auto *w : r->net[i]->weights()) r->n_params += w->size();
    return r;
  } catch (const std::exception &e) {
    fprintf(stderr, "ref_net_create: %s\n", e.what());
    return nullptr;
  }
}
REF_API void ref_net_destroy(void *h) { delete static_cast<RefNet *>(h); }
REF_API size_t ref_net_param_count(void *h) { return static_cast<RefNet *>(h)->n_params; }

// flat parameters in network order (layer order; W before b)
REF_API void ref_net_get_params(void *h, float *dst) {
  RefNet *r = static_cast<RefNet *>(h);
  for (size_t i = 0; i < r->net.depth(); ++i)
    for (auto *w : r->net[i]->weights()) {
      std::copy(w->begin(), w->end(), dst);
      dst += w->size();
    }
}
REF_API void ref_net_set_params(void *h, const float *src) {
  RefNet *r = static_cast<RefNet *>(h);
  for (size_t i = 0; i < r->net.depth(); ++i)
    for (auto *w : r->net[i]->weights()) {
      std::copy(src, src + w->size(), w->begin());
      src += w->size();
    }
}

REF_API int ref_net_predict(void *h, const float *x, float *out, int B) {
  RefNet *r = static_cast<RefNet *>(h);
  try {
    for (int n = 0; n < B; ++n) {
      vec_t in(x + (size_t)n * r->in_dim, x + (size_t)(n + 1) * r->in_dim);
      vec_t o = r->net.predict(in);
      std::copy(o.begin(), o.end(), out + (size_t)n * r->out_dim);
    }
  } catch (const std::exception &e) {
    fprintf(stderr, "ref_net_predict: %s\n", e.what());
    return 1;
  }
  return 0;
}

// network::fit<Loss>(optimizer, inputs, targets, batch, 1 epoch): `steps`
// mini-batches of `batch` samples (x holds steps*batch rows).  Optimizer
// objects persist across calls (state and Adam powers carry on).  Returns the
// seconds spent inside fit().
REF_API double ref_net_fit_n(void *h, const float *x, const float *t, long long n_samples, int batch, int epochs,
                             int loss_kind, int opt_kind, const b200_opt_hyper *hy);

REF_API double ref_net_fit(void *h, const float *x, const float *t, int batch, int steps,
                           int loss_kind, int opt_kind, const b200_opt_hyper *hy) {
  return ref_net_fit_n(h, x, t, (long long)batch * steps, batch, 1, loss_kind, opt_kind, hy);
}

// moving averages of batch normalization layer `layer` (mean_ then variance_), read through the
// layer's own save() since the members are private
REF_API int ref_net_bn_stats(void *h, int layer, float *mean, float *variance) {
  RefNet *r = static_cast<RefNet *>(h);
  auto *bn = dynamic_cast<batch_normalization_layer *>(r->net[layer]);
  if (!bn) return 1;
  const size_t C = bn->in_shape()[0].depth_;
  std::ostringstream os;
  bn->save(os, 9);
  std::istringstream is(os.str());
  for (size_t j = 0; j < C; ++j) is >> mean[j];
  for (size_t j = 0; j < C; ++j) is >> variance[j];
  return 0;
}

// the general form: n_samples rows (the last mini-batch of a pass may be ragged), `epochs` passes
REF_API double ref_net_fit_n(void *h, const float *x, const float *t, long long n_samples, int batch, int epochs,
                             int loss_kind, int opt_kind, const b200_opt_hyper *hy) {
  RefNet *r = static_cast<RefNet *>(h);
  size_t N = (size_t)n_samples;
  std::vector<vec_t> in(N), tgt(N);
  for (size_t n = 0; n < N; ++n) {
    in[n].assign(x + n * r->in_dim, x + (n + 1) * r->in_dim);
    tgt[n].assign(t + n * r->out_dim, t + (n + 1) * r->out_dim);
  }
  if (!r->opt(opt_kind, hy)) return -1.0;
  auto t0 = std::chrono::steady_clock::now();
  try {
    // fit() calls optimizer.reset() (network.h:856), which clears the state
    // maps but not Adam's powers (optimizer.h:36-38)
    switch (opt_kind) {
      case B200_OPT_ADAGRAD: fit_loss(r, r->o_adagrad, loss_kind, in, tgt, batch, epochs); break;
      case B200_OPT_ADAM: fit_loss(r, r->o_adam, loss_kind, in, tgt, batch, epochs); break;
      case B200_OPT_MOMENTUM: fit_loss(r, r->o_momentum, loss_kind, in, tgt, batch, epochs); break;
      case B200_OPT_RMSPROP: fit_loss(r, r->o_rmsprop, loss_kind, in, tgt, batch, epochs); break;
      case B200_OPT_ADAMAX: fit_loss(r, r->o_adamax, loss_kind, in, tgt, batch, epochs); break;
      case B200_OPT_GRADIENT_DESCENT: fit_loss(r, r->o_sgd, loss_kind, in, tgt, batch, epochs); break;
      default: fit_loss(r, r->o_nesterov, loss_kind, in, tgt, batch, epochs); break;
    }
  } catch (const std::exception &e) {
    fprintf(stderr, "ref_net_fit: %s\n", e.what());
    return -1.0;
  }
  auto t1 = std::chrono::steady_clock::now();
  return std::chrono::duration<double>(t1 - t0).count();
}

// Batch-summed gradients of `n` samples computed `chunk` samples at a time, the
// protocol for mini-batches whose per-sample weight gradients do not fit in
// host memory (B x len(W) floats): every chunk goes through the network's own
// fprop / bprop<Loss>, its per-sample rows are merged by the reference's
// edge::merge_grads (node.h:89-103), the merged chunks are added in sample
// order, and the gradient tensors are cleared as layer::update_weight does
// (layer.h:680).  With chunk == n this is exactly what train_onebatch hands
// to the optimizer.  grads_out: flat, network order (W before b per layer);
// out_out (optional): forward outputs of all n samples.  No weight changes.
REF_API int ref_net_grads_chunked(void *h, const float *x, const float *t, int n, int chunk,
                                  int loss_kind, float *grads_out, float *out_out) {
  RefNet *r = static_cast<RefNet *>(h);
  try {
    r->net.set_netphase(net_phase::train);
    for (size_t i = 0; i < r->net.depth(); ++i) r->net[i]->set_parallelize(true);
    std::vector<vec_t> acc;
    bool first = true;
    vec_t diff;
    for (int c0 = 0; c0 < n; c0 += chunk) {
      int nb = std::min(chunk, n - c0);
      // network::fprop / bprop index their arguments [sample][channel][feature] (nodes.h:288-303)
      std::vector<tensor_t> in(nb, tensor_t(1)), tgt(nb, tensor_t(1));
      for (int s = 0; s < nb; ++s) {
        in[s][0].assign(x + (size_t)(c0 + s) * r->in_dim, x + (size_t)(c0 + s + 1) * r->in_dim);
        tgt[s][0].assign(t + (size_t)(c0 + s) * r->out_dim, t + (size_t)(c0 + s + 1) * r->out_dim);
      }
      std::vector<tensor_t> out = r->net.fprop(in);
      if (out_out)
        for (int s = 0; s < nb; ++s)
          std::copy(out[s][0].begin(), out[s][0].end(), out_out + (size_t)(c0 + s) * r->out_dim);
      if (loss_kind == B200_LOSS_MSE)
        r->net.bprop<mse>(out, tgt, std::vector<tensor_t>());
      else if (loss_kind == B200_LOSS_CROSS_ENTROPY)
        r->net.bprop<cross_entropy>(out, tgt, std::vector<tensor_t>());
      else
        r->net.bprop<cross_entropy_multiclass>(out, tgt, std::vector<tensor_t>());
      size_t k = 0;
      for (size_t i = 0; i < r->net.depth(); ++i) {
        layer *l = r->net[i];
        auto types = l->in_types();
        for (size_t j = 0; j < types.size(); ++j) {
          if (!is_trainable_weight(types[j])) continue;
          // a mini-batch smaller than an earlier one leaves stale (cleared) rows behind: harmless zeros
          l->prev()[j]->merge_grads(&diff);
          if (first) acc.push_back(diff);
          else
            for (size_t e = 0; e < diff.size(); ++e) acc[k][e] += diff[e];
          ++k;
        }
        l->clear_grads();
      }
      first = false;
    }
    for (auto &a : acc) {
      std::copy(a.begin(), a.end(), grads_out);
      grads_out += a.size();
    }
  } catch (const std::exception &e) {
    fprintf(stderr, "ref_net_grads_chunked: %s\n", e.what());
    return 1;
  }
  return 0;
}

// optimizer::update per parameter tensor in network order with a flat gradient
// (what nodes::update_weights -> layer::update_weight does after the merge).
// The optimizer objects are the net's persistent ones (state carries on).
REF_API int ref_net_apply_update(void *h, const float *grads, int opt_kind, const b200_opt_hyper *hy) {
  RefNet *r = static_cast<RefNet *>(h);
  optimizer *o = r->opt(opt_kind, hy);
  if (!o) return 1;
  for (size_t i = 0; i < r->net.depth(); ++i)
    for (auto *w : r->net[i]->weights()) {
      vec_t g(grads, grads + w->size());
      o->update(g, *w, w->size() >= 512);  // layer.h:676
      grads += w->size();
    }
  return 0;
}

// ---------------------------------------------------------------- dataset parsers
// parse_cifar10 (io/cifar10_parser.h:36-86) on a file in the CIFAR-10 binary format; returns the
// number of records, images as rows of 3 * (32 + 2*y_pad) * (32 + 2*x_pad) floats.
REF_API long long ref_parse_cifar10(const char *filename, float scale_min, float scale_max, int x_padding,
                                    int y_padding, float *images, unsigned char *labels, long long max_records) {
  try {
    std::vector<vec_t> img;
    std::vector<label_t> lab;
    parse_cifar10(filename, &img, &lab, scale_min, scale_max, x_padding, y_padding);
    long long n = std::min<long long>((long long)img.size(), max_records);
    for (long long i = 0; i < n; ++i) {
      std::copy(img[i].begin(), img[i].end(), images + (size_t)i * img[i].size());
      labels[i] = (unsigned char)lab[i];
    }
    return (long long)img.size();
  } catch (const std::exception &e) {
    fprintf(stderr, "ref_parse_cifar10: %s\n", e.what());
    return -1;
  }
}

// parse_mnist_images (io/mnist_parser.h:130-157) on an idx3-ubyte file
REF_API long long ref_parse_mnist_images(const char *filename, float scale_min, float scale_max, int x_padding,
                                         int y_padding, float *images, long long max_records) {
  try {
    std::vector<vec_t> img;
    parse_mnist_images(filename, &img, scale_min, scale_max, x_padding, y_padding);
    long long n = std::min<long long>((long long)img.size(), max_records);
    for (long long i = 0; i < n; ++i) std::copy(img[i].begin(), img[i].end(), images + (size_t)i * img[i].size());
    return (long long)img.size();
  } catch (const std::exception &e) {
    fprintf(stderr, "ref_parse_mnist_images: %s\n", e.what());
    return -1;
  }
}

// network::train's label conversion: nodes::label2vec through normalize_tensor (network.h:268-307,
// 983-1000) for the net's own target value range
REF_API int ref_net_label_targets(void *h, const unsigned char *labels, long long n, float *targets, float *range) {
  RefNet *r = static_cast<RefNet *>(h);
  // nodes::target_value_min / max (nodes.h:147-156): the output range of the last layer
  const std::pair<float_t, float_t> rg = r->net[r->net.depth() - 1]->out_value_range();
  range[0] = rg.first;
  range[1] = rg.second;
  for (long long i = 0; i < n; ++i) {  // nodes::label2vec (nodes.h:180-189)
    vec_t v(r->out_dim, rg.first);
    v[labels[i]] = rg.second;
    std::copy(v.begin(), v.end(), targets + (size_t)i * r->out_dim);
  }
  return 0;
}

REF_API void ref_net_adam_powers(void *h, float *b1_t, float *b2_t) {
  RefNet *r = static_cast<RefNet *>(h);
  *b1_t = r->o_adam.b1_t;
  *b2_t = r->o_adam.b2_t;
}

// Timed layer-level passes for the CPU baseline of single-layer workloads:
// `reps` forward (+ backward when with_bwd) passes of one convolution layer.
REF_API double ref_time_conv(const b200_conv_desc *d, const float *in, const float *W,
                             const float *bias, const float *dout, int B, int with_bwd, int reps) {
  auto l = make_conv(d);
  size_t in_len = (size_t)d->in_c * d->in_h * d->in_w;
  size_t out_len = (size_t)d->out_c * d->out_h * d->out_w;
  size_t lenW = (size_t)d->out_c * d->in_c * d->k_h * d->k_w;
  tensor_t tin = to_tensor(in, B, in_len), tW = to_tensor(W, 1, lenW),
           tb = to_tensor(d->has_bias ? bias : nullptr, 1, d->out_c), tout(B, vec_t(out_len));
  tensor_t gout = to_tensor(dout, B, out_len), gin(B, vec_t(in_len)), gW(B, vec_t(lenW)),
           gb(B, vec_t(d->out_c));
  std::vector<tensor_t *> ins = {&tin, &tW, &tb}, gins = {&gin, &gW, &gb};
  std::vector<tensor_t *> outs = {&tout}, gouts = {&gout};
  l->setup(false);
  l->set_sample_count(B);
  l->set_parallelize(true);
  auto t0 = std::chrono::steady_clock::now();
  for (int r = 0; r < reps; ++r) {
    l->forward_propagation(ins, outs);
    if (with_bwd) l->back_propagation(ins, outs, gouts, gins);
  }
  auto t1 = std::chrono::steady_clock::now();
  return std::chrono::duration<double>(t1 - t0).count();
}
