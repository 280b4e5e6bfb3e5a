// b200_glue.h -- C++14 host side of the B200 engine for tiny-dnn.
//
// Included by the patched operator dispatchers (Conv2dOp, Conv2dGradOp,
// FullyConnectedOp, FullyConnectedGradOp, MaxPoolOp, MaxPoolGradOp) that
// make_overlay.py derives from the reference headers.  It turns the
// reference's tensor_t rows (one heap vector per sample) into the contiguous
// buffers of the C ABI (include/tinycnn_b200.h) and back, and turns a non-zero
// status into nn_error, the reference's error convention
// (tiny_dnn/util/nn_error.h:19-27).  There is no CPU fallback: if the library
// cannot create a context the call throws.
#pragma once

#include <algorithm>
#include <cstdint>
#include <cstdlib>
#include <string>
#include <vector>

#include "tiny_dnn/core/params/conv_params.h"
#include "tiny_dnn/core/params/fully_params.h"
#include "tiny_dnn/core/params/maxpool_params.h"
#include "tiny_dnn/util/nn_error.h"
#include "tiny_dnn/util/util.h"
#include "tinycnn_b200.h"

namespace tiny_dnn {
namespace b200 {

inline void check(int status) {
  if (status != 0) throw nn_error(std::string("b200: ") + b200_last_error());
}

// one context per process, with its own stream, on device 0 -- or on the device the environment
// variable B200_DEVICE names (a launcher that starts one process per GPU sets it per process; the
// other GPUs must stay visible to the process for the peer mapping of data-parallel replicas)
inline b200_ctx *ctx() {
  static b200_ctx *c = [] {
    b200_ctx *p = nullptr;
    const char *dev = std::getenv("B200_DEVICE");
    check(b200_ctx_create(dev ? std::atoi(dev) : 0, nullptr, &p));
    return p;
  }();
  return c;
}

inline std::vector<float> pack(const tensor_t &t) {
  std::vector<float> flat;
  if (t.empty()) return flat;
  const size_t n = t[0].size();
  flat.resize(t.size() * n);
  for (size_t r = 0; r < t.size(); ++r) std::copy(t[r].begin(), t[r].end(), flat.begin() + r * n);
  return flat;
}

inline void unpack(const std::vector<float> &flat, tensor_t &t) {
  if (t.empty()) return;
  const size_t n = t[0].size();
  for (size_t r = 0; r < t.size(); ++r)
    std::copy(flat.begin() + r * n, flat.begin() + (r + 1) * n, t[r].begin());
}

// core::conv_params (tiny_dnn/core/params/conv_params.h:63-90) -> b200_conv_desc.
// The op kernels receive rows that the layer has already padded
// (convolutional_layer.h:283-299), hence input_is_padded = 1.
inline b200_conv_desc conv_desc(const core::conv_params &p, std::vector<uint8_t> &tbl) {
  b200_conv_desc d{};
  d.in_w = static_cast<int32_t>(p.in.width_);
  d.in_h = static_cast<int32_t>(p.in.height_);
  d.in_c = static_cast<int32_t>(p.in.depth_);
  d.inp_w = static_cast<int32_t>(p.in_padded.width_);
  d.inp_h = static_cast<int32_t>(p.in_padded.height_);
  d.out_w = static_cast<int32_t>(p.out.width_);
  d.out_h = static_cast<int32_t>(p.out.height_);
  d.out_c = static_cast<int32_t>(p.out.depth_);
  d.k_w = static_cast<int32_t>(p.weight.width_);
  d.k_h = static_cast<int32_t>(p.weight.height_);
  d.stride_w = static_cast<int32_t>(p.w_stride);
  d.stride_h = static_cast<int32_t>(p.h_stride);
  d.dil_w = static_cast<int32_t>(p.w_dilation);
  d.dil_h = static_cast<int32_t>(p.h_dilation);
  d.has_bias = p.has_bias ? 1 : 0;
  d.pad_same = p.pad_type == padding::same ? 1 : 0;
  d.input_is_padded = 1;
  if (!p.tbl.is_empty()) {  // connected_[inc*cols + o] (conv_params.h:52-54)
    tbl.assign(p.tbl.connected_.begin(), p.tbl.connected_.end());
    d.tbl = tbl.data();
  }
  return d;
}

inline b200_pool_desc pool_desc(const core::maxpool_params &p) {
  b200_pool_desc d{};
  d.in_w = static_cast<int32_t>(p.in.width_);
  d.in_h = static_cast<int32_t>(p.in.height_);
  d.in_c = static_cast<int32_t>(p.in.depth_);
  d.out_w = static_cast<int32_t>(p.out.width_);
  d.out_h = static_cast<int32_t>(p.out.height_);
  d.pool_w = static_cast<int32_t>(p.pool_size_x);
  d.pool_h = static_cast<int32_t>(p.pool_size_y);
  d.stride_w = static_cast<int32_t>(p.stride_x);
  d.stride_h = static_cast<int32_t>(p.stride_y);
  return d;
}

// Conv2dOp::compute branch: replaces kernels::conv2d_op_internal forward
// (tiny_dnn/core/kernels/conv2d_op_internal.h:13-74).
inline void conv2d_op(const tensor_t &in_data, const vec_t &W, const vec_t &bias,
                      tensor_t &out_data, const core::conv_params &params) {
  std::vector<uint8_t> tbl;
  b200_conv_desc d = conv_desc(params, tbl);
  std::vector<float> in = pack(in_data), out(out_data.size() * out_data[0].size());
  check(b200_conv2d_fwd_host(ctx(), &d, in.data(), W.data(), params.has_bias ? bias.data() : nullptr,
                             out.data(), static_cast<int>(in_data.size())));
  unpack(out, out_data);
}

// Conv2dGradOp::compute branch: replaces the backward kernels::conv2d_op_internal
// (conv2d_op_internal.h:78-181).  The reference adds one dW/db row per sample and
// sums the rows in edge::merge_grads (tiny_dnn/node.h:89-103); the device returns
// the batch sum, which is added to row 0, so the merged gradient is the same.
inline void conv2d_grad_op(const tensor_t &prev_out, const vec_t &W, tensor_t &dW, tensor_t &db,
                           tensor_t &curr_delta, tensor_t &prev_delta,
                           const core::conv_params &params) {
  std::vector<uint8_t> tbl;
  b200_conv_desc d = conv_desc(params, tbl);
  std::vector<float> x = pack(prev_out), dy = pack(curr_delta);
  std::vector<float> dx(prev_delta.size() * prev_delta[0].size());
  check(b200_conv2d_bwd_host(ctx(), &d, x.data(), W.data(), dy.data(), dx.data(), dW[0].data(),
                             params.has_bias ? db[0].data() : nullptr, /*accumulate=*/1,
                             static_cast<int>(prev_out.size())));
  unpack(dx, prev_delta);
}

// FullyConnectedOp::compute branch (fully_connected_op_internal.h:15-36)
inline void fully_connected_op(const tensor_t &in_data, const vec_t &W, const vec_t &bias,
                               tensor_t &out_data, const core::fully_params &params) {
  std::vector<float> in = pack(in_data), out(out_data.size() * params.out_size_);
  check(b200_fc_fwd_host(ctx(), static_cast<int>(params.in_size_), static_cast<int>(params.out_size_),
                         in.data(), W.data(), params.has_bias_ ? bias.data() : nullptr, out.data(),
                         static_cast<int>(in_data.size())));
  unpack(out, out_data);
}

// FullyConnectedGradOp::compute branch (fully_connected_op_internal.h:38-71)
inline void fully_connected_grad_op(const tensor_t &prev_out, const vec_t &W, tensor_t &dW,
                                    tensor_t &db, tensor_t &curr_delta, tensor_t &prev_delta,
                                    const core::fully_params &params) {
  std::vector<float> x = pack(prev_out), dy = pack(curr_delta);
  std::vector<float> dx(prev_delta.size() * params.in_size_);
  check(b200_fc_bwd_host(ctx(), static_cast<int>(params.in_size_), static_cast<int>(params.out_size_),
                         x.data(), W.data(), dy.data(), dx.data(), dW[0].data(),
                         params.has_bias_ ? db[0].data() : nullptr, /*accumulate=*/1,
                         static_cast<int>(prev_out.size())));
  unpack(dx, prev_delta);
}

// MaxPoolOp::compute branch (maxpool_op_internal.h:16-39); the winning indices
// go back into params.out2inmax, which MaxPoolGradOp reads.
inline void maxpool_op(const tensor_t &in_data, tensor_t &out_data, core::maxpool_params &params) {
  b200_pool_desc d = pool_desc(params);
  const size_t B = in_data.size(), n_out = params.out.size();
  std::vector<float> in = pack(in_data), out(B * n_out);
  std::vector<int32_t> arg(B * n_out);
  check(b200_maxpool_fwd_host(ctx(), &d, in.data(), out.data(), arg.data(), static_cast<int>(B)));
  unpack(out, out_data);
  for (size_t s = 0; s < B; ++s) {
    params.out2inmax[s].resize(n_out);
    for (size_t i = 0; i < n_out; ++i) params.out2inmax[s][i] = static_cast<size_t>(arg[s * n_out + i]);
  }
}

// MaxPoolGradOp::compute branch (maxpool_op_internal.h:41-57)
inline void maxpool_grad_op(tensor_t &prev_delta, const tensor_t &curr_delta,
                            core::maxpool_params &params) {
  b200_pool_desc d = pool_desc(params);
  const size_t B = prev_delta.size(), n_out = params.out.size();
  std::vector<float> dy = pack(curr_delta), dx(B * params.in.size());
  std::vector<int32_t> arg(B * n_out);
  for (size_t s = 0; s < B; ++s)
    for (size_t i = 0; i < n_out; ++i) arg[s * n_out + i] = static_cast<int32_t>(params.out2inmax[s][i]);
  check(b200_maxpool_bwd_host(ctx(), &d, dy.data(), arg.data(), dx.data(), static_cast<int>(B)));
  unpack(dx, prev_delta);
}

// activation_layer::forward_propagation / back_propagation branch
// (tiny_dnn/activations/activation_layer.h:74-91).  `type` is the layer's layer_type() string;
// `param` the activation's constructor parameter (leaky relu: epsilon, elu: alpha);
// returns false for an activation that is not on the path (the caller then runs its own loop).
inline int activation_kind(const std::string &type) {
  if (type == "relu-activation") return B200_ACT_RELU;
  if (type == "tanh-activation") return B200_ACT_TANH;
  if (type == "softmax-activation") return B200_ACT_SOFTMAX;
  if (type == "sigmoid-activation") return B200_ACT_SIGMOID;
  if (type == "leaky-relu-activation") return B200_ACT_LEAKY_RELU;
  if (type == "elu-activation") return B200_ACT_ELU;
  return B200_ACT_NONE;
}

inline bool activation_op(const std::string &type, float param, const tensor_t &x, tensor_t &y) {
  const int kind = activation_kind(type);
  if (kind == B200_ACT_NONE || x.empty()) return false;
  std::vector<float> in = pack(x), out(in.size());
  check(b200_act_param_fwd_host(ctx(), kind, param, in.data(), out.data(), static_cast<int>(x[0].size()),
                          static_cast<int>(x.size())));
  unpack(out, y);
  return true;
}

inline bool activation_grad_op(const std::string &type, float param, const tensor_t &y, const tensor_t &dy,
                               tensor_t &dx) {
  const int kind = activation_kind(type);
  if (kind == B200_ACT_NONE || y.empty()) return false;
  std::vector<float> fy = pack(y), fdy = pack(dy), fdx(fy.size());
  check(b200_act_param_bwd_host(ctx(), kind, param, fy.data(), fdy.data(), fdx.data(), static_cast<int>(y[0].size()),
                          static_cast<int>(y.size())));
  unpack(fdx, dx);
  return true;
}

// batch_normalization_layer::forward_propagation / back_propagation branches
// (tiny_dnn/layers/batch_normalization_layer.h:94-168).  Train phase: `mean` / `variance` (the layer's
// mean_current_ / variance_current_) receive this mini-batch's moments; test phase: they are the moving
// averages.  `stddev` is the layer's stddev_, which the backward pass reads.
inline void batch_normalization_op(size_t channels, size_t spatial, float_t eps, bool train, const tensor_t &x,
                                   vec_t &mean, vec_t &variance, vec_t &stddev, tensor_t &y) {
  if (x.empty()) return;
  std::vector<float> in = pack(x), out(in.size());
  std::vector<float> m(mean.begin(), mean.end()), v(variance.begin(), variance.end()), sd(channels);
  m.resize(channels);
  v.resize(channels);
  check(b200_batchnorm_fwd_host(ctx(), static_cast<int>(channels), static_cast<int>(spatial), static_cast<float>(eps),
                                in.data(), m.data(), v.data(), sd.data(), out.data(), static_cast<int>(x.size()),
                                train ? 1 : 0));
  if (train) {
    mean.assign(m.begin(), m.end());
    variance.assign(v.begin(), v.end());
  }
  stddev.assign(sd.begin(), sd.end());
  unpack(out, y);
}

inline void batch_normalization_grad_op(size_t channels, size_t spatial, const tensor_t &y, const tensor_t &dy,
                                        const vec_t &stddev, tensor_t &dx) {
  if (y.empty()) return;
  std::vector<float> fy = pack(y), fdy = pack(dy), fdx(fy.size()), sd(stddev.begin(), stddev.end());
  check(b200_batchnorm_bwd_host(ctx(), static_cast<int>(channels), static_cast<int>(spatial), fy.data(), fdy.data(),
                                sd.data(), fdx.data(), static_cast<int>(y.size())));
  unpack(fdx, dx);
}

// lrn_layer::forward_propagation branch, norm_region::across_channels (tiny_dnn/layers/lrn_layer.h:82-143)
inline void lrn_op(size_t channels, size_t area, size_t size, float_t alpha, float_t beta, const tensor_t &x,
                   tensor_t &y) {
  if (x.empty()) return;
  std::vector<float> in = pack(x), out(in.size());
  check(b200_lrn_fwd_host(ctx(), in.data(), out.data(), static_cast<int>(channels), static_cast<int>(area),
                          static_cast<int>(size), static_cast<float>(alpha), static_cast<float>(beta),
                          static_cast<int>(x.size())));
  unpack(out, y);
}

// average_pooling_layer::forward_propagation branch: replaces tiny_average_pooling_kernel
// (tiny_dnn/layers/average_pooling_layer.h:25-55)
inline void average_pooling_op(const b200_pool_desc &d, const tensor_t &in_data, const vec_t &W, const vec_t &bias,
                               tensor_t &out_data) {
  std::vector<float> in = pack(in_data), out(out_data.size() * out_data[0].size());
  check(b200_avgpool_fwd_host(ctx(), &d, in.data(), W.data(), bias.data(), out.data(),
                              static_cast<int>(in_data.size())));
  unpack(out, out_data);
}

// average_pooling_layer::back_propagation branch: replaces tiny_average_pooling_back_kernel
// (average_pooling_layer.h:58-106); the batch sums of dW / db are added to row 0
inline void average_pooling_grad_op(const b200_pool_desc &d, const tensor_t &prev_out, const vec_t &W, tensor_t &dW,
                                    tensor_t &db, const tensor_t &curr_delta, tensor_t &prev_delta) {
  std::vector<float> x = pack(prev_out), dy = pack(curr_delta), dx(prev_delta.size() * prev_delta[0].size());
  check(b200_avgpool_bwd_host(ctx(), &d, x.data(), W.data(), dy.data(), dx.data(), dW[0].data(), db[0].data(),
                              /*accumulate=*/1, static_cast<int>(prev_out.size())));
  unpack(dx, prev_delta);
}

}  // namespace b200
}  // namespace tiny_dnn
