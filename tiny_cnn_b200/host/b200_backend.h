// b200_backend.h -- core::backend implementation for the quantized layers.
//
// quantized_convolutional_layer calls `layer::backend_->conv2d_q(in, out)`
// (tiny_dnn/layers/quantized_convolutional_layer.h:236-245) on whatever object
// was installed with layer::set_backend (tiny_dnn/layers/layer.h:85-87).  This
// class is that object for engine backend_t::b200: conv2d_q pads the rows the
// way the layer's own helper does and runs the bit-exact uint8 pipeline of the
// library; fully_q does the same for the fully-connected kernel.  The other
// virtuals of the interface (tiny_dnn/core/backend.h:111-171) are not on the
// path and throw nn_not_implemented_error, as the reference's own partial
// backends do.
#pragma once

#include <functional>
#include <vector>

#include "tiny_dnn/core/kernels/b200_glue.h"

namespace tiny_dnn {
namespace core {

class b200_backend : public backend {
 public:
  // quantized convolution: `pad` is the layer's copy_and_pad_input, `cws` its storage
  b200_backend(conv_params *params, std::function<void(const tensor_t &)> pad,
               conv_layer_worker_specific_storage *cws)
    : params_c_(params), params_f_(nullptr), pad_(pad), cws_(cws) {}
  // quantized fully connected
  explicit b200_backend(fully_params *params) : params_c_(nullptr), params_f_(params), cws_(nullptr) {}

  void conv2d_q(const std::vector<tensor_t *> &in_data, std::vector<tensor_t *> &out_data) override {
    pad_(*in_data[0]);
    const std::vector<const vec_t *> &in = cws_->prev_out_padded_;
    const vec_t &W = (*in_data[1])[0];
    const vec_t &bias = (*in_data[2])[0];
    tensor_t &out = *out_data[0];
    std::vector<uint8_t> tbl;
    b200_conv_desc d = tiny_dnn::b200::conv_desc(*params_c_, tbl);
    d.tbl = nullptr;
    // the quantized layer never sets the dilation members of its conv_params
    // (quantized_convolutional_layer.h:324-346); its kernel has no dilation
    d.dil_w = d.dil_h = 1;
    const size_t n_in = params_c_->in_padded.size(), n_out = params_c_->out.size();
    std::vector<float> x(in.size() * n_in), y(in.size() * n_out);
    for (size_t s = 0; s < in.size(); ++s) std::copy(in[s]->begin(), in[s]->begin() + n_in, x.begin() + s * n_in);
    if (!params_c_->tbl.is_empty()) {
      tbl.assign(params_c_->tbl.connected_.begin(), params_c_->tbl.connected_.end());
      d.tbl = tbl.data();
    }
    tiny_dnn::b200::check(b200_qconv2d_fwd_host(tiny_dnn::b200::ctx(), &d, x.data(), W.data(),
                                                params_c_->has_bias ? bias.data() : nullptr, y.data(),
                                                static_cast<int>(in.size())));
    tiny_dnn::b200::unpack(y, out);
  }

  void fully_q(const std::vector<tensor_t *> &in_data, std::vector<tensor_t *> &out_data) override {
    const tensor_t &in = *in_data[0];
    const vec_t &W = (*in_data[1])[0];
    tensor_t &out = *out_data[0];
    std::vector<float> x = tiny_dnn::b200::pack(in), y(in.size() * params_f_->out_size_);
    tiny_dnn::b200::check(b200_qfc_fwd_host(
      tiny_dnn::b200::ctx(), static_cast<int>(params_f_->in_size_), static_cast<int>(params_f_->out_size_),
      x.data(), W.data(), params_f_->has_bias_ ? (*in_data[2])[0].data() : nullptr, y.data(),
      static_cast<int>(in.size())));
    tiny_dnn::b200::unpack(y, out);
  }

  // tiny_backend::conv2d_eq (backend_tiny.h:115-135): in_data = data, W, bias, data range (2 floats
  // per sample), W range, bias range; out_data = uint8 values held in floats, their range per sample
  void conv2d_eq(const std::vector<tensor_t *> &in_data, std::vector<tensor_t *> &out_data) override {
    pad_(*in_data[0]);
    const std::vector<const vec_t *> &in = cws_->prev_out_padded_;
    const vec_t &W = (*in_data[1])[0];
    const vec_t &bias = (*in_data[2])[0];
    const tensor_t &in_r = *in_data[3];
    const vec_t &W_r = (*in_data[4])[0];
    const vec_t &b_r = (*in_data[5])[0];
    std::vector<uint8_t> tbl;
    b200_conv_desc d = tiny_dnn::b200::conv_desc(*params_c_, tbl);
    d.tbl = nullptr;
    d.dil_w = d.dil_h = 1;
    const size_t n_in = params_c_->in_padded.size(), n_out = params_c_->out.size(), B = in.size();
    std::vector<float> x(B * n_in), y(B * n_out), xr(2 * B), yr(2 * B);
    for (size_t s = 0; s < B; ++s) {
      std::copy(in[s]->begin(), in[s]->begin() + n_in, x.begin() + s * n_in);
      xr[2 * s] = in_r[s][0];
      xr[2 * s + 1] = in_r[s][1];
    }
    if (!params_c_->tbl.is_empty()) {
      tbl.assign(params_c_->tbl.connected_.begin(), params_c_->tbl.connected_.end());
      d.tbl = tbl.data();
    }
    tiny_dnn::b200::check(b200_qconv2d_eq_fwd_host(tiny_dnn::b200::ctx(), &d, x.data(), W.data(),
                                                   params_c_->has_bias ? bias.data() : nullptr, xr.data(), W_r.data(),
                                                   b_r.data(), y.data(), yr.data(), static_cast<int>(B)));
    tiny_dnn::b200::unpack(y, *out_data[0]);
    tensor_t &out_r = *out_data[1];
    for (size_t s = 0; s < B; ++s) {
      out_r[s][0] = yr[2 * s];
      out_r[s][1] = yr[2 * s + 1];
    }
  }
  void conv2d_q(const std::vector<tensor_t *> &, const std::vector<tensor_t *> &,
                std::vector<tensor_t *> &, std::vector<tensor_t *> &) override { na(); }
  void deconv2d(const std::vector<tensor_t *> &, std::vector<tensor_t *> &) override { na(); }
  void deconv2d_q(const std::vector<tensor_t *> &, std::vector<tensor_t *> &) override { na(); }
  void deconv2d_eq(const std::vector<tensor_t *> &, std::vector<tensor_t *> &) override { na(); }
  void deconv2d(const std::vector<tensor_t *> &, const std::vector<tensor_t *> &,
                std::vector<tensor_t *> &, std::vector<tensor_t *> &) override { na(); }
  void deconv2d_q(const std::vector<tensor_t *> &, const std::vector<tensor_t *> &,
                  std::vector<tensor_t *> &, std::vector<tensor_t *> &) override { na(); }
  // tiny_backend::fully_eq (backend_tiny.h:321-345)
  void fully_eq(const std::vector<tensor_t *> &in_data, std::vector<tensor_t *> &out_data) override {
    const tensor_t &in = *in_data[0];
    const vec_t &W = (*in_data[1])[0];
    const tensor_t &in_r = *in_data[3];
    const vec_t &W_r = (*in_data[4])[0];
    const vec_t &b_r = (*in_data[5])[0];
    const size_t B = in.size();
    std::vector<float> x = tiny_dnn::b200::pack(in), y(B * params_f_->out_size_), xr(2 * B), yr(2 * B);
    for (size_t s = 0; s < B; ++s) {
      xr[2 * s] = in_r[s][0];
      xr[2 * s + 1] = in_r[s][1];
    }
    tiny_dnn::b200::check(b200_qfc_eq_fwd_host(
      tiny_dnn::b200::ctx(), static_cast<int>(params_f_->in_size_), static_cast<int>(params_f_->out_size_), x.data(),
      W.data(), params_f_->has_bias_ ? (*in_data[2])[0].data() : nullptr, xr.data(), W_r.data(), b_r.data(), y.data(),
      yr.data(), static_cast<int>(B)));
    tiny_dnn::b200::unpack(y, *out_data[0]);
    tensor_t &out_r = *out_data[1];
    for (size_t s = 0; s < B; ++s) {
      out_r[s][0] = yr[2 * s];
      out_r[s][1] = yr[2 * s + 1];
    }
  }
  void fully_q(const std::vector<tensor_t *> &, const std::vector<tensor_t *> &,
               std::vector<tensor_t *> &, std::vector<tensor_t *> &) override { na(); }

  backend_t type() const override { return backend_t::b200; }

 private:
  static void na() { throw nn_not_implemented_error("not on the B200 path"); }
  conv_params *params_c_;
  fully_params *params_f_;
  std::function<void(const tensor_t &)> pad_;
  conv_layer_worker_specific_storage *cws_;
};

}  // namespace core
}  // namespace tiny_dnn
