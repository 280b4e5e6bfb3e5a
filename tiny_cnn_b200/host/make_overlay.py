"""Generate the tiny-dnn overlay that adds the engine `core::backend_t::b200`.

tiny-dnn is header-only, so the new engine is delivered as an include directory
placed BEFORE the tiny-dnn tree on the compiler's include path:

    g++ -std=c++14 -I <overlay> -I <tiny-dnn> -I <repo>/include app.cpp \
        -L <repo>/tiny_cnn_b200/csrc -ltinycnn_b200

The overlay holds patched copies of exactly the headers that carry the backend
switch, produced here from the user's own tiny-dnn tree by anchored text edits
(nothing of tiny-dnn is stored in this repository), plus the three headers of this
directory (b200_glue.h, b200_backend.h, b200_net.h) under tiny_dnn/core/kernels/
and tiny_dnn/core/.  Every edit asserts that its anchor is present, so a tiny-dnn
version the patches do not fit fails loudly instead of silently mis-patching.

    python -m tiny_cnn_b200.host.make_overlay --reference /path/to/tiny-dnn --out build/overlay
"""
from __future__ import annotations

import argparse
import shutil
from pathlib import Path

HERE = Path(__file__).resolve().parent


def _edit(text: str, old: str, new: str, path: str, count: int = 1) -> str:
    if text.count(old) < count:
        raise RuntimeError(f"overlay patch does not fit {path}: anchor not found:\n{old}")
    return text.replace(old, new, count)


GLUE_INCLUDE = '#include "tiny_dnn/core/kernels/b200_glue.h"\n'


def patch_backend_h(t, p):
    t = _edit(t, "enum class backend_t { internal, nnpack, libdnn, avx, opencl, cblas, intel_mkl };",
              "enum class backend_t { internal, nnpack, libdnn, avx, opencl, cblas, intel_mkl, b200 };", p)
    t = _edit(t, '    case backend_t::intel_mkl: os << "Intel MKL"; break;',
              '    case backend_t::intel_mkl: os << "Intel MKL"; break;\n'
              '    case backend_t::b200: os << "B200"; break;', p)
    return t


def patch_conv2d_op(t, p):
    t = _edit(t, '#include "tiny_dnn/core/kernels/conv2d_op_nnpack.h"\n',
              '#include "tiny_dnn/core/kernels/conv2d_op_nnpack.h"\n' + GLUE_INCLUDE, p)
    t = _edit(t, "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));",
              "    } else if (engine == core::backend_t::b200) {\n"
              "      b200::conv2d_op(in_data, W[0], bias[0], out_data, params);\n"
              "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));", p)
    return t


def patch_conv2d_grad_op(t, p):
    t = _edit(t, "namespace tiny_dnn {\n", GLUE_INCLUDE + "\nnamespace tiny_dnn {\n", p)
    t = _edit(t, "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));",
              "    } else if (engine == core::backend_t::b200) {\n"
              "      b200::conv2d_grad_op(prev_out, W[0], dW, db, curr_delta, prev_delta, params);\n"
              "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));", p)
    return t


def patch_fc_op(t, p):
    t = _edit(t, "namespace tiny_dnn {\n", GLUE_INCLUDE + "\nnamespace tiny_dnn {\n", p)
    t = _edit(t, "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));",
              "    } else if (engine == core::backend_t::b200) {\n"
              "      b200::fully_connected_op(in_data, W[0], params.has_bias_ ? (*bias)[0] : vec_t(),\n"
              "                               out_data, params);\n"
              "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));", p)
    return t


def patch_fc_grad_op(t, p):
    t = _edit(t, "namespace tiny_dnn {\n", GLUE_INCLUDE + "\nnamespace tiny_dnn {\n", p)
    t = _edit(t, "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));",
              "    } else if (engine == core::backend_t::b200) {\n"
              "      b200::fully_connected_grad_op(prev_out, W[0], dW, params.has_bias_ ? *db : dummy,\n"
              "                                    curr_delta, prev_delta, params);\n"
              "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));", p)
    return t


def patch_maxpool_op(t, p):
    t = _edit(t, "namespace tiny_dnn {\n", GLUE_INCLUDE + "\nnamespace tiny_dnn {\n", p)
    t = _edit(t, "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));",
              "    } else if (engine == core::backend_t::b200) {\n"
              "      b200::maxpool_op(in_data, out_data, params);\n"
              "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));", p)
    return t


def patch_maxpool_grad_op(t, p):
    t = _edit(t, "namespace tiny_dnn {\n", GLUE_INCLUDE + "\nnamespace tiny_dnn {\n", p)
    t = _edit(t, "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));",
              "    } else if (engine == core::backend_t::b200) {\n"
              "      b200::maxpool_grad_op(prev_delta, curr_delta, params);\n"
              "    } else {\n      throw nn_error(\"Not supported engine: \" + to_string(engine));", p)
    return t


def _params_accessor(t, p, anchor, type_name):
    """public read access to the layer's private params_ (the device twin of a network is
    described from them)"""
    return _edit(t, anchor, anchor + f"  const {type_name} &b200_params() const {{ return params_; }}\n\n", p)


def patch_conv_layer(t, p):
    # the same Conv2dOp / Conv2dGradOp objects serve the new engine, so that
    # layer::set_backend_type() can switch engines at run time
    t = _params_accessor(t, p, "class convolutional_layer : public layer {\n public:\n", "core::conv_params")
    return _edit(t, "    if (backend_type == core::backend_t::internal ||\n"
                    "        backend_type == core::backend_t::nnpack ||\n"
                    "        backend_type == core::backend_t::avx) {\n"
                    "      kernel_fwd_.reset(new Conv2dOp(ctx));",
                 "    if (backend_type == core::backend_t::internal ||\n"
                 "        backend_type == core::backend_t::nnpack ||\n"
                 "        backend_type == core::backend_t::b200 ||\n"
                 "        backend_type == core::backend_t::avx) {\n"
                 "      kernel_fwd_.reset(new Conv2dOp(ctx));", p)


def patch_fc_layer(t, p):
    t = _params_accessor(t, p, "class fully_connected_layer : public layer {\n public:\n", "core::fully_params")
    return _edit(t, "    if (backend_type == core::backend_t::internal ||\n"
                    "        backend_type == core::backend_t::avx ||",
                 "    if (backend_type == core::backend_t::internal ||\n"
                 "        backend_type == core::backend_t::b200 ||\n"
                 "        backend_type == core::backend_t::avx ||", p)


def patch_maxpool_layer(t, p):
    t = _params_accessor(t, p, "class max_pooling_layer : public layer {\n public:\n", "core::maxpool_params")
    return _edit(t, "    if (backend_type == core::backend_t::internal ||\n"
                    "        backend_type == core::backend_t::nnpack ||\n"
                    "        backend_type == core::backend_t::avx) {\n"
                    "      kernel_fwd_.reset(new MaxPoolOp(ctx));",
                 "    if (backend_type == core::backend_t::internal ||\n"
                 "        backend_type == core::backend_t::nnpack ||\n"
                 "        backend_type == core::backend_t::b200 ||\n"
                 "        backend_type == core::backend_t::avx) {\n"
                 "      kernel_fwd_.reset(new MaxPoolOp(ctx));", p)


def patch_qconv_layer(t, p):
    t = _edit(t, '#include "tiny_dnn/core/backend_tiny.h"\n',
              '#include "tiny_dnn/core/backend_tiny.h"\n#include "tiny_dnn/core/b200_backend.h"\n', p)
    t = _edit(t, "    } else {\n      throw nn_error(\"Not supported backend type.\");",
              "    } else if (backend_type == core::backend_t::b200) {\n"
              "      backend = std::make_shared<core::b200_backend>(\n"
              "        &params_, [this](const tensor_t &in) { return copy_and_pad_input(in); }, &cws_);\n"
              "    } else {\n      throw nn_error(\"Not supported backend type.\");", p)
    # the padded staging buffer of padding::same is only created by init(), which
    # the reference never calls; valid padding (all benchmark shapes) is unaffected
    return t


def patch_avgpool_layer(t, p):
    """average_pooling_layer has no engine argument; layer::set_backend_type(b200) selects the
    device kernels (average_pooling_layer.h:186-221)."""
    t = _edit(t, '#include "tiny_dnn/util/util.h"\n', '#include "tiny_dnn/util/util.h"\n' + GLUE_INCLUDE, p)
    t = _edit(t, "    tiny_average_pooling_kernel(parallelize_, in_data, out_data, out_,\n"
                 "                                Base::scale_factor_, Base::out2wi_);",
              "    if (layer::engine() == core::backend_t::b200) {\n"
              "      b200::average_pooling_op(b200_pool_desc(), *in_data[0], (*in_data[1])[0], (*in_data[2])[0],\n"
              "                               *out_data[0]);\n"
              "      return;\n"
              "    }\n"
              "    tiny_average_pooling_kernel(parallelize_, in_data, out_data, out_,\n"
              "                                Base::scale_factor_, Base::out2wi_);", p)
    t = _edit(t, "    tiny_average_pooling_back_kernel(\n      parallelize_, in_data, out_data, out_grad, in_grad, in_,",
              "    if (layer::engine() == core::backend_t::b200) {\n"
              "      b200::average_pooling_grad_op(b200_pool_desc(), *in_data[0], (*in_data[1])[0], *in_grad[1],\n"
              "                                    *in_grad[2], *out_grad[0], *in_grad[0]);\n"
              "      return;\n"
              "    }\n"
              "    tiny_average_pooling_back_kernel(\n      parallelize_, in_data, out_data, out_grad, in_grad, in_,", p)
    t = _edit(t, "  std::pair<size_t, size_t> pool_size() const {\n",
              "  ::b200_pool_desc b200_pool_desc() const {\n"
              "    ::b200_pool_desc d{};\n"
              "    d.in_w = static_cast<int32_t>(in_.width_);\n"
              "    d.in_h = static_cast<int32_t>(in_.height_);\n"
              "    d.in_c = static_cast<int32_t>(in_.depth_);\n"
              "    d.out_w = static_cast<int32_t>(out_.width_);\n"
              "    d.out_h = static_cast<int32_t>(out_.height_);\n"
              "    d.pool_w = static_cast<int32_t>(pool_size_x_);\n"
              "    d.pool_h = static_cast<int32_t>(pool_size_y_);\n"
              "    d.stride_w = static_cast<int32_t>(stride_x_);\n"
              "    d.stride_h = static_cast<int32_t>(stride_y_);\n"
              "    return d;\n"
              "  }\n\n"
              "  std::pair<size_t, size_t> pool_size() const {\n", p)
    return t


def patch_activation_layer(t, p):
    """relu / tanh / softmax / sigmoid / leaky relu / elu under layer::set_backend_type(b200)
    (activation_layer.h:74-91); the other activations keep their own loops.  The constructor
    parameter of leaky relu (epsilon) and elu (alpha) reaches the base class through a virtual
    that the two derived headers override."""
    t = _edit(t, "namespace tiny_dnn {\n", GLUE_INCLUDE + "\nnamespace tiny_dnn {\n", p)
    t = _edit(t, "    const tensor_t &x = *in_data[0];\n    tensor_t &y       = *out_data[0];\n",
              "    const tensor_t &x = *in_data[0];\n    tensor_t &y       = *out_data[0];\n"
              "    if (layer::engine() == core::backend_t::b200 &&\n"
              "        b200::activation_op(layer_type(), static_cast<float>(b200_act_param()), x, y))\n"
              "      return;\n", p)
    t = _edit(t, "    const tensor_t &y  = *out_data[0];\n",
              "    const tensor_t &y  = *out_data[0];\n"
              "    if (layer::engine() == core::backend_t::b200 &&\n"
              "        b200::activation_grad_op(layer_type(), static_cast<float>(b200_act_param()), y, dy, dx))\n"
              "      return;\n", p)
    t = _edit(t, "  std::string layer_type() const override = 0;\n",
              "  std::string layer_type() const override = 0;\n\n"
              "  // constructor parameter of the activation (leaky relu: epsilon, elu: alpha)\n"
              "  virtual float_t b200_act_param() const { return float_t(0); }\n", p)
    return t


def patch_leaky_relu_layer(t, p):
    return _edit(t, "  float_t epsilon_value() const { return epsilon_; }\n",
                 "  float_t epsilon_value() const { return epsilon_; }\n\n"
                 "  float_t b200_act_param() const override { return epsilon_; }\n", p)


def patch_elu_layer(t, p):
    return _edit(t, '  std::string layer_type() const override { return "elu-activation"; }\n',
                 '  std::string layer_type() const override { return "elu-activation"; }\n\n'
                 "  float_t b200_act_param() const override { return alpha_; }\n", p)


def patch_batchnorm_layer(t, p):
    """batch_normalization_layer has no engine argument; layer::set_backend_type(b200) selects the device
    kernels (batch_normalization_layer.h:94-168).  Accessors give the fit hook the moving averages."""
    t = _edit(t, '#include "tiny_dnn/util/util.h"\n', '#include "tiny_dnn/util/util.h"\n' + GLUE_INCLUDE, p)
    t = _edit(t, "    tensor_t &in  = *in_data[0];\n    tensor_t &out = *out_data[0];\n",
              "    tensor_t &in  = *in_data[0];\n    tensor_t &out = *out_data[0];\n"
              "    if (layer::engine() == core::backend_t::b200) {\n"
              "      b200::batch_normalization_op(in_channels_, in_spatial_size_, eps_, phase_ == net_phase::train, in,\n"
              "                                   mean, variance, stddev_, out);\n"
              "      if (phase_ == net_phase::train && update_immidiately_) {\n"
              "        mean_     = mean_current_;\n"
              "        variance_ = variance_current_;\n"
              "      }\n"
              "      return;\n"
              "    }\n", p)
    t = _edit(t, "    tensor_t delta_dot_y = curr_out;\n",
              "    if (layer::engine() == core::backend_t::b200) {\n"
              "      b200::batch_normalization_grad_op(in_channels_, in_spatial_size_, curr_out, curr_delta, stddev_,\n"
              "                                        prev_delta);\n"
              "      return;\n"
              "    }\n"
              "    tensor_t delta_dot_y = curr_out;\n", p)
    t = _edit(t, "  float_t epsilon() const { return eps_; }\n",
              "  float_t epsilon() const { return eps_; }\n\n"
              "  size_t b200_channels() const { return in_channels_; }\n"
              "  size_t b200_spatial() const { return in_spatial_size_; }\n"
              "  vec_t &b200_mean() { return mean_; }\n"
              "  vec_t &b200_variance() { return variance_; }\n"
              "  vec_t &b200_mean_current() { return mean_current_; }\n"
              "  vec_t &b200_variance_current() { return variance_current_; }\n"
              "  vec_t &b200_stddev() { return stddev_; }\n"
              "  net_phase b200_phase() const { return phase_; }\n", p)
    return t


def patch_lrn_layer(t, p):
    """lrn_layer across channels under layer::set_backend_type(b200) (lrn_layer.h:82-95)."""
    t = _edit(t, '#include "tiny_dnn/util/util.h"\n', '#include "tiny_dnn/util/util.h"\n' + GLUE_INCLUDE, p)
    t = _edit(t, "    // @todo revise the parallelism strategy\n",
              "    if (layer::engine() == core::backend_t::b200 && region_ == norm_region::across_channels) {\n"
              "      b200::lrn_op(in_shape_.depth_, in_shape_.area(), size_, alpha_, beta_, *in_data[0], *out_data[0]);\n"
              "      return;\n"
              "    }\n"
              "    // @todo revise the parallelism strategy\n", p)
    return t


def patch_layer_h(t, p):
    """layer::set_sample_count (layer.h:699-718) grows every gradient tensor to one row per sample.
    The device kernels return the batch sum of a weight gradient in row 0, so under engine b200
    the weight-gradient tensors stay as they are (one row for a fresh layer): edge::merge_grads
    (node.h:89-103) then reads len(W) floats instead of B x len(W)."""
    return _edit(t, "      resize(ith_in_node(i)->get_gradient());\n    }\n\n    for (size_t i = 0; i < out_channels_; i++) {",
                 "      if (backend_type_ == core::backend_t::b200 && is_trainable_weight(in_type_[i])) continue;\n"
                 "      resize(ith_in_node(i)->get_gradient());\n    }\n\n    for (size_t i = 0; i < out_channels_; i++) {", p)


def patch_optimizer_h(t, p):
    """public access to the per-weight state of adagrad / adam / momentum (stateful_optimizer::E_,
    optimizer.h:34-48): the device-resident fit writes its optimizer state back into these maps."""
    return _edit(t, " protected:\n  template <int Index>\n  vec_t &get(const vec_t &key) {",
                 "  std::unordered_map<const vec_t *, vec_t> *b200_maps() { return E_; }\n\n"
                 " protected:\n  template <int Index>\n  vec_t &get(const vec_t &key) {", p)


def patch_network_h(t, p):
    """network::fit (network.h:840-879) hands the loop over mini-batches to the device-resident step
    when the whole network is on the path (b200_net.h); otherwise nothing changes."""
    t = _edit(t, "template <typename NetType>\nclass network;\n",
              "template <typename NetType>\nclass network;\n\n"
              "// defined in tiny_dnn/core/b200_net.h (included at the end of this file)\n"
              "template <typename Error, typename Net, typename Optimizer, typename OnBatch, typename OnEpoch>\n"
              "bool b200_fit_hook(Net &nn, Optimizer &optimizer, const std::vector<tensor_t> &inputs,\n"
              "                   const std::vector<tensor_t> &desired_outputs, size_t batch_size, int epoch,\n"
              "                   OnBatch on_batch, OnEpoch on_epoch, const std::vector<tensor_t> &t_cost,\n"
              "                   bool *stop);\n"
              "template <typename Error, typename Net, typename Optimizer, typename In, typename Tg, typename OnBatch,\n"
              "          typename OnEpoch>\n"
              "bool b200_fit_hook_rows(Net &nn, Optimizer &optimizer, const std::vector<In> &inputs,\n"
              "                        const std::vector<Tg> &targets, size_t batch_size, int epoch, OnBatch on_batch,\n"
              "                        OnEpoch on_epoch, bool reset_weights, bool *stop);\n", p)
    # the public train (class labels) and fit (target vectors) overloads, before normalize_tensor
    t = _edit(t, "    std::vector<tensor_t> input_tensor, output_tensor, t_cost_tensor;\n"
                 "    normalize_tensor(inputs, input_tensor);\n"
                 "    normalize_tensor(class_labels, output_tensor);\n",
              "    if (t_cost.empty() &&\n"
              "        b200_fit_hook_rows<Error>(*this, optimizer, inputs, class_labels, batch_size, epoch,\n"
              "                                  on_batch_enumerate, on_epoch_enumerate, reset_weights, &stop_training_))\n"
              "      return true;\n"
              "    std::vector<tensor_t> input_tensor, output_tensor, t_cost_tensor;\n"
              "    normalize_tensor(inputs, input_tensor);\n"
              "    normalize_tensor(class_labels, output_tensor);\n", p)
    t = _edit(t, "    std::vector<tensor_t> input_tensor, output_tensor, t_cost_tensor;\n"
                 "    normalize_tensor(inputs, input_tensor);\n"
                 "    normalize_tensor(desired_outputs, output_tensor);\n",
              "    if (t_cost.empty() &&\n"
              "        b200_fit_hook_rows<Error>(*this, optimizer, inputs, desired_outputs, batch_size, epoch,\n"
              "                                  on_batch_enumerate, on_epoch_enumerate, reset_weights, &stop_training_))\n"
              "      return true;\n"
              "    std::vector<tensor_t> input_tensor, output_tensor, t_cost_tensor;\n"
              "    normalize_tensor(inputs, input_tensor);\n"
              "    normalize_tensor(desired_outputs, output_tensor);\n", p)
    t = _edit(t, "    optimizer.reset();\n    stop_training_ = false;\n",
              "    optimizer.reset();\n    stop_training_ = false;\n"
              "    if (b200_fit_hook<Error>(*this, optimizer, inputs, desired_outputs, batch_size, epoch,\n"
              "                             on_batch_enumerate, on_epoch_enumerate, t_cost, &stop_training_))\n"
              "      return true;\n", p)
    t = _edit(t, "  void stop_ongoing_training() { stop_training_ = true; }\n",
              "  void stop_ongoing_training() { stop_training_ = true; }\n\n"
              "  // device twin of this network under engine backend_t::b200 (tiny_dnn/core/b200_net.h)\n"
              "  std::shared_ptr<void> b200_twin_;\n", p)
    return t + '\n#include "tiny_dnn/core/b200_net.h"\n'


PATCHES = {
    "tiny_dnn/core/backend.h": patch_backend_h,
    "tiny_dnn/core/kernels/conv2d_op.h": patch_conv2d_op,
    "tiny_dnn/core/kernels/conv2d_grad_op.h": patch_conv2d_grad_op,
    "tiny_dnn/core/kernels/fully_connected_op.h": patch_fc_op,
    "tiny_dnn/core/kernels/fully_connected_grad_op.h": patch_fc_grad_op,
    "tiny_dnn/core/kernels/maxpool_op.h": patch_maxpool_op,
    "tiny_dnn/core/kernels/maxpool_grad_op.h": patch_maxpool_grad_op,
    "tiny_dnn/layers/convolutional_layer.h": patch_conv_layer,
    "tiny_dnn/layers/fully_connected_layer.h": patch_fc_layer,
    "tiny_dnn/layers/max_pooling_layer.h": patch_maxpool_layer,
    "tiny_dnn/layers/quantized_convolutional_layer.h": patch_qconv_layer,
    "tiny_dnn/layers/average_pooling_layer.h": patch_avgpool_layer,
    "tiny_dnn/activations/activation_layer.h": patch_activation_layer,
    "tiny_dnn/activations/leaky_relu_layer.h": patch_leaky_relu_layer,
    "tiny_dnn/activations/elu_layer.h": patch_elu_layer,
    "tiny_dnn/layers/batch_normalization_layer.h": patch_batchnorm_layer,
    "tiny_dnn/layers/lrn_layer.h": patch_lrn_layer,
    "tiny_dnn/layers/layer.h": patch_layer_h,
    "tiny_dnn/optimizers/optimizer.h": patch_optimizer_h,
    "tiny_dnn/network.h": patch_network_h,
}


def make_overlay(reference: Path, out: Path) -> Path:
    reference, out = Path(reference), Path(out)
    if not (reference / "tiny_dnn" / "tiny_dnn.h").exists():
        raise RuntimeError(f"{reference} is not a tiny-dnn tree")
    for rel, fn in PATCHES.items():
        src = reference / rel
        dst = out / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        dst.write_text(fn(src.read_text(), rel))
    (out / "tiny_dnn/core/kernels").mkdir(parents=True, exist_ok=True)
    shutil.copyfile(HERE / "b200_glue.h", out / "tiny_dnn/core/kernels/b200_glue.h")
    shutil.copyfile(HERE / "b200_backend.h", out / "tiny_dnn/core/b200_backend.h")
    shutil.copyfile(HERE / "b200_net.h", out / "tiny_dnn/core/b200_net.h")
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the tiny-dnn tree")
    ap.add_argument("--out", required=True, help="directory to write the overlay into")
    a = ap.parse_args()
    print(make_overlay(Path(a.reference), Path(a.out)))


if __name__ == "__main__":
    main()
