"""ctypes binding of the C ABI declared in include/tinycnn_b200.h.

The library is the product's only compute path: if it cannot be loaded this
module raises, it never substitutes a CPU implementation.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "csrc" / "libtinycnn_b200.so"


class B200Error(RuntimeError):
    """A C ABI call returned a non-zero status (text from b200_last_error)."""


class ConvDesc(C.Structure):
    """b200_conv_desc: mirror of core::conv_params (tiny_dnn/core/params/conv_params.h:63-90)."""
    _fields_ = [
        ("in_w", C.c_int32), ("in_h", C.c_int32), ("in_c", C.c_int32),
        ("inp_w", C.c_int32), ("inp_h", C.c_int32),
        ("out_w", C.c_int32), ("out_h", C.c_int32), ("out_c", C.c_int32),
        ("k_w", C.c_int32), ("k_h", C.c_int32),
        ("stride_w", C.c_int32), ("stride_h", C.c_int32),
        ("dil_w", C.c_int32), ("dil_h", C.c_int32),
        ("has_bias", C.c_int32), ("pad_same", C.c_int32),
        ("input_is_padded", C.c_int32), ("algo", C.c_int32),
        ("tbl", C.POINTER(C.c_uint8)),
    ]


class PoolDesc(C.Structure):
    """b200_pool_desc: mirror of core::maxpool_params (tiny_dnn/core/params/maxpool_params.h:17-34)."""
    _fields_ = [
        ("in_w", C.c_int32), ("in_h", C.c_int32), ("in_c", C.c_int32),
        ("out_w", C.c_int32), ("out_h", C.c_int32),
        ("pool_w", C.c_int32), ("pool_h", C.c_int32),
        ("stride_w", C.c_int32), ("stride_h", C.c_int32),
    ]


class OptHyper(C.Structure):
    """b200_opt_hyper: public members of adagrad/adam/momentum (tiny_dnn/optimizers/optimizer.h)."""
    _fields_ = [
        ("alpha", C.c_float), ("b1", C.c_float), ("b2", C.c_float),
        ("b1_t", C.c_float), ("b2_t", C.c_float),
        ("mu", C.c_float), ("lambda_", C.c_float), ("eps", C.c_float),
    ]


class ImageDesc(C.Structure):
    """b200_image_desc: how uint8 pixels become the first layer's float rows
    (tiny_dnn/io/cifar10_parser.h:26-86, tiny_dnn/io/mnist_parser.h:43-68)."""
    _fields_ = [
        ("mode", C.c_int32), ("channels", C.c_int32), ("height", C.c_int32), ("width", C.c_int32),
        ("x_padding", C.c_int32), ("y_padding", C.c_int32),
        ("scale_min", C.c_float), ("scale_max", C.c_float),
    ]


IMAGE_CIFAR10, IMAGE_MNIST = 0, 1


class LayerSpec(C.Structure):
    """b200_layer_spec: one layer of a network<sequential>."""
    _fields_ = [
        ("kind", C.c_int32),
        ("conv", ConvDesc),
        ("pool", PoolDesc),
        ("fc_in", C.c_int32), ("fc_out", C.c_int32), ("fc_has_bias", C.c_int32),
        ("act_param", C.c_float),
        ("bn_channels", C.c_int32), ("bn_spatial", C.c_int32),
        ("bn_eps", C.c_float), ("bn_momentum", C.c_float),
    ]


# enums of the header
ACT_NONE, ACT_RELU, ACT_TANH, ACT_SOFTMAX, ACT_SIGMOID, ACT_LEAKY_RELU, ACT_ELU = range(7)
LOSS_MSE, LOSS_CROSS_ENTROPY, LOSS_CROSS_ENTROPY_MULTICLASS = 0, 1, 2
OPT_ADAGRAD, OPT_ADAM, OPT_MOMENTUM, OPT_RMSPROP, OPT_ADAMAX, OPT_GRADIENT_DESCENT, OPT_NESTEROV_MOMENTUM = range(7)
(LAYER_CONV, LAYER_FC, LAYER_MAXPOOL, LAYER_AVGPOOL, LAYER_RELU, LAYER_TANH, LAYER_SOFTMAX, LAYER_SIGMOID,
 LAYER_LEAKY_RELU, LAYER_ELU, LAYER_BATCHNORM) = range(1, 12)

_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
_cd, _pd, _oh = C.POINTER(ConvDesc), C.POINTER(PoolDesc), C.POINTER(OptHyper)

# name -> (restype, argtypes); every symbol the header declares
SIGNATURES = {
    "b200_version": (C.c_char_p, []),
    "b200_last_error": (C.c_char_p, []),
    "b200_device_count": (_i, []),
    "b200_launch_count": (C.c_ulonglong, []),
    "b200_ctx_create": (_i, [_i, _vp, C.POINTER(_vp)]),
    "b200_ctx_destroy": (_i, [_vp]),
    "b200_ctx_set_stream": (_i, [_vp, _vp]),
    "b200_ctx_set_option": (_i, [_vp, C.c_char_p, _i]),
    "b200_ctx_stream": (_vp, [_vp]),
    "b200_ctx_sync": (_i, [_vp]),
    "b200_host_alloc": (_i, [_sz, C.POINTER(_vp)]),
    "b200_host_free": (_i, [_vp]),
    "b200_malloc": (_i, [_vp, _sz, C.POINTER(_vp)]),
    "b200_free": (_i, [_vp, _vp]),
    "b200_memcpy_h2d": (_i, [_vp, _vp, _vp, _sz]),
    "b200_memcpy_d2h": (_i, [_vp, _vp, _vp, _sz]),
    "b200_memset": (_i, [_vp, _vp, _i, _sz]),
    "b200_conv_desc_init": (_i, [_cd] + [_i] * 12),
    "b200_conv2d_fwd": (_i, [_vp, _cd, _vp, _vp, _vp, _vp, _i]),
    "b200_conv2d_bwd": (_i, [_vp, _cd, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "b200_conv2d_dw_noalloc": (_i, [_vp, _cd, _vp, _vp, _vp, _vp, _i, _i]),
    "b200_conv2d_time_pass": (_i, [_vp, _cd, _vp, _vp, _vp, _i, _i, _i, C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "b200_conv2d_fwd_host": (_i, [_vp, _cd, _vp, _vp, _vp, _vp, _i]),
    "b200_conv2d_bwd_host": (_i, [_vp, _cd, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "b200_fc_fwd": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i]),
    "b200_fc_bwd": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "b200_fc_fwd_host": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i]),
    "b200_fc_bwd_host": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "b200_pool_desc_init": (_i, [_pd] + [_i] * 9),
    "b200_maxpool_fwd": (_i, [_vp, _pd, _vp, _vp, _vp, _i]),
    "b200_maxpool_bwd": (_i, [_vp, _pd, _vp, _vp, _vp, _i]),
    "b200_maxpool_fwd_host": (_i, [_vp, _pd, _vp, _vp, _vp, _i]),
    "b200_maxpool_bwd_host": (_i, [_vp, _pd, _vp, _vp, _vp, _i]),
    "b200_avgpool_fwd": (_i, [_vp, _pd, _vp, _vp, _vp, _vp, _i]),
    "b200_avgpool_bwd": (_i, [_vp, _pd, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "b200_avgpool_fwd_host": (_i, [_vp, _pd, _vp, _vp, _vp, _vp, _i]),
    "b200_avgpool_bwd_host": (_i, [_vp, _pd, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "b200_act_fwd": (_i, [_vp, _i, _vp, _vp, _i, _i]),
    "b200_act_bwd": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i]),
    "b200_act_param_fwd": (_i, [_vp, _i, C.c_float, _vp, _vp, _i, _i]),
    "b200_act_param_bwd": (_i, [_vp, _i, C.c_float, _vp, _vp, _vp, _i, _i]),
    "b200_act_param_fwd_host": (_i, [_vp, _i, C.c_float, _vp, _vp, _i, _i]),
    "b200_act_param_bwd_host": (_i, [_vp, _i, C.c_float, _vp, _vp, _vp, _i, _i]),
    "b200_act_fwd_host": (_i, [_vp, _i, _vp, _vp, _i, _i]),
    "b200_act_bwd_host": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i]),
    "b200_qconv2d_eq_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "b200_qfc_eq_fwd": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "b200_qconv2d_eq_fwd_host": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "b200_qfc_eq_fwd_host": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "b200_net_set_phase": (_i, [_vp, _i]),
    "b200_net_set_input_grad": (_i, [_vp, _i]),
    "b200_net_bn_stats": (_i, [_vp, _i, _vp, _vp, _i]),
    "b200_batchnorm_fwd": (_i, [_vp, _i, _i, C.c_float, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "b200_batchnorm_bwd": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i]),
    "b200_batchnorm_post_update": (_i, [_vp, _i, C.c_float, _vp, _vp, _vp, _vp]),
    "b200_batchnorm_fwd_host": (_i, [_vp, _i, _i, C.c_float, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "b200_batchnorm_bwd_host": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i]),
    "b200_dropout": (_i, [_vp, _vp, _vp, C.c_float, _vp, C.c_longlong]),
    "b200_dropout_host": (_i, [_vp, _vp, _vp, C.c_float, _vp, C.c_longlong]),
    "b200_lrn_fwd": (_i, [_vp, _vp, _vp, _i, _i, _i, C.c_float, C.c_float, _i]),
    "b200_lrn_fwd_host": (_i, [_vp, _vp, _vp, _i, _i, _i, C.c_float, C.c_float, _i]),
    "b200_loss_grad": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i]),
    "b200_loss_value": (_i, [_vp, _i, _vp, _vp, _vp, _i, _i]),
    "b200_merge_grads": (_i, [_vp, _vp, _i, _sz, _vp]),
    "b200_opt_update": (_i, [_vp, _i, _oh, _vp, _vp, _vp, _vp, _sz]),
    "b200_merge_update": (_i, [_vp, _i, _oh, _vp, _i, _sz, _vp, _vp, _vp, _vp, _sz]),
    "b200_qconv2d_fwd": (_i, [_vp, _cd, _vp, _vp, _vp, _vp, _i]),
    "b200_qfc_fwd": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i]),
    "b200_qconv2d_fwd_host": (_i, [_vp, _cd, _vp, _vp, _vp, _vp, _i]),
    "b200_qfc_fwd_host": (_i, [_vp, _i, _i, _vp, _vp, _vp, _vp, _i]),
    "b200_net_create": (_i, [_vp, C.POINTER(LayerSpec), _i, _i, C.POINTER(_vp)]),
    "b200_net_destroy": (_i, [_vp]),
    "b200_net_param_count": (_sz, [_vp]),
    "b200_net_tensor_count": (_i, [_vp]),
    "b200_net_tensor_info": (_i, [_vp, _i, C.POINTER(_sz), C.POINTER(_sz)]),
    "b200_net_in_dim": (_i, [_vp]),
    "b200_net_out_dim": (_i, [_vp]),
    "b200_net_set_params": (_i, [_vp, _vp]),
    "b200_net_get_params": (_i, [_vp, _vp]),
    "b200_net_get_grads": (_i, [_vp, _vp]),
    "b200_net_params_ptr": (_vp, [_vp]),
    "b200_net_grads_ptr": (_vp, [_vp]),
    "b200_net_output_ptr": (_vp, [_vp]),
    "b200_net_layer_out_ptr": (_vp, [_vp, _i]),
    "b200_net_layer_grad_ptr": (_vp, [_vp, _i]),
    "b200_net_forward": (_i, [_vp, _vp, _i]),
    "b200_net_backward": (_i, [_vp, _vp, _i]),
    "b200_net_opt_reset": (_i, [_vp, _i]),
    "b200_net_update": (_i, [_vp, _i, _oh]),
    "b200_net_train_step": (_i, [_vp, _vp, _vp, _i, _i, _i, _oh]),
    "b200_net_forward_backward": (_i, [_vp, _vp, _vp, _i, _i]),
    "b200_net_peer_reduce_bytes": (_sz, [_vp, _i]),
    "b200_net_peer_reduce_init": (_i, [_vp, _i, _i, C.POINTER(C.c_ulonglong), _i]),
    "b200_net_peer_reduce": (_i, [_vp]),
    "b200_net_peer_push": (_i, [_vp]),
    "b200_net_peer_sum": (_i, [_vp]),
    "b200_peer_buffer_create": (_i, [_vp, _sz, _vp, _vp]),
    "b200_peer_buffer_open": (_i, [_vp, _vp, _vp]),
    "b200_peer_buffer_close": (_i, [_vp, _vp]),
    "b200_peer_buffer_destroy": (_i, [_vp, _vp]),
    "b200_net_train_step_host": (_i, [_vp, _vp, _vp, _i, _i, _i, _oh, _vp]),
    "b200_net_fit_host": (_i, [_vp, _vp, _vp, C.c_longlong, _i, _i, _i, _i, _oh, _vp]),
    "b200_net_fit_host_enqueue": (_i, [_vp, _vp, _vp, C.c_longlong, _i, _i, _i, _i, _oh, _vp]),
    "b200_net_fit_host_wait": (_i, [_vp]),
    "b200_images_u8_to_float": (_i, [_vp, C.POINTER(ImageDesc), _vp, C.c_longlong, _vp]),
    "b200_labels_to_targets": (_i, [_vp, _vp, C.c_longlong, _i, C.c_float, C.c_float, _vp]),
    "b200_net_fit_u8_host": (_i, [_vp, C.POINTER(ImageDesc), _vp, _vp, C.c_longlong, _i, _i, C.c_float, C.c_float,
                                  _i, _i, _oh, _vp]),
    "b200_net_adam_powers": (_i, [_vp, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "b200_net_get_opt_state": (_i, [_vp, _i, _vp]),
    "b200_net_set_opt_state": (_i, [_vp, _i, _vp]),
    "b200_net_set_adam_powers": (_i, [_vp, C.c_float, C.c_float, C.c_float, C.c_float]),
}

_lib = None


def load() -> C.CDLL:
    """Load the native library (once) and type every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    path = Path(os.environ.get("TINYCNN_B200_LIB", LIB_PATH))
    if not path.exists():
        raise B200Error(
            f"native library {path} is missing; build it with "
            "`python -m tiny_cnn_b200.build` (there is no CPU fallback)")
    lib = C.CDLL(str(path))
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(status: int) -> None:
    if status != 0:
        msg = load().b200_last_error().decode("utf-8", "replace")
        raise B200Error(f"status {status}: {msg}")


def ptr(x):
    """Device/host address of a torch tensor, numpy array, int or None as c_void_p."""
    if x is None:
        return None
    if isinstance(x, int):
        return C.c_void_p(x)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    if hasattr(x, "ctypes"):
        return C.c_void_p(x.ctypes.data)
    raise TypeError(f"cannot take the address of {type(x)}")
