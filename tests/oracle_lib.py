"""ctypes bindings of the test oracle (oracle/liboracle.so) and of the compiled
reference (oracle/_ref/libtinydnn_ref.so).  Test infrastructure only."""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

from tiny_cnn_b200._lib import ConvDesc, ImageDesc, LayerSpec, OptHyper, PoolDesc  # noqa: E402

_vp, _i, _sz, _f = C.c_void_p, C.c_int, C.c_size_t, C.c_float
_cd, _pd, _oh = C.POINTER(ConvDesc), C.POINTER(PoolDesc), C.POINTER(OptHyper)
_fp = C.POINTER(C.c_float)

ORACLE_SIGS = {
    "orc_conv_pad": (None, [_cd, _vp, _vp, _i]),
    "orc_conv_unpad": (None, [_cd, _vp, _vp, _i]),
    "orc_conv2d_fwd": (None, [_cd, _vp, _vp, _vp, _vp, _i]),
    "orc_conv2d_bwd": (None, [_cd, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "orc_fc_fwd": (None, [_i, _i, _vp, _vp, _vp, _vp, _i]),
    "orc_fc_bwd": (None, [_i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "orc_maxpool_fwd": (None, [_pd, _vp, _vp, _vp, _i]),
    "orc_maxpool_bwd": (None, [_pd, _vp, _vp, _vp, _i]),
    "orc_avgpool_fwd": (None, [_pd, _vp, _vp, _vp, _vp, _i]),
    "orc_avgpool_bwd": (None, [_pd, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "orc_qconv2d_eq_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "orc_qfc_eq_fwd": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "orc_net_set_phase": (None, [_vp, _i]),
    "orc_net_bn_mean": (C.POINTER(C.c_float), [_vp, _i]),
    "orc_net_bn_var": (C.POINTER(C.c_float), [_vp, _i]),
    "orc_batchnorm_fwd": (None, [_i, _i, C.c_float, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "orc_batchnorm_bwd": (None, [_i, _i, _vp, _vp, _vp, _vp, _i]),
    "orc_batchnorm_post_update": (None, [_i, C.c_float, _vp, _vp, _vp, _vp]),
    "orc_dropout": (None, [_vp, _vp, C.c_float, _vp, C.c_longlong]),
    "orc_lrn_fwd": (None, [_vp, _vp, _i, _i, _i, C.c_float, C.c_float, _i]),
    "orc_act_param_fwd": (None, [_i, C.c_float, _vp, _vp, _i, _i]),
    "orc_act_param_bwd": (None, [_i, C.c_float, _vp, _vp, _vp, _i, _i]),
    "orc_act_fwd": (None, [_i, _vp, _vp, _i, _i]),
    "orc_act_bwd": (None, [_i, _vp, _vp, _vp, _i, _i]),
    "orc_loss_grad": (None, [_i, _vp, _vp, _vp, _i, _i]),
    "orc_loss_value": (_f, [_i, _vp, _vp, _i, _i]),
    "orc_merge_grads": (None, [_vp, _i, _sz, _vp]),
    "orc_opt_update": (None, [_i, _oh, _vp, _vp, _vp, _vp, _sz]),
    "orc_f2q_unclamped": (C.c_int64, [_i, _f, _f, _f]),
    "orc_f2q": (C.c_int64, [_i, _f, _f, _f]),
    "orc_q2f": (_f, [_i, C.c_int64, _f, _f]),
    "orc_range_for_multiplication": (None, [_f, _f, _f, _f, _fp, _fp]),
    "orc_requantize_in_new_range": (C.c_int64, [_i, _i, C.c_int64, _f, _f, _f, _f]),
    "orc_requantize_many_i32_u8": (None, [_vp, _sz, _f, _f, _f, _f, _vp]),
    "orc_quantize_down_and_shrink_range": (None, [_vp, _sz, _f, _f, _fp, _fp, _vp]),
    "orc_qconv2d_fwd": (_i, [_cd, _vp, _vp, _vp, _vp, _i, _vp, _vp]),
    "orc_qfc_fwd": (_i, [_i, _i, _vp, _vp, _vp, _vp, _i]),
    "orc_net_create": (_vp, [C.POINTER(LayerSpec), _i, _i]),
    "orc_net_destroy": (None, [_vp]),
    "orc_net_param_count": (_sz, [_vp]),
    "orc_net_params": (_fp, [_vp]),
    "orc_net_grads": (_fp, [_vp]),
    "orc_net_output": (_fp, [_vp]),
    "orc_net_layer_out": (_fp, [_vp, _i]),
    "orc_net_layer_grad": (_fp, [_vp, _i]),
    "orc_net_forward": (None, [_vp, _vp, _i]),
    "orc_net_backward": (None, [_vp, _vp, _vp, _i, _i]),
    "orc_net_update": (None, [_vp, _i, _oh]),
    "orc_net_adam_powers": (None, [_vp, _fp, _fp]),
    "orc_net_opt_reset": (None, [_vp, _i]),
    "orc_net_fit": (_i, [_vp, _vp, _vp, C.c_longlong, _i, _i, _i, _i, _oh]),
    "orc_images_u8_to_float": (None, [C.POINTER(ImageDesc), _vp, C.c_longlong, _vp]),
    "orc_labels_to_targets": (None, [_vp, C.c_longlong, _i, _f, _f, _vp]),
    "orc_net_train_step": (None, [_vp, _vp, _vp, _i, _i, _i, _oh]),
}

REF_SIGS = {
    "ref_version": (C.c_char_p, []),
    "ref_openmp_threads": (_i, []),
    "ref_set_threads": (_i, [_i]),
    "ref_conv2d_fwd": (_i, [_cd, _vp, _vp, _vp, _vp, _i]),
    "ref_conv2d_bwd": (_i, [_cd, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "ref_fc_fwd": (_i, [_i, _i, _vp, _vp, _vp, _vp, _i]),
    "ref_fc_bwd": (_i, [_i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "ref_maxpool_fwd_bwd": (_i, [_pd, _i, _i, _vp, _vp, _vp, _vp, _i]),
    "ref_avgpool_fwd_bwd": (_i, [_pd, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "ref_act_fwd_bwd": (_i, [_i, _vp, _vp, _vp, _vp, _i, _i]),
    "ref_qconv2d_eq_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "ref_qfc_eq_fwd": (_i, [_i, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i]),
    "ref_net_bn_stats": (_i, [_vp, _i, _vp, _vp]),
    "ref_batchnorm_fwd_bwd": (_i, [_i, _i, C.c_float, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i]),
    "ref_lrn_fwd": (_i, [_vp, _vp, _i, _i, _i, _i, C.c_float, C.c_float, _i]),
    "ref_dropout_fwd_bwd": (_i, [_i, C.c_float, _vp, _vp, _vp, _vp, _vp, _i]),
    "ref_act_param_fwd_bwd": (_i, [_i, C.c_float, _vp, _vp, _vp, _vp, _i, _i]),
    "ref_loss_grad": (_i, [_i, _vp, _vp, _vp, _i, _i]),
    "ref_opt_steps": (_i, [_i, _oh, _vp, _vp, _sz, _i]),
    "ref_f2q_unclamped": (C.c_int64, [_i, _f, _f, _f]),
    "ref_f2q": (C.c_int64, [_i, _f, _f, _f]),
    "ref_q2f": (_f, [_i, C.c_int64, _f, _f]),
    "ref_requantize_many_i32_u8": (None, [_vp, _sz, _f, _f, _f, _f, _vp]),
    "ref_quantize_down_and_shrink_range": (None, [_vp, _sz, _f, _f, _fp, _fp, _vp]),
    "ref_qconv2d_fwd": (_i, [_cd, _vp, _vp, _vp, _vp, _i]),
    "ref_qfc_fwd": (_i, [_i, _i, _vp, _vp, _vp, _vp, _i]),
    "ref_net_create": (_vp, [C.POINTER(LayerSpec), _i, C.c_uint]),
    "ref_net_destroy": (None, [_vp]),
    "ref_net_param_count": (_sz, [_vp]),
    "ref_net_get_params": (None, [_vp, _vp]),
    "ref_net_set_params": (None, [_vp, _vp]),
    "ref_net_predict": (_i, [_vp, _vp, _vp, _i]),
    "ref_net_fit": (C.c_double, [_vp, _vp, _vp, _i, _i, _i, _i, _oh]),
    "ref_net_fit_n": (C.c_double, [_vp, _vp, _vp, C.c_longlong, _i, _i, _i, _i, _oh]),
    "ref_net_adam_powers": (None, [_vp, _fp, _fp]),
    "ref_parse_cifar10": (C.c_longlong, [C.c_char_p, _f, _f, _i, _i, _vp, _vp, C.c_longlong]),
    "ref_parse_mnist_images": (C.c_longlong, [C.c_char_p, _f, _f, _i, _i, _vp, C.c_longlong]),
    "ref_net_label_targets": (_i, [_vp, _vp, C.c_longlong, _vp, _vp]),
    "ref_net_grads_chunked": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp]),
    "ref_net_apply_update": (_i, [_vp, _vp, _i, _oh]),
    "ref_time_conv": (C.c_double, [_cd, _vp, _vp, _vp, _vp, _i, _i, _i]),
}


def _bind(path: Path, sigs):
    lib = C.CDLL(str(path))
    for name, (res, args) in sigs.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


_oracle = None
_ref = None


def load_oracle():
    global _oracle
    if _oracle is None:
        path = ROOT / "oracle" / "liboracle.so"
        if not path.exists():
            sys.path.insert(0, str(ROOT / "oracle"))
            import build_oracle
            build_oracle.build_oracle()
        _oracle = _bind(path, ORACLE_SIGS)
    return _oracle


def load_reference():
    """The compiled reference, or None when oracle/_ref has not been built."""
    global _ref
    if _ref is None:
        path = ROOT / "oracle" / "_ref" / "libtinydnn_ref.so"
        if not path.exists():
            return None
        _ref = _bind(path, REF_SIGS)
    return _ref


_ref_avx = None


def load_reference_avx():
    """The reference compiled with its AVX kernels and backend_t::avx (timed only), or None."""
    global _ref_avx
    if _ref_avx is None:
        path = ROOT / "oracle" / "_ref" / "libtinydnn_ref_avx.so"
        if not path.exists():
            return None
        sigs = {k: v for k, v in REF_SIGS.items() if k not in ("ref_qfc_fwd", "ref_qfc_eq_fwd")}
        _ref_avx = _bind(path, sigs)
    return _ref_avx


def p(a):
    """c_void_p of a numpy array (or None)."""
    return None if a is None else C.c_void_p(a.ctypes.data)


def f32(*shape):
    return np.zeros(shape, dtype=np.float32)
