"""Generate the tiny-dnn overlay that adds the engine `core::backend_t::b200`.

tiny-dnn is header-only, so the new engine is delivered as an include directory
placed BEFORE the tiny-dnn tree on the compiler's include path:

    g++ -std=c++14 -I <overlay> -I <tiny-dnn> -I <repo>/include app.cpp \
        -L <repo>/tiny_cnn_b200/csrc -ltinycnn_b200

The overlay holds patched copies of exactly the headers that carry the backend
switch, produced here from the user's own tiny-dnn tree by anchored text edits
(nothing of tiny-dnn is stored in this repository), plus the two headers of this
directory (b200_glue.h, b200_backend.h) under tiny_dnn/core/kernels/ and
tiny_dnn/core/.  Every edit asserts that its anchor is present, so a tiny-dnn
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


def patch_conv_layer(t, p):
    # the same Conv2dOp / Conv2dGradOp objects serve the new engine, so that
    # layer::set_backend_type() can switch engines at run time
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
    return _edit(t, "    if (backend_type == core::backend_t::internal ||\n"
                    "        backend_type == core::backend_t::avx ||",
                 "    if (backend_type == core::backend_t::internal ||\n"
                 "        backend_type == core::backend_t::b200 ||\n"
                 "        backend_type == core::backend_t::avx ||", p)


def patch_maxpool_layer(t, p):
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
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of the tiny-dnn tree")
    ap.add_argument("--out", required=True, help="directory to write the overlay into")
    a = ap.parse_args()
    print(make_overlay(Path(a.reference), Path(a.out)))


if __name__ == "__main__":
    main()
