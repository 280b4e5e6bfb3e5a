"""Host-side mirror of the reference's operator interface over the C ABI.

Function names follow the reference's op kernels (`Conv2dOp`, `Conv2dGradOp`,
`FullyConnectedOp`, `FullyConnectedGradOp`, `MaxPoolOp`, `MaxPoolGradOp`:
tiny_dnn/core/kernels/*_op.h) and helpers (`conv_params`, `maxpool_params`).
Tensors are torch CUDA tensors used purely as device memory; every function
calls one C ABI entry point and raises `B200Error` on a non-zero status.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import _lib as L
from ._lib import (ACT_NONE, ACT_RELU, ACT_SOFTMAX, ACT_TANH, LOSS_CROSS_ENTROPY,
                   LOSS_CROSS_ENTROPY_MULTICLASS, LOSS_MSE, OPT_ADAGRAD, OPT_ADAM, OPT_MOMENTUM,
                   B200Error, ConvDesc, OptHyper, PoolDesc, check, ptr)


class Context:
    """b200_ctx bound to one GPU; work is issued on torch's current stream of that device.

    The legacy default stream cannot be captured into a CUDA graph, so when torch's
    current stream is the default one a new torch stream is created and made current:
    torch copies and the library's kernels then share one ordered stream."""

    def __init__(self, device: int = 0, stream: Optional[int] = None):
        self.lib = L.load()
        if self.lib.b200_device_count() <= 0:
            raise B200Error("no CUDA device is visible; this library has no CPU path")
        self.device = device
        self.torch_stream = None
        if stream is None:
            ts = torch.cuda.current_stream(device)
            if ts.cuda_stream == 0:
                # above the default priority: the net's side branch (default priority) then yields the
                # SMs to the kernels of this stream, which carry the critical path of a step
                ts = torch.cuda.Stream(device, priority=-1)
                torch.cuda.set_stream(ts)
            self.torch_stream = ts
            stream = ts.cuda_stream
        h = C.c_void_p()
        check(self.lib.b200_ctx_create(device, C.c_void_p(stream), C.byref(h)))
        self.handle = h
        self._tables = []  # keep connection-table arrays alive

    def sync(self) -> None:
        check(self.lib.b200_ctx_sync(self.handle))

    def close(self) -> None:
        if self.handle:
            self.lib.b200_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):  # pragma: no cover - best effort
        try:
            self.close()
        except Exception:
            pass


def conv_params(in_w, in_h, in_c, k_w, k_h, out_c, pad_same=False, has_bias=True, stride_w=1,
                stride_h=1, dil_w=1, dil_h=1, table: Optional[np.ndarray] = None, algo=0,
                input_is_padded=False) -> ConvDesc:
    """Descriptor filled like convolutional_layer::conv_set_params
    (tiny_dnn/layers/convolutional_layer.h:404-438).  `table` is a bool/uint8 array
    [in_c][out_c] (connection_table rows = inputs, cols = outputs)."""
    d = ConvDesc()
    check(L.load().b200_conv_desc_init(C.byref(d), in_w, in_h, in_c, k_w, k_h, out_c, int(pad_same),
                                       int(has_bias), stride_w, stride_h, dil_w, dil_h))
    d.algo = algo
    d.input_is_padded = int(input_is_padded)
    if table is not None:
        t = np.ascontiguousarray(np.asarray(table, dtype=np.uint8).reshape(in_c, out_c))
        d._table_keepalive = t
        d.tbl = t.ctypes.data_as(C.POINTER(C.c_uint8))
    return d


def maxpool_params(in_w, in_h, in_c, pool_w, pool_h=None, stride_w=None, stride_h=None,
                   ceil_mode=False, pad_same=False) -> PoolDesc:
    """Descriptor with the output size of pool_out_length (tiny_dnn/util/util.h:346-363)."""
    pool_h = pool_w if pool_h is None else pool_h
    stride_w = pool_w if stride_w is None else stride_w
    stride_h = pool_h if stride_h is None else stride_h
    d = PoolDesc()
    check(L.load().b200_pool_desc_init(C.byref(d), in_w, in_h, in_c, pool_w, pool_h, stride_w,
                                       stride_h, int(ceil_mode), int(pad_same)))
    return d


def hyper(alpha=0.01, b1=0.9, b2=0.999, b1_t=0.9, b2_t=0.999, mu=0.9, lambda_=0.0,
          eps=1e-8) -> OptHyper:
    return OptHyper(alpha, b1, b2, b1_t, b2_t, mu, lambda_, eps)


def _f32(*shape, device):
    return torch.empty(*shape, dtype=torch.float32, device=device)


def conv_in_len(d: ConvDesc) -> int:
    padded = d.input_is_padded or not d.pad_same
    return d.in_c * (d.inp_h * d.inp_w if padded else d.in_h * d.in_w)


def conv_out_len(d: ConvDesc) -> int:
    return d.out_c * d.out_h * d.out_w


def conv_w_len(d: ConvDesc) -> int:
    return d.out_c * d.in_c * d.k_h * d.k_w


# --------------------------------------------------------------------------- convolution
def conv2d_op(ctx: Context, d: ConvDesc, x, W, bias, out=None):
    """Conv2dOp::compute (tiny_dnn/core/kernels/conv2d_op.h:23-51)."""
    B = x.shape[0]
    out = _f32(B, conv_out_len(d), device=x.device) if out is None else out
    check(ctx.lib.b200_conv2d_fwd(ctx.handle, C.byref(d), ptr(x), ptr(W), ptr(bias), ptr(out), B))
    return out


def conv2d_grad_op(ctx: Context, d: ConvDesc, x, W, dout, need_dx=True, dW=None, db=None,
                   accumulate=False):
    """Conv2dGradOp::compute (tiny_dnn/core/kernels/conv2d_grad_op.h:22-50); returns
    (dx, dW, db) with dW/db summed over the batch."""
    B = x.shape[0]
    dx = _f32(B, conv_in_len(d), device=x.device) if need_dx else None
    dW = torch.zeros(conv_w_len(d), dtype=torch.float32, device=x.device) if dW is None else dW
    if d.has_bias and db is None:
        db = torch.zeros(d.out_c, dtype=torch.float32, device=x.device)
    check(ctx.lib.b200_conv2d_bwd(ctx.handle, C.byref(d), ptr(x), ptr(W), ptr(dout), ptr(dx),
                                  ptr(dW), ptr(db), int(accumulate), B))
    return dx, dW, db


# --------------------------------------------------------------------------- fully connected
def fully_connected_op(ctx: Context, in_size, out_size, x, W, bias, out=None):
    """FullyConnectedOp::compute (tiny_dnn/core/kernels/fully_connected_op.h:25-64)."""
    B = x.shape[0]
    out = _f32(B, out_size, device=x.device) if out is None else out
    check(ctx.lib.b200_fc_fwd(ctx.handle, in_size, out_size, ptr(x), ptr(W), ptr(bias), ptr(out), B))
    return out


def fully_connected_grad_op(ctx: Context, in_size, out_size, x, W, dout, has_bias=True,
                            need_dx=True, dW=None, db=None, accumulate=False):
    """FullyConnectedGradOp::compute (tiny_dnn/core/kernels/fully_connected_grad_op.h:22-52)."""
    B = x.shape[0]
    dx = _f32(B, in_size, device=x.device) if need_dx else None
    dW = torch.zeros(in_size * out_size, dtype=torch.float32, device=x.device) if dW is None else dW
    if has_bias and db is None:
        db = torch.zeros(out_size, dtype=torch.float32, device=x.device)
    check(ctx.lib.b200_fc_bwd(ctx.handle, in_size, out_size, ptr(x), ptr(W), ptr(dout), ptr(dx),
                              ptr(dW), ptr(db), int(accumulate), B))
    return dx, dW, db


# --------------------------------------------------------------------------- pooling
def maxpool_op(ctx: Context, d: PoolDesc, x):
    """MaxPoolOp::compute (tiny_dnn/core/kernels/maxpool_op.h:23-61); returns (out, argmax)."""
    B = x.shape[0]
    n = d.in_c * d.out_h * d.out_w
    out = _f32(B, n, device=x.device)
    arg = torch.empty(B, n, dtype=torch.int32, device=x.device)
    check(ctx.lib.b200_maxpool_fwd(ctx.handle, C.byref(d), ptr(x), ptr(out), ptr(arg), B))
    return out, arg


def maxpool_grad_op(ctx: Context, d: PoolDesc, dout, argmax):
    """MaxPoolGradOp::compute (tiny_dnn/core/kernels/maxpool_grad_op.h:22-47)."""
    B = dout.shape[0]
    dx = _f32(B, d.in_c * d.in_h * d.in_w, device=dout.device)
    check(ctx.lib.b200_maxpool_bwd(ctx.handle, C.byref(d), ptr(dout), ptr(argmax), ptr(dx), B))
    return dx


def average_pooling_forward(ctx: Context, d: PoolDesc, x, W, bias):
    """tiny_average_pooling_kernel (tiny_dnn/layers/average_pooling_layer.h:25-55)."""
    B = x.shape[0]
    out = _f32(B, d.in_c * d.out_h * d.out_w, device=x.device)
    check(ctx.lib.b200_avgpool_fwd(ctx.handle, C.byref(d), ptr(x), ptr(W), ptr(bias), ptr(out), B))
    return out


def average_pooling_backward(ctx: Context, d: PoolDesc, x, W, dout, need_dx=True, accumulate=False,
                             dW=None, db=None):
    """tiny_average_pooling_back_kernel (average_pooling_layer.h:58-106)."""
    B = x.shape[0]
    dx = _f32(B, d.in_c * d.in_h * d.in_w, device=x.device) if need_dx else None
    wlen = d.pool_w * d.pool_h * d.in_c
    dW = torch.zeros(wlen, dtype=torch.float32, device=x.device) if dW is None else dW
    db = torch.zeros(d.in_c, dtype=torch.float32, device=x.device) if db is None else db
    check(ctx.lib.b200_avgpool_bwd(ctx.handle, C.byref(d), ptr(x), ptr(W), ptr(dout), ptr(dx),
                                   ptr(dW), ptr(db), int(accumulate), B))
    return dx, dW, db


# --------------------------------------------------------------------------- activations / loss
def forward_activation(ctx: Context, kind: int, x, param=None):
    """activation_layer::forward_propagation (tiny_dnn/activations/activation_layer.h:74-79).
    `param`: epsilon of leaky_relu_layer / alpha of elu_layer (None: the reference's default)."""
    y = torch.empty_like(x)
    if param is None:
        check(ctx.lib.b200_act_fwd(ctx.handle, kind, ptr(x), ptr(y), x.shape[1], x.shape[0]))
    else:
        check(ctx.lib.b200_act_param_fwd(ctx.handle, kind, float(param), ptr(x), ptr(y), x.shape[1], x.shape[0]))
    return y


def backward_activation(ctx: Context, kind: int, y, dy, param=None):
    """activation_layer::back_propagation (activation_layer.h:81-91)."""
    dx = torch.empty_like(y)
    if param is None:
        check(ctx.lib.b200_act_bwd(ctx.handle, kind, ptr(y), ptr(dy), ptr(dx), y.shape[1], y.shape[0]))
    else:
        check(ctx.lib.b200_act_param_bwd(ctx.handle, kind, float(param), ptr(y), ptr(dy), ptr(dx), y.shape[1],
                                         y.shape[0]))
    return dx


# --------------------------------------------------------------------------- batch norm / dropout / lrn
def batch_normalization_forward(ctx: Context, channels: int, spatial: int, eps: float, x, mean=None, variance=None,
                                train=True):
    """batch_normalization_layer::forward_propagation (tiny_dnn/layers/batch_normalization_layer.h:136-168).
    Train phase: returns (y, mean, variance, stddev) of this mini-batch; test phase: `mean` / `variance`
    are the layer's moving averages."""
    B = x.shape[0]
    y = torch.empty_like(x)
    if train:
        mean = torch.empty(channels, device=x.device)
        variance = torch.empty(channels, device=x.device)
    stddev = torch.empty(channels, device=x.device)
    check(ctx.lib.b200_batchnorm_fwd(ctx.handle, channels, spatial, float(eps), ptr(x), ptr(mean), ptr(variance),
                                     ptr(stddev), ptr(y), B, int(train)))
    return y, mean, variance, stddev


def batch_normalization_backward(ctx: Context, channels: int, spatial: int, y, dy, stddev):
    """batch_normalization_layer::back_propagation (batch_normalization_layer.h:94-134)."""
    dx = torch.empty_like(y)
    check(ctx.lib.b200_batchnorm_bwd(ctx.handle, channels, spatial, ptr(y), ptr(dy), ptr(stddev), ptr(dx), y.shape[0]))
    return dx


def dropout(ctx: Context, x, mask, scale: float):
    """dropout_layer with the caller's mask (tiny_dnn/layers/dropout_layer.h:66-115): mask * scale * x."""
    out = torch.empty_like(x)
    check(ctx.lib.b200_dropout(ctx.handle, ptr(x), ptr(mask), float(scale), ptr(out), x.numel()))
    return out


def lrn_forward(ctx: Context, x, channels: int, area: int, size: int, alpha: float, beta: float):
    """lrn_layer::forward_propagation across channels (tiny_dnn/layers/lrn_layer.h:82-143)."""
    out = torch.empty_like(x)
    check(ctx.lib.b200_lrn_fwd(ctx.handle, ptr(x), ptr(out), channels, area, size, float(alpha), float(beta),
                               x.shape[0]))
    return out


def gradient(ctx: Context, loss: int, y, t):
    """gradient<E>(y, t) for a mini-batch (tiny_dnn/lossfunctions/loss_function.h:190-218)."""
    dy = torch.empty_like(y)
    check(ctx.lib.b200_loss_grad(ctx.handle, loss, ptr(y), ptr(t), ptr(dy), y.shape[1], y.shape[0]))
    return dy


def loss_value(ctx: Context, loss: int, y, t):
    out = torch.zeros(1, dtype=torch.float32, device=y.device)
    check(ctx.lib.b200_loss_value(ctx.handle, loss, ptr(y), ptr(t), ptr(out), y.shape[1], y.shape[0]))
    return out


# --------------------------------------------------------------------------- merge + optimizer
def merge_grads(ctx: Context, grads):
    """edge::merge_grads (tiny_dnn/node.h:89-103): grads is [rows][len]."""
    dst = _f32(grads.shape[1], device=grads.device)
    check(ctx.lib.b200_merge_grads(ctx.handle, ptr(grads), grads.shape[0], grads.shape[1], ptr(dst)))
    return dst


def optimizer_update(ctx: Context, kind: int, h: OptHyper, dW, W, state0, state1=None):
    """optimizer::update (tiny_dnn/optimizers/optimizer.h:60-66,112-127,205-213), in place."""
    check(ctx.lib.b200_opt_update(ctx.handle, kind, C.byref(h), ptr(dW), ptr(W), ptr(state0),
                                  ptr(state1), W.numel()))


def merge_update(ctx: Context, kind: int, h: OptHyper, grads, W, state0, state1=None, merged=None):
    """merge_grads + optimizer::update of layer::update_weight (tiny_dnn/layers/layer.h:663-682)."""
    check(ctx.lib.b200_merge_update(ctx.handle, kind, C.byref(h), ptr(grads), grads.shape[0],
                                    grads.shape[1], ptr(merged), ptr(W), ptr(state0), ptr(state1),
                                    W.numel()))


# --------------------------------------------------------------------------- quantized
def quantized_conv2d(ctx: Context, d: ConvDesc, x_padded, W, bias):
    """tiny_backend::conv2d_q (tiny_dnn/core/backend_tiny.h:97-112); x has in_padded geometry."""
    B = x_padded.shape[0]
    out = _f32(B, conv_out_len(d), device=x_padded.device)
    check(ctx.lib.b200_qconv2d_fwd(ctx.handle, C.byref(d), ptr(x_padded), ptr(W), ptr(bias),
                                   ptr(out), B))
    return out


def quantized_fully_connected(ctx: Context, in_size, out_size, x, W, bias):
    """tiny_backend::fully_q (tiny_dnn/core/backend_tiny.h:300-319)."""
    B = x.shape[0]
    out = _f32(B, out_size, device=x.device)
    check(ctx.lib.b200_qfc_fwd(ctx.handle, in_size, out_size, ptr(x), ptr(W), ptr(bias), ptr(out), B))
    return out
