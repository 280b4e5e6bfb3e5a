"""Host-side mirror of `network<sequential>` driving the device-resident step.

`Sequential` is built with `<<`-style calls named after the reference's layer
classes (tiny_dnn/layers/*.h) and trained with `fit` / `train_onebatch`
(tiny_dnn/network.h:840-926).  All arithmetic happens in the native library;
this class only carries descriptors, pointers and the optimizer's public
hyper-parameters.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence

import numpy as np
import torch

from . import _lib as L
from ._lib import (LAYER_AVGPOOL, LAYER_BATCHNORM, LAYER_CONV, LAYER_ELU, LAYER_FC, LAYER_LEAKY_RELU, LAYER_MAXPOOL, LAYER_RELU,
                   LAYER_SIGMOID, LAYER_SOFTMAX,
                   LAYER_TANH, LOSS_CROSS_ENTROPY, LOSS_MSE, OPT_ADAGRAD, OPT_ADAM, OPT_ADAMAX, OPT_GRADIENT_DESCENT,
                   OPT_MOMENTUM, OPT_NESTEROV_MOMENTUM, OPT_RMSPROP,
                   LayerSpec, OptHyper, check, ptr)
from .ops import Context, conv_params, hyper, maxpool_params


class DevicePtr:
    """Wraps a raw device pointer so torch can alias it (CUDA array interface)."""

    def __init__(self, address: int, n: int, typestr: str = "<f4"):
        self.__cuda_array_interface__ = {
            "shape": (n,), "typestr": typestr, "data": (address, False), "version": 2,
        }


# --- optimizers: the public members of the reference classes --------------------------
class adagrad:
    """tiny_dnn/optimizers/optimizer.h:57-71"""
    kind = OPT_ADAGRAD

    def __init__(self, alpha=0.01):
        self.alpha = alpha

    def hyper(self) -> OptHyper:
        return hyper(alpha=self.alpha)


class adam:
    """tiny_dnn/optimizers/optimizer.h:103-137"""
    kind = OPT_ADAM

    def __init__(self, alpha=0.001, b1=0.9, b2=0.999):
        self.alpha, self.b1, self.b2 = alpha, b1, b2

    def hyper(self) -> OptHyper:
        return hyper(alpha=self.alpha, b1=self.b1, b2=self.b2)


class momentum:
    """tiny_dnn/optimizers/optimizer.h:201-218"""
    kind = OPT_MOMENTUM

    def __init__(self, alpha=0.01, mu=0.9, lambda_=0.0):
        self.alpha, self.mu, self.lambda_ = alpha, mu, lambda_

    def hyper(self) -> OptHyper:
        return hyper(alpha=self.alpha, mu=self.mu, lambda_=self.lambda_)


class RMSprop:
    """tiny_dnn/optimizers/optimizer.h:79-95"""
    kind = OPT_RMSPROP

    def __init__(self, alpha=0.0001, mu=0.99):
        self.alpha, self.mu = alpha, mu

    def hyper(self) -> OptHyper:
        return hyper(alpha=self.alpha, mu=self.mu)


class adamax:
    """tiny_dnn/optimizers/optimizer.h:145-175"""
    kind = OPT_ADAMAX

    def __init__(self, alpha=0.002, b1=0.9, b2=0.999):
        self.alpha, self.b1, self.b2 = alpha, b1, b2

    def hyper(self) -> OptHyper:
        return hyper(alpha=self.alpha, b1=self.b1, b2=self.b2)


class gradient_descent:
    """tiny_dnn/optimizers/optimizer.h:182-193"""
    kind = OPT_GRADIENT_DESCENT

    def __init__(self, alpha=0.01, lambda_=0.0):
        self.alpha, self.lambda_ = alpha, lambda_

    def hyper(self) -> OptHyper:
        return hyper(alpha=self.alpha, lambda_=self.lambda_)


class nesterov_momentum:
    """tiny_dnn/optimizers/optimizer.h:227-245"""
    kind = OPT_NESTEROV_MOMENTUM

    def __init__(self, alpha=0.01, mu=0.9, lambda_=0.0):
        self.alpha, self.mu, self.lambda_ = alpha, mu, lambda_

    def hyper(self) -> OptHyper:
        return hyper(alpha=self.alpha, mu=self.mu, lambda_=self.lambda_)


class Sequential:
    """network<sequential> (tiny_dnn/network.h, tiny_dnn/nodes.h:268-360) on one GPU."""

    def __init__(self, device: int = 0):
        self.device = device
        self.specs: List[LayerSpec] = []
        self._keep = []
        self.ctx: Optional[Context] = None
        self.handle = None
        self.max_batch = 0
        self._out_dim = 0

    # ---- layer constructors, named after the reference classes --------------------------
    def _dim(self) -> int:
        return self._out_dim

    def convolutional_layer(self, in_w, in_h, window, in_c, out_c, pad_same=False, has_bias=True,
                            w_stride=1, h_stride=1, table=None, window_h=None, w_dilation=1,
                            h_dilation=1, algo=0):
        d = conv_params(in_w, in_h, in_c, window, window if window_h is None else window_h, out_c,
                        pad_same, has_bias, w_stride, h_stride, w_dilation, h_dilation, table, algo)
        s = LayerSpec()
        s.kind = LAYER_CONV
        s.conv = d
        self._keep.append(d)
        self.specs.append(s)
        self._out_dim = d.out_c * d.out_h * d.out_w
        return self

    def fully_connected_layer(self, in_dim, out_dim, has_bias=True):
        s = LayerSpec()
        s.kind, s.fc_in, s.fc_out, s.fc_has_bias = LAYER_FC, in_dim, out_dim, int(has_bias)
        self.specs.append(s)
        self._out_dim = out_dim
        return self

    def max_pooling_layer(self, in_w, in_h, in_c, pool, stride=None):
        d = maxpool_params(in_w, in_h, in_c, pool, pool, stride or pool, stride or pool)
        s = LayerSpec()
        s.kind, s.pool = LAYER_MAXPOOL, d
        self.specs.append(s)
        self._out_dim = d.in_c * d.out_h * d.out_w
        return self

    def average_pooling_layer(self, in_w, in_h, in_c, pool, stride=None):
        d = maxpool_params(in_w, in_h, in_c, pool, pool, stride or pool, stride or pool)
        s = LayerSpec()
        s.kind, s.pool = LAYER_AVGPOOL, d
        self.specs.append(s)
        self._out_dim = d.in_c * d.out_h * d.out_w
        return self

    def _act(self, kind, param=0.0):
        s = LayerSpec()
        s.kind = kind
        s.act_param = param
        self.specs.append(s)
        return self

    def relu_layer(self):
        return self._act(LAYER_RELU)

    def tanh_layer(self):
        return self._act(LAYER_TANH)

    def softmax_layer(self):
        return self._act(LAYER_SOFTMAX)

    def sigmoid_layer(self):
        return self._act(LAYER_SIGMOID)

    def leaky_relu_layer(self, epsilon=0.01):
        return self._act(LAYER_LEAKY_RELU, epsilon)

    def elu_layer(self, alpha=1.0):
        return self._act(LAYER_ELU, alpha)

    def batch_normalization_layer(self, in_spatial_size, in_channels, epsilon=1e-5, momentum=0.999):
        """batch_normalization_layer(in_spatial_size, in_channels, epsilon, momentum)
        (tiny_dnn/layers/batch_normalization_layer.h:59-72)."""
        s = LayerSpec()
        s.kind = LAYER_BATCHNORM
        s.bn_spatial, s.bn_channels, s.bn_eps, s.bn_momentum = in_spatial_size, in_channels, epsilon, momentum
        self.specs.append(s)
        self._out_dim = in_spatial_size * in_channels
        return self

    # ---- device twin ---------------------------------------------------------------------
    def spec_array(self):
        arr = (LayerSpec * len(self.specs))(*self.specs)
        return arr

    def build(self, max_batch: int, ctx: Optional[Context] = None):
        self.ctx = ctx or Context(self.device)
        self.lib = self.ctx.lib
        h = C.c_void_p()
        arr = self.spec_array()
        check(self.lib.b200_net_create(self.ctx.handle, arr, len(self.specs), max_batch, C.byref(h)))
        self.handle = h
        self.max_batch = max_batch
        self.n_params = int(self.lib.b200_net_param_count(h))
        self.in_dim = int(self.lib.b200_net_in_dim(h))
        self.out_dim = int(self.lib.b200_net_out_dim(h))
        return self

    def close(self):
        if self.handle:
            self.lib.b200_net_destroy(self.handle)
            self.handle = None

    def tensors(self):
        """(offset, length) of every trainable tensor in update order."""
        out = []
        for i in range(self.lib.b200_net_tensor_count(self.handle)):
            off, ln = C.c_size_t(), C.c_size_t()
            check(self.lib.b200_net_tensor_info(self.handle, i, C.byref(off), C.byref(ln)))
            out.append((off.value, ln.value))
        return out

    def fan_in_out(self):
        """(fan_in, fan_out) per trainable tensor, as the layers report them
        (convolutional_layer.h:269-277, fully_connected_layer.h:51-53,
        partial_connected_layer.h:45-47)."""
        fans = []
        for s in self.specs:
            if s.kind == LAYER_CONV:
                d = s.conv
                fi = d.k_w * d.k_h * d.in_c
                fo = (d.k_w // d.stride_w) * (d.k_h // d.stride_h) * d.out_c
                fans.append((fi, fo))
                if d.has_bias:
                    fans.append((fi, fo))
            elif s.kind == LAYER_FC:
                fans.append((s.fc_in, s.fc_out))
                if s.fc_has_bias:
                    fans.append((s.fc_in, s.fc_out))
            elif s.kind == LAYER_AVGPOOL:
                fi = s.pool.pool_w * s.pool.pool_h
                fans += [(fi, 1), (fi, 1)]
        return fans

    def init_weight(self, rng: np.random.Generator) -> np.ndarray:
        """Xavier-uniform weights, zero biases (tiny_dnn/util/weight_init.h:37-47,
        tiny_dnn/layers/layer.h:72-73), drawn from `rng`; returns the flat vector."""
        flat = np.zeros(self.n_params, dtype=np.float32)
        is_weight = []
        for s in self.specs:
            if s.kind == LAYER_CONV:
                is_weight += [True] + ([False] if s.conv.has_bias else [])
            elif s.kind == LAYER_FC:
                is_weight += [True] + ([False] if s.fc_has_bias else [])
            elif s.kind == LAYER_AVGPOOL:
                is_weight += [True, False]
        for (off, ln), (fi, fo), w in zip(self.tensors(), self.fan_in_out(), is_weight):
            if w:
                b = np.sqrt(6.0 / (fi + fo))
                flat[off:off + ln] = rng.uniform(-b, b, size=ln).astype(np.float32)
        self.set_params(flat)
        return flat

    def set_params(self, flat: np.ndarray):
        flat = np.ascontiguousarray(flat, dtype=np.float32)
        assert flat.size == self.n_params
        check(self.lib.b200_net_set_params(self.handle, ptr(flat)))

    def get_params(self) -> np.ndarray:
        flat = np.empty(self.n_params, dtype=np.float32)
        check(self.lib.b200_net_get_params(self.handle, ptr(flat)))
        return flat

    def get_grads(self) -> np.ndarray:
        flat = np.empty(self.n_params, dtype=np.float32)
        check(self.lib.b200_net_get_grads(self.handle, ptr(flat)))
        return flat

    def grads_tensor(self) -> torch.Tensor:
        """torch view of the device gradient bucket (for the all-reduce)."""
        addr = self.lib.b200_net_grads_ptr(self.handle)
        return torch.as_tensor(DevicePtr(addr, self.n_params), device=f"cuda:{self.device}")

    def output_tensor(self, batch: int) -> torch.Tensor:
        addr = self.lib.b200_net_output_ptr(self.handle)
        t = torch.as_tensor(DevicePtr(addr, batch * self.out_dim), device=f"cuda:{self.device}")
        return t.view(batch, self.out_dim)

    def layer_out(self, i: int, batch: int, dim: int) -> Optional[torch.Tensor]:
        addr = self.lib.b200_net_layer_out_ptr(self.handle, i)
        if not addr:
            return None
        return torch.as_tensor(DevicePtr(addr, batch * dim), device=f"cuda:{self.device}").view(batch, dim)

    # ---- the step ---------------------------------------------------------------------------
    def forward(self, x: torch.Tensor):
        check(self.lib.b200_net_forward(self.handle, ptr(x), x.shape[0]))

    def backward(self, t: torch.Tensor, loss: int):
        check(self.lib.b200_net_backward(self.handle, ptr(t), loss))

    def forward_backward(self, x: torch.Tensor, t: torch.Tensor, loss: int):
        """fprop + bprop in one (graph-captured) call; leaves the gradient bucket ready."""
        check(self.lib.b200_net_forward_backward(self.handle, ptr(x), ptr(t), x.shape[0], loss))

    def update(self, opt):
        h = opt.hyper()
        check(self.lib.b200_net_update(self.handle, opt.kind, C.byref(h)))

    def train_onebatch(self, opt, x: torch.Tensor, t: torch.Tensor, loss: int):
        """network::train_onebatch (tiny_dnn/network.h:911-926) with device-resident x, t."""
        h = opt.hyper()
        check(self.lib.b200_net_train_step(self.handle, ptr(x), ptr(t), x.shape[0], loss, opt.kind,
                                           C.byref(h)))

    def train_onebatch_host(self, opt, x_host, t_host, loss: int, out_host=None):
        """The same step from HOST buffers (numpy arrays or pinned torch CPU tensors)."""
        h = opt.hyper()
        check(self.lib.b200_net_train_step_host(self.handle, ptr(x_host), ptr(t_host),
                                                x_host.shape[0], loss, opt.kind, C.byref(h),
                                                ptr(out_host)))

    def fit(self, opt, inputs, targets, batch_size: int, epochs: int, loss: int, outputs=None):
        """network::fit (tiny_dnn/network.h:840-879) over HOST arrays [N][dim]: one library call,
        uploads overlapped with the steps.  `outputs` [N][out_dim] receives every step's forward
        output.  When N is not a multiple of the mini-batch, the short last step is completed with
        the previous step's rows, as the reference's batch buffers do (network.h:911-926)."""
        h = opt.hyper()
        check(self.lib.b200_net_fit_host(self.handle, ptr(inputs), ptr(targets), inputs.shape[0],
                                         batch_size, epochs, loss, opt.kind, C.byref(h), ptr(outputs)))

    def set_input_grad(self, on: bool):
        """Whether the backward pass also produces the gradient with respect to the input rows (the
        first layer's prev_delta: the reference computes it, network::fit never reads it).  Off drops
        that kernel; the weights come out bit for bit the same."""
        check(self.lib.b200_net_set_input_grad(self.handle, 1 if on else 0))

    def adam_powers(self):
        a, b = C.c_float(), C.c_float()
        check(self.lib.b200_net_adam_powers(self.handle, C.byref(a), C.byref(b)))
        return a.value, b.value


# --- the networks of the benchmark configurations -------------------------------------------
LENET_TABLE = np.array([
    # connection table of examples/mnist/train.cpp:44-51: rows = 6 inputs, cols = 16 outputs
    [1, 0, 0, 0, 1, 1, 1, 0, 0, 1, 1, 1, 1, 0, 1, 1],
    [1, 1, 0, 0, 0, 1, 1, 1, 0, 0, 1, 1, 1, 1, 0, 1],
    [1, 1, 1, 0, 0, 0, 1, 1, 1, 0, 0, 1, 0, 1, 1, 1],
    [0, 1, 1, 1, 0, 0, 1, 1, 1, 1, 0, 0, 1, 0, 1, 1],
    [0, 0, 1, 1, 1, 0, 0, 1, 1, 1, 1, 0, 1, 1, 0, 1],
    [0, 0, 0, 1, 1, 1, 0, 0, 1, 1, 1, 1, 0, 1, 1, 1],
], dtype=np.uint8)


def lenet5(device=0) -> Sequential:
    """LeNet-5 of examples/mnist/train.cpp:44-59 (conv-tanh-avgpool-tanh ... fc-tanh)."""
    n = Sequential(device)
    n.convolutional_layer(32, 32, 5, 1, 6).tanh_layer()
    n.average_pooling_layer(28, 28, 6, 2).tanh_layer()
    n.convolutional_layer(14, 14, 5, 6, 16, table=LENET_TABLE).tanh_layer()
    n.average_pooling_layer(10, 10, 16, 2).tanh_layer()
    n.convolutional_layer(5, 5, 5, 16, 120).tanh_layer()
    n.fully_connected_layer(120, 10).tanh_layer()
    return n


def cifar10_net(device=0) -> Sequential:
    """CIFAR-10 net: conv5x5(same)->32 relu, maxpool; conv5x5->32 relu, maxpool;
    conv5x5->64 relu, maxpool; fc 1024->64 relu; fc 64->10 softmax
    (layers of examples/cifar10/train.cpp:26-42 in conv-relu-pool order)."""
    n = Sequential(device)
    n.convolutional_layer(32, 32, 5, 3, 32, pad_same=True).relu_layer().max_pooling_layer(32, 32, 32, 2)
    n.convolutional_layer(16, 16, 5, 32, 32, pad_same=True).relu_layer().max_pooling_layer(16, 16, 32, 2)
    n.convolutional_layer(8, 8, 5, 32, 64, pad_same=True).relu_layer().max_pooling_layer(8, 8, 64, 2)
    n.fully_connected_layer(4 * 4 * 64, 64).relu_layer()
    n.fully_connected_layer(64, 10).softmax_layer()
    return n


def mlp(device=0, hidden=4096) -> Sequential:
    """MLP 784 -> hidden -> hidden -> 10, relu, relu, softmax."""
    n = Sequential(device)
    n.fully_connected_layer(784, hidden).relu_layer()
    n.fully_connected_layer(hidden, hidden).relu_layer()
    n.fully_connected_layer(hidden, 10).softmax_layer()
    return n
