"""Seeded test cases shared by the golden-fixture generator, the CPU tests of the
oracle and the GPU parity tests.  Every case regenerates its inputs from its
seed, so a fixture only has to store the reference's outputs."""
from __future__ import annotations

import ctypes as C

import numpy as np

from tiny_cnn_b200._lib import (LAYER_AVGPOOL, LAYER_BATCHNORM, LAYER_CONV, LAYER_ELU, LAYER_FC, LAYER_LEAKY_RELU, LAYER_MAXPOOL,
                                LAYER_RELU, LAYER_SIGMOID, LAYER_SOFTMAX, LAYER_TANH, LayerSpec, OptHyper)
from tiny_cnn_b200._lib import ConvDesc, PoolDesc
from tiny_cnn_b200.network import LENET_TABLE


# Descriptor arithmetic restated in Python, so that the fixture generator, the oracle tests and the
# benchmark's CPU legs describe a network without loading the CUDA library (tests/test_abi.py checks
# these against b200_conv_desc_init / b200_pool_desc_init).
def _conv_out_length(n, k, stride, dil, same):
    """conv_out_length (tiny_dnn/util/util.h:329-344)."""
    return -(-n // stride) if same else -(-(n - dil * k + dil) // stride)


def conv_params(in_w, in_h, in_c, k_w, k_h, out_c, pad_same=False, has_bias=True, stride_w=1,
                stride_h=1, dil_w=1, dil_h=1, table=None, algo=0, input_is_padded=False) -> ConvDesc:
    """conv_set_params (tiny_dnn/layers/convolutional_layer.h:404-438) into a b200_conv_desc."""
    d = ConvDesc()
    d.in_w, d.in_h, d.in_c = in_w, in_h, in_c
    d.inp_w = in_w + k_w - 1 if pad_same else in_w
    d.inp_h = in_h + k_h - 1 if pad_same else in_h
    d.out_w = _conv_out_length(in_w, k_w, stride_w, dil_w, pad_same)
    d.out_h = _conv_out_length(in_h, k_h, stride_h, dil_h, pad_same)
    d.out_c, d.k_w, d.k_h = out_c, k_w, k_h
    d.stride_w, d.stride_h, d.dil_w, d.dil_h = stride_w, stride_h, dil_w, dil_h
    d.has_bias, d.pad_same = int(has_bias), int(pad_same)
    d.algo, d.input_is_padded = algo, int(input_is_padded)
    assert d.out_w > 0 and d.out_h > 0
    if table is not None:
        t = np.ascontiguousarray(np.asarray(table, dtype=np.uint8).reshape(in_c, out_c))
        d._table_keepalive = t
        d.tbl = t.ctypes.data_as(C.POINTER(C.c_uint8))
    return d


def maxpool_params(in_w, in_h, in_c, pool_w, pool_h=None, stride_w=None, stride_h=None,
                   ceil_mode=False, pad_same=False) -> PoolDesc:
    """pool_out_length (tiny_dnn/util/util.h:346-363) into a b200_pool_desc."""
    pool_h = pool_w if pool_h is None else pool_h
    stride_w = pool_w if stride_w is None else stride_w
    stride_h = pool_h if stride_h is None else stride_h

    def out_len(n, win, stride):
        ln = n if pad_same else n - win + 1
        tmp = np.float32(ln + stride - 1) / np.float32(stride)
        return int(np.ceil(tmp) if ceil_mode else np.floor(tmp))
    d = PoolDesc()
    d.in_w, d.in_h, d.in_c = in_w, in_h, in_c
    d.pool_w, d.pool_h, d.stride_w, d.stride_h = pool_w, pool_h, stride_w, stride_h
    d.out_w, d.out_h = out_len(in_w, pool_w, stride_w), out_len(in_h, pool_h, stride_h)
    assert d.out_w > 0 and d.out_h > 0
    return d


def hyper(alpha=0.01, b1=0.9, b2=0.999, b1_t=0.9, b2_t=0.999, mu=0.9, lambda_=0.0, eps=1e-8) -> OptHyper:
    return OptHyper(alpha, b1, b2, b1_t, b2_t, mu, lambda_, eps)

_rng_tbl = np.random.default_rng(5)
RANDOM_TABLE_4x6 = (_rng_tbl.random((4, 6)) > 0.4).astype(np.uint8)
RANDOM_TABLE_4x6[0, :] = 1  # every output keeps at least one input

# name -> convolution case.  w,h,c: input; k: window (kw,kh); oc: output maps
CONV_CASES = {
    "valid3x3": dict(w=8, h=8, c=3, kw=3, kh=3, oc=4, same=False, bias=True, B=3, seed=1),
    "same3x3": dict(w=8, h=8, c=3, kw=3, kh=3, oc=4, same=True, bias=True, B=3, seed=2),
    "same5x5_rect": dict(w=12, h=10, c=2, kw=5, kh=5, oc=6, same=True, bias=True, B=2, seed=3),
    "valid5x5_tbl": dict(w=10, h=10, c=4, kw=5, kh=5, oc=6, same=False, bias=True, B=3, seed=4,
                         table=RANDOM_TABLE_4x6),
    "stride2": dict(w=9, h=9, c=2, kw=3, kh=3, oc=3, same=False, bias=True, B=2, seed=5, sw=2, sh=2),
    "stride2_same": dict(w=9, h=8, c=2, kw=3, kh=3, oc=3, same=True, bias=True, B=2, seed=6, sw=2, sh=2),
    "dilation2": dict(w=11, h=11, c=2, kw=3, kh=3, oc=3, same=False, bias=True, B=2, seed=7, dw=2, dh=2),
    "nobias": dict(w=10, h=10, c=4, kw=5, kh=5, oc=6, same=False, bias=False, B=2, seed=8),
    "rect_kernel": dict(w=9, h=10, c=2, kw=3, kh=2, oc=3, same=False, bias=True, B=2, seed=9),
    "even_same": dict(w=8, h=8, c=2, kw=4, kh=4, oc=3, same=True, bias=True, B=2, seed=10),
    "lenet_c1": dict(w=32, h=32, c=1, kw=5, kh=5, oc=6, same=False, bias=True, B=4, seed=11),
    "lenet_c3": dict(w=14, h=14, c=6, kw=5, kh=5, oc=16, same=False, bias=True, B=4, seed=12,
                     table=LENET_TABLE),
    "lenet_c5": dict(w=5, h=5, c=16, kw=5, kh=5, oc=120, same=False, bias=True, B=4, seed=13),
    "cifar_c1": dict(w=32, h=32, c=3, kw=5, kh=5, oc=32, same=True, bias=True, B=3, seed=14),
    "cifar_c2": dict(w=16, h=16, c=32, kw=5, kh=5, oc=32, same=True, bias=True, B=3, seed=15),
    "cifar_c3": dict(w=8, h=8, c=32, kw=5, kh=5, oc=64, same=True, bias=True, B=5, seed=16),
    "sweep3x3_small": dict(w=14, h=14, c=16, kw=3, kh=3, oc=24, same=True, bias=True, B=2, seed=17),
    "odd_sizes": dict(w=13, h=7, c=5, kw=3, kh=3, oc=7, same=True, bias=True, B=3, seed=18),
    "one_sample": dict(w=6, h=6, c=1, kw=3, kh=3, oc=1, same=False, bias=True, B=1, seed=19),
}


def conv_desc(c, algo=0, input_is_padded=False):
    return conv_params(c["w"], c["h"], c["c"], c["kw"], c["kh"], c["oc"], c["same"], c["bias"],
                       c.get("sw", 1), c.get("sh", 1), c.get("dw", 1), c.get("dh", 1),
                       c.get("table"), algo, input_is_padded)


def gen_conv_inputs(c, d):
    """x ~ N(0,1), W ~ U(-0.5, 0.5), b ~ U(-0.1, 0.1), dy ~ N(0,1) from the case seed."""
    rng = np.random.default_rng(c["seed"])
    B = c["B"]
    x = rng.standard_normal((B, c["c"] * c["h"] * c["w"])).astype(np.float32)
    if c.get("xrange"):
        lo, hi = c["xrange"]
        x = rng.uniform(lo, hi, x.shape).astype(np.float32)
    W = rng.uniform(-0.5, 0.5, c["oc"] * c["c"] * c["kh"] * c["kw"]).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, c["oc"]).astype(np.float32) if c["bias"] else None
    if c.get("zero_bias"):
        b = np.zeros(c["oc"], dtype=np.float32)
    dy = rng.standard_normal((B, d.out_c * d.out_h * d.out_w)).astype(np.float32)
    return x, W, b, dy


FC_CASES = {
    "small": dict(B=3, **{"in": 7, "out": 5}, bias=True, seed=21),
    "nobias": dict(B=2, **{"in": 9, "out": 4}, bias=False, seed=22),
    "lenet_f6": dict(B=16, **{"in": 120, "out": 10}, bias=True, seed=23),
    "cifar_fc1": dict(B=8, **{"in": 1024, "out": 64}, bias=True, seed=24),
    "ragged": dict(B=5, **{"in": 130, "out": 67}, bias=True, seed=25),
    # long inner dimension, few outputs, an odd batch, no bias: the split-k path of the small GEMM
    "skinny_tail": dict(B=11, **{"in": 576, "out": 48}, bias=False, seed=26),
}

MAXPOOL_CASES = {
    "2x2": dict(w=8, h=8, c=3, pw=2, ph=2, sw=2, sh=2, B=3, seed=31),
    "overlap": dict(w=7, h=7, c=2, pw=3, ph=3, sw=2, sh=2, B=2, seed=32),
    "stride1_same": dict(w=6, h=5, c=2, pw=2, ph=2, sw=1, sh=1, same=1, B=2, seed=33),
    "gap": dict(w=9, h=9, c=2, pw=2, ph=2, sw=3, sh=3, B=2, seed=34),
    "ceil": dict(w=7, h=7, c=2, pw=2, ph=2, sw=2, sh=2, ceil=1, B=2, seed=35),
    "cifar_p1": dict(w=32, h=32, c=32, pw=2, ph=2, sw=2, sh=2, B=2, seed=36),
    "rect": dict(w=8, h=6, c=2, pw=2, ph=1, sw=2, sh=1, B=2, seed=37),
}

AVGPOOL_CASES = {
    "2x2": dict(w=8, h=8, c=3, pw=2, ph=2, sw=2, sh=2, B=3, seed=41),
    "lenet_s2": dict(w=28, h=28, c=6, pw=2, ph=2, sw=2, sh=2, B=4, seed=42),
    "overlap": dict(w=6, h=6, c=2, pw=2, ph=2, sw=1, sh=1, B=2, seed=43),
    "3x3": dict(w=9, h=9, c=2, pw=3, ph=3, sw=3, sh=3, B=2, seed=44),
}


def pool_desc(c):
    return maxpool_params(c["w"], c["h"], c["c"], c["pw"], c["ph"], c["sw"], c["sh"],
                          bool(c.get("ceil", 0)), bool(c.get("same", 0)))


ACT_CASES = {
    "relu": dict(kind=1, B=4, dim=37, seed=51),
    "tanh": dict(kind=2, B=4, dim=37, seed=52, scale=2.0),
    "softmax": dict(kind=3, B=6, dim=10, seed=53, scale=3.0),
    "softmax_wide": dict(kind=3, B=3, dim=33, seed=54, scale=5.0),
    # sigmoid / leaky relu / elu with the reference's default parameter and with another one
    "sigmoid": dict(kind=4, B=4, dim=37, seed=55, scale=3.0),
    "leaky_relu": dict(kind=5, B=4, dim=37, seed=56),
    "leaky_relu_0.2": dict(kind=5, B=3, dim=41, seed=57, param=0.2),
    "elu": dict(kind=6, B=4, dim=37, seed=58, scale=2.0),
    "elu_0.7": dict(kind=6, B=3, dim=41, seed=59, scale=2.0, param=0.7),
}

# batch normalization (channels x spatial rows), local response normalization, dropout
BATCHNORM_CASES = {
    "conv_like": dict(C=6, S=49, B=5, eps=1e-5, seed=71, shift=0.7, scale=2.0),
    "fc_like": dict(C=33, S=1, B=16, eps=1e-3, seed=72, shift=-0.3, scale=0.5),
    "one_sample": dict(C=4, S=25, B=1, eps=1e-5, seed=73, shift=0.0, scale=1.0),
    "wide": dict(C=3, S=1024, B=12, eps=1e-5, seed=74, shift=5.0, scale=3.0),
}
LRN_CASES = {
    "alexnet_like": dict(C=8, w=6, h=5, size=5, alpha=1e-4, beta=0.75, B=3, seed=75),
    "default_params": dict(C=5, w=4, h=4, size=3, alpha=1.0, beta=5.0, B=2, seed=76),
    "window_wider_than_channels": dict(C=3, w=3, h=3, size=5, alpha=0.5, beta=2.0, B=2, seed=77),
}
DROPOUT_CASES = {
    "half": dict(dim=101, rate=0.5, B=4, seed=78),
    "light": dict(dim=64, rate=0.2, B=3, seed=79),
}


def gen_batchnorm_inputs(c):
    rng = np.random.default_rng(c["seed"])
    n = c["C"] * c["S"]
    x = (rng.standard_normal((c["B"], n)) * c["scale"] + c["shift"]).astype(np.float32)
    dy = rng.standard_normal((c["B"], n)).astype(np.float32)
    run_mean = rng.uniform(-1, 1, c["C"]).astype(np.float32)
    run_var = rng.uniform(0.5, 2.0, c["C"]).astype(np.float32)
    return x, dy, run_mean, run_var


# quantized forward: x ~ U[-1, 1], W ~ U[-0.5, 0.5] as the benchmark configuration states
QCONV_CASES = {
    "valid5x5": dict(w=12, h=12, c=4, kw=5, kh=5, oc=6, same=False, bias=True, B=3, seed=61,
                     xrange=(-1, 1)),
    "zero_bias": dict(w=12, h=12, c=4, kw=5, kh=5, oc=6, same=False, bias=True, B=2, seed=62,
                      xrange=(-1, 1), zero_bias=True),
    "stride2": dict(w=12, h=12, c=4, kw=5, kh=5, oc=8, same=False, bias=True, B=2, seed=63,
                    xrange=(-1, 1), sw=2, sh=2),
    "cfg5_small_batch": dict(w=28, h=28, c=32, kw=5, kh=5, oc=64, same=False, bias=True, B=2, seed=65,
                             xrange=(-1, 1)),
}

# padding::same: the reference's quantized layer never allocates its padded
# staging buffer (quantized_convolutional_layer.h:349-358 `init()` has no
# caller), so it cannot be run; the kernel restatement still defines the result
# for an already padded input.
QCONV_ORACLE_ONLY = {
    "same3x3": dict(w=10, h=10, c=2, kw=3, kh=3, oc=10, same=True, bias=True, B=2, seed=64,
                    xrange=(-1, 1)),
}

QFC_CASES = {
    "small": dict(B=3, **{"in": 40, "out": 12}, bias=True, seed=71),
    "nobias": dict(B=2, **{"in": 33, "out": 7}, bias=False, seed=72),
    "wide": dict(B=2, **{"in": 1152, "out": 64}, bias=True, seed=73),
}


# the forms for chained quantized layers: operands are uint8 values held in floats, with ranges
QEQ_CONV_CASES = {"valid5x5": dict(seed=81), "stride2": dict(seed=82), "zero_bias": dict(seed=83, flat_filter_range=True)}
QEQ_FC_CASES = {"small": dict(seed=84), "nobias": dict(seed=85), "wide": dict(seed=86, flat_ranges=True)}


def gen_qeq_conv_inputs(name):
    """(desc, x, W, bias, in_r, W_r, b_r) for QEQ_CONV_CASES[name] on the geometry of QCONV_CASES[name]."""
    c, e = QCONV_CASES[name], QEQ_CONV_CASES[name]
    d = conv_desc(c)
    rng = np.random.default_rng(e["seed"])
    B = c["B"]
    x = rng.integers(0, 256, (B, d.in_c * d.inp_h * d.inp_w)).astype(np.float32)
    W = rng.integers(0, 256, d.out_c * d.in_c * d.k_h * d.k_w).astype(np.float32)
    bias = rng.integers(0, 256, d.out_c).astype(np.float32)
    in_r = np.stack([np.array([-1.0 - 0.25 * n, 1.0 + 0.125 * n], np.float32) for n in range(B)])
    W_r = np.array([0.25, 0.25] if e.get("flat_filter_range") else [-0.5, 0.5], np.float32)
    b_r = np.array([-0.1, 0.1], np.float32)
    return d, x, W, bias, np.ascontiguousarray(in_r), W_r, b_r


def gen_qeq_fc_inputs(name):
    c, e = QFC_CASES[name], QEQ_FC_CASES[name]
    rng = np.random.default_rng(e["seed"])
    B, I, O = c["B"], c["in"], c["out"]
    x = rng.integers(0, 256, (B, I)).astype(np.float32)
    W = rng.integers(0, 256, I * O).astype(np.float32)
    bias = rng.integers(0, 256, O).astype(np.float32) if c["bias"] else None
    in_r = np.stack([np.array([-1.0 - 0.25 * n, 1.0 + 0.125 * n], np.float32) for n in range(B)])
    flat = e.get("flat_ranges")
    W_r = np.array([0.25, 0.25] if flat else [-0.5, 0.5], np.float32)
    b_r = np.array([0.05, 0.05] if flat else [-0.1, 0.1], np.float32)
    return I, O, x, W, bias, np.ascontiguousarray(in_r), W_r, b_r


def hyper_for(kind: int) -> OptHyper:
    """Default hyper-parameters of the reference optimizers (optimizer.h:57-58,104-110,203)."""
    if kind == 0:
        return hyper(alpha=0.01)
    if kind == 1:
        return hyper(alpha=0.001, b1=0.9, b2=0.999, b1_t=0.9, b2_t=0.999)
    if kind == 3:  # RMSprop (optimizer.h:80)
        return hyper(alpha=0.0001, mu=0.99)
    if kind == 4:  # adamax (optimizer.h:146-151)
        return hyper(alpha=0.002, b1=0.9, b2=0.999, b1_t=0.9)
    if kind == 5:  # gradient_descent; a weight decay so that the lambda term is exercised
        return hyper(alpha=0.01, lambda_=0.001)
    if kind == 6:  # nesterov_momentum, with weight decay
        return hyper(alpha=0.01, mu=0.9, lambda_=0.001)
    return hyper(alpha=0.01, mu=0.9, lambda_=0.0)


OPT_KINDS = (0, 1, 2, 3, 4, 5, 6)


# ---- networks ------------------------------------------------------------------------------
def _conv(w, h, k, c, oc, same=False, table=None):
    s = LayerSpec()
    s.kind = LAYER_CONV
    d = conv_params(w, h, c, k, k, oc, same, True, table=table)
    s.conv = d
    return s, d


def _fc(i, o):
    s = LayerSpec()
    s.kind, s.fc_in, s.fc_out, s.fc_has_bias = LAYER_FC, i, o, 1
    return s, None


def _pool(kind, w, h, c, p):
    s = LayerSpec()
    s.kind = kind
    s.pool = maxpool_params(w, h, c, p, p, p, p)
    return s, None


def _act(kind, param=0.0):
    s = LayerSpec()
    s.kind = kind
    s.act_param = param
    return s, None


def _bn(spatial, channels, eps=1e-5, momentum=0.999):
    s = LayerSpec()
    s.kind = LAYER_BATCHNORM
    s.bn_spatial, s.bn_channels, s.bn_eps, s.bn_momentum = spatial, channels, eps, momentum
    return s, None


def build_net_specs(name):
    """Layer specs of a named network; returns (specs, keepalive)."""
    if name == "lenet":
        L = [_conv(32, 32, 5, 1, 6), _act(LAYER_TANH), _pool(LAYER_AVGPOOL, 28, 28, 6, 2), _act(LAYER_TANH),
             _conv(14, 14, 5, 6, 16, table=LENET_TABLE), _act(LAYER_TANH),
             _pool(LAYER_AVGPOOL, 10, 10, 16, 2), _act(LAYER_TANH),
             _conv(5, 5, 5, 16, 120), _act(LAYER_TANH), _fc(120, 10), _act(LAYER_TANH)]
    elif name == "cifar":
        L = [_conv(32, 32, 5, 3, 32, True), _act(LAYER_RELU), _pool(LAYER_MAXPOOL, 32, 32, 32, 2),
             _conv(16, 16, 5, 32, 32, True), _act(LAYER_RELU), _pool(LAYER_MAXPOOL, 16, 16, 32, 2),
             _conv(8, 8, 5, 32, 64, True), _act(LAYER_RELU), _pool(LAYER_MAXPOOL, 8, 8, 64, 2),
             _fc(1024, 64), _act(LAYER_RELU), _fc(64, 10), _act(LAYER_SOFTMAX)]
    elif name == "mlp_small":
        L = [_fc(784, 96), _act(LAYER_RELU), _fc(96, 96), _act(LAYER_RELU), _fc(96, 10),
             _act(LAYER_SOFTMAX)]
    elif name == "mlp":
        L = [_fc(784, 4096), _act(LAYER_RELU), _fc(4096, 4096), _act(LAYER_RELU), _fc(4096, 10),
             _act(LAYER_SOFTMAX)]
    elif name == "tiny_conv":
        L = [_conv(12, 12, 3, 2, 4, True), _act(LAYER_RELU), _pool(LAYER_MAXPOOL, 12, 12, 4, 2),
             _conv(6, 6, 3, 4, 5), _act(LAYER_TANH), _fc(80, 6), _act(LAYER_SOFTMAX)]
    elif name == "tiny_conv_bn":
        # batch normalization between a convolution and its relu, and before the classifier
        L = [_conv(12, 12, 3, 2, 4, True), _bn(144, 4), _act(LAYER_RELU), _pool(LAYER_MAXPOOL, 12, 12, 4, 2),
             _conv(6, 6, 3, 4, 5), _bn(16, 5, 1e-3, 0.9), _act(LAYER_TANH), _fc(80, 6), _act(LAYER_SOFTMAX)]
    elif name == "tiny_conv_acts":
        # the activations with a constructor parameter between the hot operators
        L = [_conv(12, 12, 3, 2, 4, True), _act(LAYER_LEAKY_RELU, 0.1), _pool(LAYER_MAXPOOL, 12, 12, 4, 2),
             _conv(6, 6, 3, 4, 5), _act(LAYER_ELU, 0.8), _fc(80, 6), _act(LAYER_SIGMOID)]
    else:
        raise KeyError(name)
    return [s for s, _ in L], [k for _, k in L]


NET_CASES = {
    # LeNet-5, +-1 targets through fit<mse>, adagrad lr 0.01 (benchmark config 1, fewer steps)
    "lenet_adagrad": dict(net="lenet", B=16, steps=4, seed=101, in_dim=1024, out_dim=10, loss=0, opt=0,
                          t_lo=-1.0, t_hi=1.0, xgen=lambda r, s: r.uniform(-1, 1, s)),
    # CIFAR-10 net, cross-entropy after softmax, adam lr 1e-3 (benchmark config 2, small batch)
    "cifar_adam": dict(net="cifar", B=8, steps=3, seed=102, in_dim=3072, out_dim=10, loss=1, opt=1,
                       t_lo=0.0, t_hi=1.0, xgen=lambda r, s: r.standard_normal(s)),
    # MLP with momentum SGD (benchmark config 4 at reduced width)
    "mlp_momentum": dict(net="mlp_small", B=16, steps=3, seed=103, in_dim=784, out_dim=10, loss=1, opt=2,
                         t_lo=0.0, t_hi=1.0, xgen=lambda r, s: r.uniform(0, 1, s)),
    "tiny_conv_adam": dict(net="tiny_conv", B=5, steps=4, seed=104, in_dim=288, out_dim=6, loss=2, opt=1,
                           t_lo=0.0, t_hi=1.0, xgen=lambda r, s: r.standard_normal(s)),
    # batch normalization layers (train phase while fitting, moving averages for predict), adam
    "tiny_conv_bn_adam": dict(net="tiny_conv_bn", B=6, steps=4, seed=106, in_dim=288, out_dim=6, loss=1, opt=1,
                              t_lo=0.0, t_hi=1.0, xgen=lambda r, s: r.standard_normal(s)),
    # leaky relu / elu / sigmoid, mse, RMSprop
    "tiny_conv_acts_rmsprop": dict(net="tiny_conv_acts", B=6, steps=4, seed=105, in_dim=288, out_dim=6, loss=0, opt=3,
                                   t_lo=0.0, t_hi=1.0, xgen=lambda r, s: r.standard_normal(s)),
}


def bn_layers(specs):
    """indices of the batch normalization layers"""
    return [i for i, s in enumerate(specs) if s.kind == LAYER_BATCHNORM]


def null_gradient_biases(specs):
    """Offsets (into the flat parameter buffer) of the biases of layers that feed a batch normalization
    layer.  Their gradient is exactly zero in exact arithmetic (the normalization subtracts the channel
    mean), so what any implementation holds there is the rounding noise of its sums: such a tensor is
    checked to be noise, not to match the other side's noise."""
    offs, off = set(), 0
    for i, s in enumerate(specs):
        if s.kind == LAYER_CONV:
            d = s.conv
            w, b = d.out_c * d.in_c * d.k_h * d.k_w, (d.out_c if d.has_bias else 0)
        elif s.kind == LAYER_FC:
            w, b = s.fc_in * s.fc_out, (s.fc_out if s.fc_has_bias else 0)
        elif s.kind == LAYER_AVGPOOL:
            w, b = s.pool.pool_w * s.pool.pool_h * s.pool.in_c, s.pool.in_c
        else:
            continue
        if b and i + 1 < len(specs) and specs[i + 1].kind == LAYER_BATCHNORM:
            offs.add(off + w)
        off += w + b
    return offs


def net_layout(specs):
    """(offset, length, fan_in, fan_out, is_weight) of every trainable tensor in update
    order (layer order, W before b), with the fan sizes the reference layers report
    (convolutional_layer.h:269-277, fully_connected_layer.h:51-53,
    partial_connected_layer.h:45-47)."""
    out, off = [], 0
    for s in specs:
        if s.kind == LAYER_CONV:
            d = s.conv
            fi = d.k_w * d.k_h * d.in_c
            fo = (d.k_w // d.stride_w) * (d.k_h // d.stride_h) * d.out_c
            lens = [(d.out_c * d.in_c * d.k_h * d.k_w, True)] + ([(d.out_c, False)] if d.has_bias else [])
        elif s.kind == LAYER_FC:
            fi, fo = s.fc_in, s.fc_out
            lens = [(s.fc_in * s.fc_out, True)] + ([(s.fc_out, False)] if s.fc_has_bias else [])
        elif s.kind == LAYER_AVGPOOL:
            fi, fo = s.pool.pool_w * s.pool.pool_h, 1
            lens = [(s.pool.pool_w * s.pool.pool_h * s.pool.in_c, True), (s.pool.in_c, False)]
        else:
            continue
        for ln, is_w in lens:
            out.append((off, ln, fi, fo, is_w))
            off += ln
    return out, off


def xavier_params(specs, seed):
    """Flat parameter vector: weights ~ U(+-sqrt(6/(fan_in+fan_out))) (weight_init.h:37-47),
    biases 0 (layer.h:72-73), drawn from numpy's generator."""
    layout, n = net_layout(specs)
    rng = np.random.default_rng(seed)
    flat = np.zeros(n, dtype=np.float32)
    for off, ln, fi, fo, is_w in layout:
        if is_w:
            b = np.sqrt(6.0 / (fi + fo))
            flat[off:off + ln] = rng.uniform(-b, b, ln).astype(np.float32)
    return flat


def gen_net_data(c):
    """(x, t) of a network case: inputs from the case's generator, one-hot targets."""
    rng = np.random.default_rng(c["seed"] + 1000)
    n = c["B"] * c["steps"]
    x = c["xgen"](rng, (n, c["in_dim"])).astype(np.float32)
    labels = rng.integers(0, c["out_dim"], n)
    t = np.full((n, c["out_dim"]), c["t_lo"], dtype=np.float32)
    t[np.arange(n), labels] = c["t_hi"]
    return x, t


def merge_rows_np(rows):
    """edge::merge_grads (node.h:89-103): rows summed in order in float32."""
    acc = rows[0].copy()
    for r in rows[1:]:
        acc += r
    return acc


# ---- benchmark configurations at their stated sizes -------------------------------------------
# The reference's outputs for these are too large to commit whole; tests/golden/ref_fullsize.npz
# keeps a digest of every tensor (strided samples, float64 sum, sum of magnitudes, largest
# magnitude, per-row float64 sums) made by tests/golden/make_golden_fullsize.py.
FULL_CONV_CASES = {  # single-layer sweep: 3x3, stride 1, same padding, batch 256
    "sweep_56x56x64": dict(w=56, h=56, c=64, kw=3, kh=3, oc=64, same=True, bias=True, B=256, seed=301),
    "sweep_28x28x128": dict(w=28, h=28, c=128, kw=3, kh=3, oc=128, same=True, bias=True, B=256, seed=302),
    "sweep_14x14x256": dict(w=14, h=14, c=256, kw=3, kh=3, oc=256, same=True, bias=True, B=256, seed=303),
}


def gen_full_conv_inputs(c, d):
    """x ~ N(0,1), W xavier-uniform, b ~ U(-0.1, 0.1), dy ~ N(0,1), drawn in float32."""
    rng = np.random.default_rng(c["seed"])
    B = c["B"]
    x = rng.standard_normal((B, c["c"] * c["h"] * c["w"]), dtype=np.float32)
    fan_in, fan_out = c["kw"] * c["kh"] * c["c"], c["kw"] * c["kh"] * c["oc"]
    bound = np.float32(np.sqrt(6.0 / (fan_in + fan_out)))
    W = (rng.random(c["oc"] * c["c"] * c["kh"] * c["kw"], dtype=np.float32) * 2 - 1) * bound
    b = (rng.random(c["oc"], dtype=np.float32) * 2 - 1) * np.float32(0.1)
    dy = rng.standard_normal((B, d.out_c * d.out_h * d.out_w), dtype=np.float32)
    return x, W, b, dy


FULL_NET_CASES = {
    # CIFAR-10 net at the benchmarked batch, 3 adam steps
    "cifar_adam_b256": dict(net="cifar", B=256, steps=3, seed=202, in_dim=3072, out_dim=10, loss=1, opt=1,
                            t_lo=0.0, t_hi=1.0, chunk=256, xgen=lambda r, s: r.standard_normal(s)),
    # MLP 784 -> 4096 -> 4096 -> 10, batch 1024, momentum; the reference cannot hold the per-sample
    # weight gradients of one such mini-batch (1024 x 16.8 M floats), so its gradients are computed
    # 16 samples at a time and the merged chunks added in order
    "mlp_momentum_b1024": dict(net="mlp", B=1024, steps=2, seed=204, in_dim=784, out_dim=10, loss=1, opt=2,
                               t_lo=0.0, t_hi=1.0, chunk=16, xgen=lambda r, s: r.uniform(0, 1, s)),
}

FULL_Q_CASE = dict(w=28, h=28, c=32, kw=5, kh=5, oc=64, B=128, seed=505, fc_out=256)


def gen_full_q_inputs():
    """Quantized-inference configuration: x ~ U[-1,1], conv W ~ U[-0.5,0.5], conv bias zero or
    U[-0.1,0.1], fc W ~ U[-0.5,0.5], fc bias ~ U[-0.1,0.1]."""
    c = FULL_Q_CASE
    rng = np.random.default_rng(c["seed"])
    x = rng.uniform(-1, 1, (c["B"], c["c"] * c["h"] * c["w"])).astype(np.float32)
    W = rng.uniform(-0.5, 0.5, c["oc"] * c["c"] * c["kh"] * c["kw"]).astype(np.float32)
    biases = {"bias0": np.zeros(c["oc"], np.float32),
              "bias_u": rng.uniform(-0.1, 0.1, c["oc"]).astype(np.float32)}
    Wf = rng.uniform(-0.5, 0.5, 9216 * c["fc_out"]).astype(np.float32)
    bf = rng.uniform(-0.1, 0.1, c["fc_out"]).astype(np.float32)
    return x, W, biases, Wf, bf


def digest(a, stride=101):
    """What the full-size fixture keeps of a tensor."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    flat = a.ravel()
    d64 = flat.astype(np.float64)
    out = {"samples": flat[::stride].copy(),
           "stats": np.array([d64.sum(), np.abs(d64).sum(), np.abs(d64).max() if flat.size else 0.0])}
    if a.ndim == 2 and a.shape[0] > 1:
        out["row_sums"] = a.astype(np.float64).sum(axis=1)
    return out


def check_digest(got, gold, key, tol, stride=101):
    """Compare a tensor with its stored digest: samples within tol of the tensor's largest
    magnitude, total and per-row sums within tol of the corresponding sum of magnitudes."""
    got = np.ascontiguousarray(got, dtype=np.float32)
    samples, stats = gold[f"{key}/samples"], gold[f"{key}/stats"]
    s, abs_s, mx = (float(v) for v in stats)
    mine = got.ravel()[::stride]
    assert mine.shape == samples.shape, f"{key}: {mine.shape} samples vs {samples.shape}"
    err = np.abs(mine.astype(np.float64) - samples.astype(np.float64))
    worst = float(err.max()) if err.size else 0.0
    assert worst <= tol * max(mx, 1e-30), f"{key}: sample off by {worst:g} (largest magnitude {mx:g}, tol {tol:g})"
    g64 = got.astype(np.float64)
    assert abs(float(g64.sum()) - s) <= tol * max(abs_s, 1e-30), \
        f"{key}: sum {float(g64.sum())!r} vs {s!r} (sum of magnitudes {abs_s:g})"
    if f"{key}/row_sums" in gold:
        rows = gold[f"{key}/row_sums"]
        row_abs = np.abs(g64).sum(axis=1)
        bad = np.abs(g64.sum(axis=1) - rows) > tol * np.maximum(row_abs, 1e-30)
        assert not bad.any(), f"{key}: {int(bad.sum())} row sums differ beyond {tol:g}"
    return worst / max(mx, 1e-30)


# ---- dataset formats ---------------------------------------------------------------------------
# synthetic files in the CIFAR-10 binary format (records of 1 label byte + 3 x 32 x 32 pixel bytes)
# and in the MNIST idx3-ubyte format; every byte value occurs
DATA_CASES = {
    "cifar_m1p1": dict(mode=0, n=4, c=3, h=32, w=32, xp=0, yp=0, smin=-1.0, smax=1.0, seed=81),
    "cifar_0_1_pad": dict(mode=0, n=3, c=3, h=32, w=32, xp=2, yp=1, smin=0.0, smax=1.0, seed=82),
    "cifar_odd_range": dict(mode=0, n=2, c=3, h=32, w=32, xp=0, yp=0, smin=-0.3, smax=2.7, seed=83),
    "mnist_m1p1_pad2": dict(mode=1, n=5, c=1, h=28, w=28, xp=2, yp=2, smin=-1.0, smax=1.0, seed=84),
    "mnist_0_1": dict(mode=1, n=3, c=1, h=28, w=28, xp=0, yp=0, smin=0.0, smax=1.0, seed=85),
}


def gen_dataset_bytes(c):
    """(images uint8 [n][c*h*w], labels uint8 [n]) of a dataset case; the first 256 pixels run
    through every byte value."""
    rng = np.random.default_rng(c["seed"])
    img = rng.integers(0, 256, (c["n"], c["c"] * c["h"] * c["w"]), dtype=np.uint8)
    img[0, :256] = np.arange(256, dtype=np.uint8)
    labels = rng.integers(0, 10, c["n"], dtype=np.uint8)
    return img, labels


def dataset_file_bytes(c, img, labels):
    """The file the reference's parser reads for a dataset case."""
    if c["mode"] == 0:  # CIFAR-10 binary: label byte, then the planar image
        return b"".join(bytes([int(labels[i])]) + img[i].tobytes() for i in range(c["n"]))
    header = (0x00000803).to_bytes(4, "big") + c["n"].to_bytes(4, "big") + c["h"].to_bytes(4, "big") + \
        c["w"].to_bytes(4, "big")
    return header + img.tobytes()


def image_desc(c):
    from tiny_cnn_b200._lib import ImageDesc
    return ImageDesc(c["mode"], c["c"], c["h"], c["w"], c["xp"], c["yp"], c["smin"], c["smax"])


# network::fit over data whose size is not a multiple of the mini-batch: (net case, samples,
# mini-batch, epochs).  The reference completes a short last mini-batch with the previous step's rows
# (its batch buffers keep them); one left-over sample becomes a one-sample step.
RAGGED_FIT_CASES = {
    "lenet_165_b16_e2": ("lenet_adagrad", 165, 16, 2),
    "cifar_28_b8_e2": ("cifar_adam", 28, 8, 2),
    "lenet_33_b16_e1": ("lenet_adagrad", 33, 16, 1),   # one sample left over
    "tiny_23_b5_e3": ("tiny_conv_adam", 23, 5, 3),
}


def gen_ragged_fit_data(name):
    case, n, B, epochs = RAGGED_FIT_CASES[name]
    c = NET_CASES[case]
    rng = np.random.default_rng(c["seed"] + 2000)
    x = c["xgen"](rng, (n, c["in_dim"])).astype(np.float32)
    t = np.full((n, c["out_dim"]), c["t_lo"], dtype=np.float32)
    t[np.arange(n), rng.integers(0, c["out_dim"], n)] = c["t_hi"]
    return c, x, t, n, B, epochs


# ---- discrete decisions --------------------------------------------------------------------------
# Two fp32 evaluations of the same network that differ only in summation order agree on the
# forward outputs to ~1e-6, but a relu whose input is that close to zero, or a max-pooling window
# whose two largest values are that close, can be DECIDED differently -- and then the whole
# gradient contribution of that position is routed differently (one position's dY * x is not
# small against a tolerance of 1e-3 of the tensor's largest entry).  The functions below find the
# decisions on which two forward passes differ, per output unit (channel / neuron) of the layer
# that owns the gradient, so that a comparison can hold every other unit to the strict tolerance.
def _pool_winners(a, c, h, w):
    """argmax of every 2x2/2 window in window-scan order (first maximum wins, as strict '>' does)."""
    v = a.reshape(-1, c, h // 2, 2, w // 2, 2).transpose(0, 1, 2, 4, 3, 5).reshape(-1, c, h // 2, w // 2, 4)
    return v.argmax(axis=-1)


def decision_mismatch(specs, outs_a, outs_b):
    """{index of a conv / fc layer: bool[out units]} -- units for which the relu gates or the
    2x2 max-pooling winners behind that layer differ between two forward passes; outs_x[i] is
    layer i's output [B][dim] (None where it is not available)."""
    res = {}
    owner = None
    for i, sp in enumerate(specs):
        if sp.kind == LAYER_CONV:
            owner = (i, sp.conv.out_c, sp.conv.out_h, sp.conv.out_w)
            res[i] = np.zeros(sp.conv.out_c, bool)
        elif sp.kind == LAYER_FC:
            owner = (i, sp.fc_out, 1, 1)
            res[i] = np.zeros(sp.fc_out, bool)
        elif sp.kind == LAYER_RELU and owner is not None:
            li, c, h, w = owner
            ga = (outs_a[i] > 0).reshape(-1, c, h * w)
            gb = (outs_b[i] > 0).reshape(-1, c, h * w)
            res[li] |= (ga != gb).any(axis=(0, 2))
        elif sp.kind == LAYER_MAXPOOL and owner is not None:
            li, c, h, w = owner
            if (sp.pool.pool_w, sp.pool.pool_h, sp.pool.stride_w, sp.pool.stride_h) == (2, 2, 2, 2) and \
                    outs_a[i - 1] is not None and outs_b[i - 1] is not None:
                wa, wb = _pool_winners(outs_a[i - 1], c, h, w), _pool_winners(outs_b[i - 1], c, h, w)
                res[li] |= (wa != wb).any(axis=(0, 2, 3))
            owner = None
        elif sp.kind in (LAYER_TANH, LAYER_SOFTMAX, LAYER_AVGPOOL):
            pass
    return res


def entry_units(spec, is_weight, length):
    """output unit (channel / neuron) each entry of a conv / fc parameter tensor belongs to"""
    idx = np.arange(length)
    if not is_weight:
        return idx
    if spec.kind == LAYER_CONV:
        return idx // (spec.conv.in_c * spec.conv.k_h * spec.conv.k_w)
    return idx % spec.fc_out   # fully connected: W[in][out]


def param_layers(specs):
    """layer index of every trainable tensor in update order (as net_layout lists them)"""
    out = []
    for i, sp in enumerate(specs):
        if sp.kind == LAYER_CONV:
            out += [i] * (2 if sp.conv.has_bias else 1)
        elif sp.kind == LAYER_FC:
            out += [i] * (2 if sp.fc_has_bias else 1)
        elif sp.kind == LAYER_AVGPOOL:
            out += [i, i]
    return out
