"""GPU parity tests of the uint8 quantized forward path.  Results are compared
BIT FOR BIT with the oracle restatement and with outputs recorded from the
unmodified reference."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle_lib as o
from cases import (QCONV_CASES, QCONV_ORACLE_ONLY, QEQ_CONV_CASES, QEQ_FC_CASES, QFC_CASES, conv_desc, gen_conv_inputs,
                   gen_qeq_conv_inputs, gen_qeq_fc_inputs)
from tiny_cnn_b200._lib import check, ptr
from test_ops_gpu import dev, host
from tiny_cnn_b200 import ops

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD / "ref_outputs.npz")


def bit_equal(a, b, what):
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    if a.tobytes() != b.tobytes():
        bad = np.flatnonzero(a.view(np.uint32).ravel() != b.view(np.uint32).ravel())
        i = int(bad[0])
        raise AssertionError(f"{what}: {bad.size}/{a.size} floats differ; first at {i}: "
                             f"got {a.ravel()[i]!r} want {b.ravel()[i]!r}")


def padded(oracle, d, x):
    B = x.shape[0]
    xp = o.f32(B, d.in_c * d.inp_h * d.inp_w)
    oracle.orc_conv_pad(C.byref(d), o.p(x), o.p(xp), B)
    return xp


@pytest.mark.parametrize("name", list(QCONV_CASES) + list(QCONV_ORACLE_ONLY))
def test_qconv_bit_exact(ctx, oracle, gold, name):
    c = QCONV_CASES.get(name) or QCONV_ORACLE_ONLY[name]
    d = conv_desc(c)
    x, W, b, _ = gen_conv_inputs(c, d)
    B = x.shape[0]
    xp = padded(oracle, d, x)
    y_ref = o.f32(B, d.out_c * d.out_h * d.out_w)
    assert oracle.orc_qconv2d_fwd(C.byref(d), o.p(xp), o.p(W), o.p(b), o.p(y_ref), B, None, None) == 0
    y = ops.quantized_conv2d(ctx, d, dev(xp), dev(W), dev(b))
    bit_equal(host(y), y_ref, f"{name} vs oracle")
    if name in QCONV_CASES:
        bit_equal(host(y), gold[f"qconv/{name}/y"], f"{name} vs reference")


@pytest.mark.parametrize("name", list(QFC_CASES))
def test_qfc_bit_exact(ctx, oracle, gold, name):
    c = QFC_CASES[name]
    rng = np.random.default_rng(c["seed"])
    B, I, O = c["B"], c["in"], c["out"]
    x = rng.uniform(-1, 1, (B, I)).astype(np.float32)
    W = rng.uniform(-0.5, 0.5, I * O).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, O).astype(np.float32) if c["bias"] else None
    y = ops.quantized_fully_connected(ctx, I, O, dev(x), dev(W), dev(b))
    bit_equal(host(y), gold[f"qfc/{name}/y"], f"{name} vs reference")


@pytest.mark.parametrize("name", list(QEQ_CONV_CASES))
def test_qconv_eq_bit_exact(ctx, oracle, gold, name):
    """tiny_backend::conv2d_eq's kernel: uint8 values held in floats and their ranges in and out."""
    d, x, W, bias, in_r, W_r, b_r = gen_qeq_conv_inputs(name)
    B = x.shape[0]
    y = torch.empty(B, d.out_c * d.out_h * d.out_w, device="cuda")
    yr = torch.empty(B, 2, device="cuda")
    t = [dev(a) for a in (x, W, bias, in_r, W_r, b_r)]
    check(ctx.lib.b200_qconv2d_eq_fwd(ctx.handle, C.byref(d), *[ptr(a) for a in t], ptr(y), ptr(yr), B))
    bit_equal(host(y), gold[f"qconv_eq/{name}/y"], f"{name} values vs reference")
    bit_equal(host(yr), gold[f"qconv_eq/{name}/range"], f"{name} range vs reference")
    yh, yrh = np.empty((B, y.shape[1]), np.float32), np.empty((B, 2), np.float32)
    check(ctx.lib.b200_qconv2d_eq_fwd_host(ctx.handle, C.byref(d), ptr(x), ptr(W), ptr(bias), ptr(in_r), ptr(W_r),
                                           ptr(b_r), ptr(yh), ptr(yrh), B))
    bit_equal(yh, gold[f"qconv_eq/{name}/y"], f"{name} host entry point")
    bit_equal(yrh, gold[f"qconv_eq/{name}/range"], f"{name} host entry point range")


@pytest.mark.parametrize("name", list(QEQ_FC_CASES))
def test_qfc_eq_bit_exact(ctx, oracle, gold, name):
    I, O, x, W, bias, in_r, W_r, b_r = gen_qeq_fc_inputs(name)
    B = x.shape[0]
    y, yr = torch.empty(B, O, device="cuda"), torch.empty(B, 2, device="cuda")
    t = [dev(a) for a in (x, W, bias, in_r, W_r, b_r)]
    check(ctx.lib.b200_qfc_eq_fwd(ctx.handle, I, O, *[ptr(a) for a in t], ptr(y), ptr(yr), B))
    bit_equal(host(y), gold[f"qfc_eq/{name}/y"], f"{name} values vs reference")
    bit_equal(host(yr), gold[f"qfc_eq/{name}/range"], f"{name} range vs reference")
    yh, yrh = np.empty((B, O), np.float32), np.empty((B, 2), np.float32)
    check(ctx.lib.b200_qfc_eq_fwd_host(ctx.handle, I, O, ptr(x), ptr(W), ptr(bias), ptr(in_r), ptr(W_r), ptr(b_r),
                                       ptr(yh), ptr(yrh), B))
    bit_equal(yh, gold[f"qfc_eq/{name}/y"], f"{name} host entry point")
    bit_equal(yrh, gold[f"qfc_eq/{name}/range"], f"{name} host entry point range")


def test_quantized_pipeline_config5(ctx, oracle):
    """Benchmark configuration 5 at a reduced batch: 28x28x32 input U[-1,1], 5x5 -> 64 maps
    stride 2 (12*12*64 = 9216 outputs), then quantized fully connected 9216 -> 256; and the
    stride-1 convolution alone.  Bit-exact against the oracle."""
    rng = np.random.default_rng(505)
    B = 6
    x = rng.uniform(-1, 1, (B, 32 * 28 * 28)).astype(np.float32)
    W = rng.uniform(-0.5, 0.5, 64 * 32 * 25).astype(np.float32)
    for bias in (np.zeros(64, np.float32), rng.uniform(-0.1, 0.1, 64).astype(np.float32)):
        for stride in (1, 2):
            d = ops.conv_params(28, 28, 32, 5, 5, 64, False, True, stride, stride)
            y_ref = o.f32(B, ops.conv_out_len(d))
            assert oracle.orc_qconv2d_fwd(C.byref(d), o.p(x), o.p(W), o.p(bias), o.p(y_ref), B, None, None) == 0
            y = ops.quantized_conv2d(ctx, d, dev(x), dev(W), dev(bias))
            bit_equal(host(y), y_ref, f"cfg5 conv stride {stride}")
        assert y_ref.shape[1] == 9216
        Wf = rng.uniform(-0.5, 0.5, 9216 * 256).astype(np.float32)
        bf = rng.uniform(-0.1, 0.1, 256).astype(np.float32)
        z_ref = o.f32(B, 256)
        assert oracle.orc_qfc_fwd(9216, 256, o.p(y_ref), o.p(Wf), o.p(bf), o.p(z_ref), B) == 0
        z = ops.quantized_fully_connected(ctx, 9216, 256, y, dev(Wf), dev(bf))
        bit_equal(host(z), z_ref, "cfg5 fc")


def test_quantized_edge_inputs(ctx, oracle):
    """Constant rows (min == max) and rows with extreme magnitudes."""
    rng = np.random.default_rng(606)
    I, O, B = 64, 16, 4
    x = rng.uniform(-1, 1, (B, I)).astype(np.float32)
    x[1, :] = 0.25          # constant row: range collapses, everything quantizes to 0
    x[2, :] *= 1e4          # large range
    x[3, :] = np.abs(x[3])  # strictly non-negative row
    W = rng.uniform(-0.5, 0.5, I * O).astype(np.float32)
    b = np.zeros(O, np.float32)
    z_ref = o.f32(B, O)
    assert oracle.orc_qfc_fwd(I, O, o.p(x), o.p(W), o.p(b), o.p(z_ref), B) == 0
    z = ops.quantized_fully_connected(ctx, I, O, dev(x), dev(W), dev(b))
    # row 1 collapses the accumulator range to a point, where the reference divides by zero
    keep = [0, 2, 3]
    bit_equal(host(z)[keep], z_ref[keep], "edge rows")


def test_qconv_rejects_shapes_the_reference_overruns(ctx):
    d = ops.conv_params(8, 12, 2, 3, 3, 4, False, True)  # height > width: range scan overruns
    x = torch.zeros(1, 2 * 96, device="cuda")
    with pytest.raises(ops.B200Error):
        ops.quantized_conv2d(ctx, d, x, torch.zeros(4 * 2 * 9, device="cuda"), torch.zeros(4, device="cuda"))
