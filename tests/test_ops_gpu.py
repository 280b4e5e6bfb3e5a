"""GPU parity tests of the operator entry points: every call goes through the C
ABI (tiny_cnn_b200.ops -> libtinycnn_b200.so) and is compared with the CPU
oracle on the same seeded inputs, and with the reference's recorded outputs.

Tolerances (relative to the largest reference magnitude of the tensor):
forward outputs 1e-4, gradients 1e-3 -- the bounds the reference parity target
states; integer/byte results are compared bit for bit."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle_lib as o
from cases import (BATCHNORM_CASES, DROPOUT_CASES, LRN_CASES, gen_batchnorm_inputs,
                   ACT_CASES, AVGPOOL_CASES, CONV_CASES, FC_CASES, MAXPOOL_CASES, conv_desc,
                   gen_conv_inputs, hyper_for, merge_rows_np, pool_desc)
from test_oracle import orc_conv
from tiny_cnn_b200 import ops
from tiny_cnn_b200._lib import check, ptr

pytestmark = pytest.mark.gpu

FWD_TOL = 1e-4
GRAD_TOL = 1e-3
GOLD = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD / "ref_outputs.npz")


def dev(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def assert_close(got, want, tol, what=""):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    scale = max(float(np.abs(want).max()), 1e-30)
    err = np.abs(got - want)
    bad = err > tol * (np.abs(want) + scale)
    if bad.any():
        i = int(np.argmax(err))
        raise AssertionError(
            f"{what}: {int(bad.sum())}/{bad.size} elements beyond {tol:g}; worst at flat index {i}: "
            f"got {got.flat[i]!r} want {want.flat[i]!r} (max|want| {scale:g}, max err {err.max():g})")


def tiled_applies(c):
    return (c.get("sw", 1) == 1 and c.get("sh", 1) == 1 and c.get("dw", 1) == 1 and c.get("dh", 1) == 1
            and (c["kw"], c["kh"]) in ((3, 3), (5, 5)))


# --------------------------------------------------------------------------- convolution
def tensor_core_applies(c):
    return (c.get("sw", 1) == 1 and c.get("sh", 1) == 1 and c.get("dw", 1) == 1 and c.get("dh", 1) == 1
            and c["kw"] <= 8 and c["kh"] <= 8)


@pytest.mark.parametrize("algo", [1, 2, 3])
@pytest.mark.parametrize("name", list(CONV_CASES))
def test_conv_fwd_bwd(ctx, oracle, gold, name, algo):
    c = CONV_CASES[name]
    if algo == 2 and not tiled_applies(c):
        pytest.skip("tiled kernels take stride 1, dilation 1, 3x3/5x5 only")
    if algo == 3 and not tensor_core_applies(c):
        pytest.skip("tensor-core kernels take stride 1, dilation 1, windows up to 8x8 only")
    d = conv_desc(c, algo=algo)
    x, W, b, dy = gen_conv_inputs(c, d)
    y_ref, dx_ref, dW_ref, db_ref = orc_conv(oracle, d, x, W, b, dy, per_sample=0)
    y = ops.conv2d_op(ctx, d, dev(x), dev(W), dev(b))
    assert_close(host(y), y_ref, FWD_TOL, f"{name} fwd")
    assert_close(host(y), gold[f"conv/{name}/y"], FWD_TOL, f"{name} fwd vs reference")
    dx, dW, db = ops.conv2d_grad_op(ctx, d, dev(x), dev(W), dev(dy))
    assert_close(host(dx), dx_ref, GRAD_TOL, f"{name} dx")
    assert_close(host(dW), dW_ref[0], GRAD_TOL, f"{name} dW")
    assert_close(host(dW), gold[f"conv/{name}/dW_sum"], GRAD_TOL, f"{name} dW vs reference")
    if c["bias"]:
        assert_close(host(db), db_ref[0], GRAD_TOL, f"{name} db")


@pytest.mark.parametrize("name", ["same3x3", "same5x5_rect", "cifar_c2", "stride2_same"])
def test_conv_padded_geometry(ctx, oracle, name):
    """The form Conv2dOp/Conv2dGradOp::compute receive: rows already padded, dX padded."""
    c = CONV_CASES[name]
    d = conv_desc(c, input_is_padded=True)
    x, W, b, dy = gen_conv_inputs(c, d)
    B = x.shape[0]
    pad_len = d.in_c * d.inp_h * d.inp_w
    xp = o.f32(B, pad_len)
    oracle.orc_conv_pad(C.byref(d), o.p(x), o.p(xp), B)
    y_ref = o.f32(B, d.out_c * d.out_h * d.out_w)
    oracle.orc_conv2d_fwd(C.byref(d), o.p(xp), o.p(W), o.p(b), o.p(y_ref), B)
    dxp_ref, dW_ref, db_ref = o.f32(B, pad_len), o.f32(W.size), o.f32(d.out_c)
    oracle.orc_conv2d_bwd(C.byref(d), o.p(xp), o.p(W), o.p(dy), o.p(dxp_ref), o.p(dW_ref), o.p(db_ref), 0, B)
    y = ops.conv2d_op(ctx, d, dev(xp), dev(W), dev(b))
    assert_close(host(y), y_ref, FWD_TOL, f"{name} padded fwd")
    dxp, dW, db = ops.conv2d_grad_op(ctx, d, dev(xp), dev(W), dev(dy))
    assert_close(host(dxp), dxp_ref, GRAD_TOL, f"{name} padded dx")
    assert_close(host(dW), dW_ref, GRAD_TOL, f"{name} padded dW")
    assert_close(host(db), db_ref, GRAD_TOL, f"{name} padded db")


def test_conv_accumulate_and_determinism(ctx, oracle):
    c = CONV_CASES["cifar_c2"]
    d = conv_desc(c)
    x, W, b, dy = gen_conv_inputs(c, d)
    dx1, dW1, db1 = ops.conv2d_grad_op(ctx, d, dev(x), dev(W), dev(dy))
    dx2, dW2, db2 = ops.conv2d_grad_op(ctx, d, dev(x), dev(W), dev(dy))
    assert torch.equal(dW1, dW2) and torch.equal(db1, db2) and torch.equal(dx1, dx2)
    # accumulate != 0 adds onto what is there (the reference never clears dW/db)
    base_W, base_b = torch.full_like(dW1, 0.5), torch.full_like(db1, -0.25)
    _, dW3, db3 = ops.conv2d_grad_op(ctx, d, dev(x), dev(W), dev(dy), dW=base_W.clone(), db=base_b.clone(),
                                     accumulate=True)
    assert_close(host(dW3), host(dW1) + 0.5, GRAD_TOL, "accumulated dW")
    assert_close(host(db3), host(db1) - 0.25, GRAD_TOL, "accumulated db")


def test_conv_empty_batch(ctx):
    c = CONV_CASES["valid3x3"]
    d = conv_desc(c)
    x = torch.empty(0, c["c"] * c["h"] * c["w"], device="cuda")
    W = torch.zeros(c["oc"] * c["c"] * 9, device="cuda")
    b = torch.zeros(c["oc"], device="cuda")
    y = ops.conv2d_op(ctx, d, x, W, b)
    assert y.shape[0] == 0
    dy = torch.empty(0, ops.conv_out_len(d), device="cuda")
    _, dW, db = ops.conv2d_grad_op(ctx, d, x, W, dy, dW=torch.ones_like(W), db=torch.ones_like(b))
    assert float(dW.abs().sum()) == 0.0 and float(db.abs().sum()) == 0.0


def test_conv_rejects_bad_descriptor(ctx):
    d = conv_desc(CONV_CASES["valid3x3"])
    d.out_w = 100  # window leaves the input
    x = torch.zeros(1, 3 * 8 * 8, device="cuda")
    with pytest.raises(ops.B200Error):
        ops.conv2d_op(ctx, d, x, torch.zeros(4 * 3 * 9, device="cuda"), torch.zeros(4, device="cuda"))


def test_conv_tiled_vs_general_full_size(ctx):
    """Benchmark-size layers (batch 256): the tiled kernels against the general
    kernels, which the small cases above tie to the oracle."""
    g = torch.Generator(device="cuda").manual_seed(7)
    for (w, c, oc, k) in [(32, 3, 32, 5), (16, 32, 32, 5), (8, 32, 64, 5), (14, 256, 256, 3)]:
        B = 256 if w != 14 else 32
        x = torch.randn(B, c * w * w, device="cuda", generator=g)
        W = (torch.rand(oc * c * k * k, device="cuda", generator=g) - 0.5) * 0.2
        b = torch.rand(oc, device="cuda", generator=g) - 0.5
        dy = torch.randn(B, oc * w * w, device="cuda", generator=g)
        res = []
        for algo in (1, 2, 3):
            d = ops.conv_params(w, w, c, k, k, oc, True, True, algo=algo)
            y = ops.conv2d_op(ctx, d, x, W, b)
            dx, dW, db = ops.conv2d_grad_op(ctx, d, x, W, dy)
            res.append([host(t) for t in (y, dx, dW, db)])
        for other, label in list(zip(res[1:], ("tiled", "tensor-core"))):
            for a, bb, tol, nm in zip(res[0], other, (FWD_TOL, GRAD_TOL, GRAD_TOL, GRAD_TOL), "y dx dW db".split()):
                assert_close(bb, a, tol, f"{w}x{w}x{c}->{oc} {nm} {label} vs general")


def test_conv_linearity_full_size(ctx):
    """conv(x1 + x2) - bias == (conv(x1) - bias) + (conv(x2) - bias) at CIFAR conv2 size."""
    g = torch.Generator(device="cuda").manual_seed(11)
    d = ops.conv_params(16, 16, 32, 5, 5, 32, True, True)
    x1 = torch.randn(256, 32 * 256, device="cuda", generator=g)
    x2 = torch.randn(256, 32 * 256, device="cuda", generator=g)
    W = (torch.rand(32 * 32 * 25, device="cuda", generator=g) - 0.5) * 0.2
    b = torch.zeros(32, device="cuda")
    y12 = ops.conv2d_op(ctx, d, x1 + x2, W, b)
    y1 = ops.conv2d_op(ctx, d, x1, W, b)
    y2 = ops.conv2d_op(ctx, d, x2, W, b)
    assert_close(host(y12), host(y1 + y2), 1e-4, "linearity")


# --------------------------------------------------------------------------- fully connected
@pytest.mark.parametrize("name", list(FC_CASES))
def test_fc(ctx, oracle, gold, name):
    c = FC_CASES[name]
    rng = np.random.default_rng(c["seed"])
    B, I, O = c["B"], c["in"], c["out"]
    x = rng.uniform(0, 1, (B, I)).astype(np.float32)
    W = rng.uniform(-0.3, 0.3, I * O).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, O).astype(np.float32) if c["bias"] else None
    dy = rng.standard_normal((B, O)).astype(np.float32)
    y = ops.fully_connected_op(ctx, I, O, dev(x), dev(W), dev(b))
    assert_close(host(y), gold[f"fc/{name}/y"], FWD_TOL, f"{name} fwd")
    dx, dW, db = ops.fully_connected_grad_op(ctx, I, O, dev(x), dev(W), dev(dy), has_bias=c["bias"])
    assert_close(host(dx), gold[f"fc/{name}/dx"], GRAD_TOL, f"{name} dx")
    assert_close(host(dW), gold[f"fc/{name}/dW_sum"], GRAD_TOL, f"{name} dW")
    if c["bias"]:
        assert_close(host(db), gold[f"fc/{name}/db_sum"], GRAD_TOL, f"{name} db")


def test_fc_mlp_layer_size(ctx, oracle):
    """784 -> 4096 at batch 64: oracle forward, and dW through the rank-1 identity."""
    rng = np.random.default_rng(5)
    B, I, O = 64, 784, 4096
    x = rng.uniform(0, 1, (B, I)).astype(np.float32)
    W = rng.uniform(-0.05, 0.05, I * O).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, O).astype(np.float32)
    dy = rng.standard_normal((B, O)).astype(np.float32)
    y_ref = o.f32(B, O)
    oracle.orc_fc_fwd(I, O, o.p(x), o.p(W), o.p(b), o.p(y_ref), B)
    y = ops.fully_connected_op(ctx, I, O, dev(x), dev(W), dev(b))
    assert_close(host(y), y_ref, FWD_TOL, "mlp fwd")
    dx_ref, dW_ref, db_ref = o.f32(B, I), o.f32(I * O), o.f32(O)
    oracle.orc_fc_bwd(I, O, o.p(x), o.p(W), o.p(dy), o.p(dx_ref), o.p(dW_ref), o.p(db_ref), 0, B)
    dx, dW, db = ops.fully_connected_grad_op(ctx, I, O, dev(x), dev(W), dev(dy))
    assert_close(host(dx), dx_ref, GRAD_TOL, "mlp dx")
    assert_close(host(dW), dW_ref, GRAD_TOL, "mlp dW")
    assert_close(host(db), db_ref, GRAD_TOL, "mlp db")


@pytest.mark.parametrize("B,I,O", [(128, 784, 4096), (200, 4096, 330), (256, 1024, 64)])
def test_fc_tensor_core_path(ctx, oracle, B, I, O):
    """The 3xTF32 tensor-core GEMMs (forced on) against the oracle at the forward /
    gradient tolerances, ragged extents included."""
    rng = np.random.default_rng(17)
    x = rng.uniform(0, 1, (B, I)).astype(np.float32)
    W = rng.uniform(-0.05, 0.05, I * O).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, O).astype(np.float32)
    dy = rng.standard_normal((B, O)).astype(np.float32)
    y_ref = o.f32(B, O)
    oracle.orc_fc_fwd(I, O, o.p(x), o.p(W), o.p(b), o.p(y_ref), B)
    dx_ref, dW_ref, db_ref = o.f32(B, I), o.f32(I * O), o.f32(O)
    oracle.orc_fc_bwd(I, O, o.p(x), o.p(W), o.p(dy), o.p(dx_ref), o.p(dW_ref), o.p(db_ref), 0, B)
    check(ctx.lib.b200_ctx_set_option(ctx.handle, b"fc_tensor_cores", 2))
    try:
        y = ops.fully_connected_op(ctx, I, O, dev(x), dev(W), dev(b))
        dx, dW, db = ops.fully_connected_grad_op(ctx, I, O, dev(x), dev(W), dev(dy))
        ctx.sync()
    finally:
        check(ctx.lib.b200_ctx_set_option(ctx.handle, b"fc_tensor_cores", 1))
    assert_close(host(y), y_ref, FWD_TOL, "tc fwd")
    assert_close(host(dx), dx_ref, GRAD_TOL, "tc dx")
    assert_close(host(dW), dW_ref, GRAD_TOL, "tc dW")
    assert_close(host(db), db_ref, GRAD_TOL, "tc db")
    # the hi/lo split keeps fp32-level accuracy: a single-pass TF32 product would sit near 1e-3
    assert np.abs(host(y) - y_ref).max() <= 5e-5 * np.abs(y_ref).max()


# --------------------------------------------------------------------------- pooling
@pytest.mark.parametrize("name", list(MAXPOOL_CASES))
def test_maxpool(ctx, oracle, gold, name):
    c = MAXPOOL_CASES[name]
    d = pool_desc(c)
    rng = np.random.default_rng(c["seed"])
    B = c["B"]
    x = rng.standard_normal((B, d.in_c * d.in_h * d.in_w)).astype(np.float32)
    n_out = d.in_c * d.out_h * d.out_w
    dy = rng.standard_normal((B, n_out)).astype(np.float32)
    y_ref, arg_ref = o.f32(B, n_out), np.zeros((B, n_out), dtype=np.int32)
    oracle.orc_maxpool_fwd(C.byref(d), o.p(x), o.p(y_ref), o.p(arg_ref), B)
    y, arg = ops.maxpool_op(ctx, d, dev(x))
    assert np.array_equal(host(y), y_ref) and np.array_equal(host(y), gold[f"maxpool/{name}/y"])
    assert np.array_equal(host(arg), arg_ref)
    dx = ops.maxpool_grad_op(ctx, d, dev(dy), arg)
    assert np.array_equal(host(dx), gold[f"maxpool/{name}/dx"])


def test_maxpool_ties(ctx, oracle):
    """Equal values: the first element of the window scan wins (strict '>')."""
    d = ops.maxpool_params(4, 4, 2, 2)
    x = np.ones((2, 32), dtype=np.float32)
    y_ref, arg_ref = o.f32(2, 8), np.zeros((2, 8), dtype=np.int32)
    oracle.orc_maxpool_fwd(C.byref(d), o.p(x), o.p(y_ref), o.p(arg_ref), 2)
    y, arg = ops.maxpool_op(ctx, d, dev(x))
    assert np.array_equal(host(arg), arg_ref)


@pytest.mark.parametrize("name", list(AVGPOOL_CASES))
def test_avgpool(ctx, oracle, gold, name):
    c = AVGPOOL_CASES[name]
    d = pool_desc(c)
    rng = np.random.default_rng(c["seed"])
    B = c["B"]
    x = rng.standard_normal((B, d.in_c * d.in_h * d.in_w)).astype(np.float32)
    wlen = d.pool_w * d.pool_h * d.in_c
    W = rng.uniform(0.5, 1.5, wlen).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, d.in_c).astype(np.float32)
    n_out = d.in_c * d.out_h * d.out_w
    dy = rng.standard_normal((B, n_out)).astype(np.float32)
    y = ops.average_pooling_forward(ctx, d, dev(x), dev(W), dev(b))
    assert_close(host(y), gold[f"avgpool/{name}/y"], FWD_TOL, f"{name} fwd")
    dx, dW, db = ops.average_pooling_backward(ctx, d, dev(x), dev(W), dev(dy))
    assert_close(host(dx), gold[f"avgpool/{name}/dx"], GRAD_TOL, f"{name} dx")
    assert_close(host(dW), gold[f"avgpool/{name}/dW_sum"], GRAD_TOL, f"{name} dW")
    assert_close(host(db), gold[f"avgpool/{name}/db_sum"], GRAD_TOL, f"{name} db")
    assert float(dW[d.in_c:].abs().sum()) == 0.0  # unused weight slots get no gradient


def test_avgpool_rejects_uncovered_inputs(ctx):
    d = ops.maxpool_params(9, 9, 1, 2, 2, 3, 3)  # stride > pool: some inputs lie in no window
    x = torch.zeros(1, 81, device="cuda")
    with pytest.raises(ops.B200Error):
        ops.average_pooling_forward(ctx, d, x, torch.ones(4, device="cuda"), torch.zeros(1, device="cuda"))


# --------------------------------------------------------------------------- activations / loss
@pytest.mark.parametrize("name", list(ACT_CASES))
def test_activation_and_loss(ctx, gold, name):
    c = ACT_CASES[name]
    rng = np.random.default_rng(c["seed"])
    B, dim = c["B"], c["dim"]
    x = (rng.standard_normal((B, dim)) * c.get("scale", 1.0)).astype(np.float32)
    dy = rng.standard_normal((B, dim)).astype(np.float32)
    y = ops.forward_activation(ctx, c["kind"], dev(x), c.get("param"))
    assert_close(host(y), gold[f"act/{name}/y"], FWD_TOL, f"{name} fwd")
    dx = ops.backward_activation(ctx, c["kind"], dev(gold[f"act/{name}/y"]), dev(dy), c.get("param"))
    assert_close(host(dx), gold[f"act/{name}/dx"], GRAD_TOL, f"{name} bwd")
    for loss in (0, 1, 2):
        yy, tt = gold[f"loss/{name}/{loss}/y"], gold[f"loss/{name}/{loss}/t"]
        g = ops.gradient(ctx, loss, dev(yy), dev(tt))
        assert_close(host(g), gold[f"loss/{name}/{loss}/g"], 1e-6, f"{name} loss {loss}")


# --------------------------------------------------------------------------- batch norm / lrn / dropout
@pytest.mark.parametrize("name", list(BATCHNORM_CASES))
def test_batchnorm(ctx, gold, name):
    """Forward (train and test phase) and backward against the reference's recorded outputs: 1e-4 / 1e-3
    (the per-channel sums are formed by a tree here, sample by sample in the reference)."""
    c = BATCHNORM_CASES[name]
    x, dy, run_mean, run_var = gen_batchnorm_inputs(c)
    Cn, S = c["C"], c["S"]
    y, mean, var, sd = ops.batch_normalization_forward(ctx, Cn, S, c["eps"], dev(x), train=True)
    assert_close(host(y), gold[f"batchnorm/{name}/train/y"], FWD_TOL, f"{name} train y")
    assert_close(host(mean), gold[f"batchnorm/{name}/train/mean"], FWD_TOL, f"{name} mean")
    assert_close(host(var), gold[f"batchnorm/{name}/train/var"], FWD_TOL, f"{name} variance")
    assert_close(host(sd), gold[f"batchnorm/{name}/train/stddev"], FWD_TOL, f"{name} stddev")
    dx = ops.batch_normalization_backward(ctx, Cn, S, dev(gold[f"batchnorm/{name}/train/y"]), dev(dy),
                                          dev(gold[f"batchnorm/{name}/train/stddev"]))
    assert_close(host(dx), gold[f"batchnorm/{name}/train/dx"], GRAD_TOL, f"{name} train dx")
    y2, _, _, sd2 = ops.batch_normalization_forward(ctx, Cn, S, c["eps"], dev(x), dev(run_mean), dev(run_var),
                                                    train=False)
    assert_close(host(y2), gold[f"batchnorm/{name}/test/y"], FWD_TOL, f"{name} test y")
    assert np.array_equal(host(sd2), gold[f"batchnorm/{name}/test/stddev"])
    # host-row entry points give the device entry points' bits
    yh, mh, vh, sh = (np.empty_like(x), np.empty(Cn, np.float32), np.empty(Cn, np.float32), np.empty(Cn, np.float32))
    check(ctx.lib.b200_batchnorm_fwd_host(ctx.handle, Cn, S, c["eps"], ptr(x), ptr(mh), ptr(vh), ptr(sh), ptr(yh),
                                          c["B"], 1))
    assert np.array_equal(yh, host(y)) and np.array_equal(mh, host(mean)) and np.array_equal(sh, host(sd))
    dxh = np.empty_like(x)
    yg, sg = gold[f"batchnorm/{name}/train/y"], gold[f"batchnorm/{name}/train/stddev"]
    check(ctx.lib.b200_batchnorm_bwd_host(ctx.handle, Cn, S, ptr(yg), ptr(dy), ptr(sg), ptr(dxh), c["B"]))
    assert np.array_equal(dxh, host(dx))


def test_batchnorm_post_update(ctx, oracle):
    rng = np.random.default_rng(5)
    mean, var, mc, vc = (rng.standard_normal(7).astype(np.float32) for _ in range(4))
    dm, dv, dmc, dvc = dev(mean), dev(var), dev(mc), dev(vc)
    check(ctx.lib.b200_batchnorm_post_update(ctx.handle, 7, 0.999, ptr(dm), ptr(dv), ptr(dmc), ptr(dvc)))
    oracle.orc_batchnorm_post_update(7, 0.999, o.p(mean), o.p(var), o.p(mc), o.p(vc))
    assert np.array_equal(host(dm), mean) and np.array_equal(host(dv), var)


@pytest.mark.parametrize("name", list(LRN_CASES))
def test_lrn_forward(ctx, gold, name):
    c = LRN_CASES[name]
    rng = np.random.default_rng(c["seed"])
    x = rng.standard_normal((c["B"], c["C"] * c["w"] * c["h"])).astype(np.float32)
    y = ops.lrn_forward(ctx, dev(x), c["C"], c["w"] * c["h"], c["size"], c["alpha"], c["beta"])
    assert_close(host(y), gold[f"lrn/{name}/y"], FWD_TOL, f"lrn {name}")
    yh = np.empty_like(x)
    check(ctx.lib.b200_lrn_fwd_host(ctx.handle, ptr(x), ptr(yh), c["C"], c["w"] * c["h"], c["size"], c["alpha"],
                                    c["beta"], c["B"]))
    assert np.array_equal(yh, host(y))


@pytest.mark.parametrize("name", list(DROPOUT_CASES))
def test_dropout_with_the_reference_mask(ctx, gold, name):
    """Bit for bit given the mask the reference drew."""
    c = DROPOUT_CASES[name]
    rng = np.random.default_rng(c["seed"])
    x = rng.standard_normal((c["B"], c["dim"])).astype(np.float32)
    dy = rng.standard_normal((c["B"], c["dim"])).astype(np.float32)
    mask = gold[f"dropout/{name}/mask"]
    scale = float(np.float32(1) / (np.float32(1) - np.float32(c["rate"])))
    dm = torch.from_numpy(np.ascontiguousarray(mask)).cuda()
    assert np.array_equal(host(ops.dropout(ctx, dev(x), dm, scale)), gold[f"dropout/{name}/y"])
    assert np.array_equal(host(ops.dropout(ctx, dev(dy), dm, 1.0)), gold[f"dropout/{name}/dx"])
    yh = np.empty_like(x)
    check(ctx.lib.b200_dropout_host(ctx.handle, ptr(x), ptr(np.ascontiguousarray(mask)), scale, ptr(yh), x.size))
    assert np.array_equal(yh, gold[f"dropout/{name}/y"])


def test_loss_value(ctx, oracle):
    rng = np.random.default_rng(3)
    y = rng.uniform(0.05, 0.95, (32, 10)).astype(np.float32)
    t = (rng.random((32, 10)) > 0.8).astype(np.float32)
    for loss in (0, 1, 2):
        want = oracle.orc_loss_value(loss, o.p(y), o.p(t), 10, 32)
        got = float(ops.loss_value(ctx, loss, dev(y), dev(t))[0])
        assert abs(got - want) <= 1e-4 * abs(want)


# --------------------------------------------------------------------------- merge + optimizer
@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4, 5, 6])
def test_optimizer_steps(ctx, gold, kind):
    W, g = dev(gold["opt/W0"].copy()), dev(gold["opt/g"])
    s0, s1 = torch.zeros_like(W), torch.zeros_like(W)
    h = hyper_for(kind)
    for _ in range(5):
        ops.optimizer_update(ctx, kind, h, g, W, s0, s1)
        if kind in (1, 4):
            h.b1_t = np.float32(h.b1_t) * np.float32(h.b1)
            h.b2_t = np.float32(h.b2_t) * np.float32(h.b2)
    # same rounding sequence as the reference: bit-identical
    assert np.array_equal(host(W), gold[f"opt/{kind}/W5"])


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4, 5, 6])
def test_merge_update(ctx, oracle, kind):
    rng = np.random.default_rng(9)
    rows, n = 16, 5000
    grads = rng.standard_normal((rows, n)).astype(np.float32)
    W0 = rng.standard_normal(n).astype(np.float32)
    merged_ref = o.f32(n)
    oracle.orc_merge_grads(o.p(grads), rows, n, o.p(merged_ref))
    assert np.array_equal(host(ops.merge_grads(ctx, dev(grads))), merged_ref)
    W_ref, s0_ref, s1_ref = W0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
    h = hyper_for(kind)
    oracle.orc_opt_update(kind, C.byref(h), o.p(merged_ref), o.p(W_ref), o.p(s0_ref), o.p(s1_ref), n)
    W, s0, s1 = dev(W0.copy()), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    merged = torch.empty(n, device="cuda")
    ops.merge_update(ctx, kind, h, dev(grads), W, s0, s1, merged)
    assert np.array_equal(host(merged), merged_ref)
    assert np.array_equal(host(W), W_ref)
    assert np.array_equal(host(s0), s0_ref)


# --------------------------------------------------------------------------- HOST-buffer entry points
def test_host_entry_points(ctx, oracle):
    c = CONV_CASES["same5x5_rect"]
    d = conv_desc(c)
    x, W, b, dy = gen_conv_inputs(c, d)
    B = x.shape[0]
    y_ref, dx_ref, dW_ref, db_ref = orc_conv(oracle, d, x, W, b, dy, per_sample=0)
    lib = ctx.lib
    y = o.f32(*y_ref.shape)
    check(lib.b200_conv2d_fwd_host(ctx.handle, C.byref(d), ptr(x), ptr(W), ptr(b), ptr(y), B))
    assert_close(y, y_ref, FWD_TOL, "host conv fwd")
    dx, dW, db = o.f32(*x.shape), np.full(W.size, 1.0, np.float32), np.full(d.out_c, 2.0, np.float32)
    check(lib.b200_conv2d_bwd_host(ctx.handle, C.byref(d), ptr(x), ptr(W), ptr(dy), ptr(dx), ptr(dW),
                                   ptr(db), 1, B))
    assert_close(dx, dx_ref, GRAD_TOL, "host conv dx")
    assert_close(dW, dW_ref[0] + 1.0, GRAD_TOL, "host conv dW (accumulated)")
    assert_close(db, db_ref[0] + 2.0, GRAD_TOL, "host conv db (accumulated)")
    # fully connected
    rng = np.random.default_rng(1)
    xi = rng.uniform(0, 1, (4, 30)).astype(np.float32)
    Wf = rng.uniform(-0.3, 0.3, 30 * 12).astype(np.float32)
    bf = rng.uniform(-0.1, 0.1, 12).astype(np.float32)
    yf_ref, yf = o.f32(4, 12), o.f32(4, 12)
    oracle.orc_fc_fwd(30, 12, o.p(xi), o.p(Wf), o.p(bf), o.p(yf_ref), 4)
    check(lib.b200_fc_fwd_host(ctx.handle, 30, 12, ptr(xi), ptr(Wf), ptr(bf), ptr(yf), 4))
    assert_close(yf, yf_ref, FWD_TOL, "host fc fwd")
    # max pooling round trip
    pd = ops.maxpool_params(8, 8, 3, 2)
    xm = rng.standard_normal((2, 192)).astype(np.float32)
    ym_ref, am_ref = o.f32(2, 48), np.zeros((2, 48), np.int32)
    oracle.orc_maxpool_fwd(C.byref(pd), o.p(xm), o.p(ym_ref), o.p(am_ref), 2)
    ym, am = o.f32(2, 48), np.zeros((2, 48), np.int32)
    check(lib.b200_maxpool_fwd_host(ctx.handle, C.byref(pd), ptr(xm), ptr(ym), ptr(am), 2))
    assert np.array_equal(ym, ym_ref) and np.array_equal(am, am_ref)
