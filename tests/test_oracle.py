"""Pins the CPU oracle (oracle/oracle.c):

  * against the known-answer vectors of the reference's own unit tests
    (tests/golden/reference_kats.json), and
  * against outputs of the unmodified reference recorded in
    tests/golden/ref_outputs.npz (tests/golden/make_golden.py), bit for bit.

Runs without a GPU."""
import ctypes as C
import json
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as o
from cases import (BATCHNORM_CASES, DROPOUT_CASES, LRN_CASES, QEQ_CONV_CASES, QEQ_FC_CASES, bn_layers,
                   gen_batchnorm_inputs, gen_qeq_conv_inputs, gen_qeq_fc_inputs,
                   ACT_CASES, AVGPOOL_CASES, CONV_CASES, FC_CASES, MAXPOOL_CASES, NET_CASES,
                   QCONV_CASES, QFC_CASES, build_net_specs, conv_desc, gen_conv_inputs, gen_net_data,
                   hyper_for, merge_rows_np, pool_desc, xavier_params)
from tiny_cnn_b200.ops import conv_params, hyper, maxpool_params

GOLD = Path(__file__).parent / "golden"
KATS = json.loads((GOLD / "reference_kats.json").read_text())


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD / "ref_outputs.npz")


def a32(v):
    return np.asarray(v, dtype=np.float32)


# --------------------------------------------------------------------------- helpers
def orc_conv(orc, d, x, W, b, dy=None, per_sample=1):
    B = x.shape[0]
    pad_len = d.in_c * d.inp_h * d.inp_w
    xp = o.f32(B, pad_len)
    orc.orc_conv_pad(C.byref(d), o.p(x), o.p(xp), B)
    y = o.f32(B, d.out_c * d.out_h * d.out_w)
    orc.orc_conv2d_fwd(C.byref(d), o.p(xp), o.p(W), o.p(b), o.p(y), B)
    if dy is None:
        return y
    rows = B if per_sample else 1
    dxp, dW, db = o.f32(B, pad_len), o.f32(rows, W.size), o.f32(rows, d.out_c)
    orc.orc_conv2d_bwd(C.byref(d), o.p(xp), o.p(W), o.p(dy), o.p(dxp), o.p(dW), o.p(db), per_sample, B)
    dx = o.f32(*x.shape)
    orc.orc_conv_unpad(C.byref(d), o.p(dxp), o.p(dx), B)
    return y, dx, dW, db


# --------------------------------------------------------------------------- KATs
def test_kat_conv_fprop(oracle):
    k = KATS["conv_fprop"]
    d = conv_params(5, 5, 1, 3, 3, 2, False, True)
    y = orc_conv(oracle, d, a32(k["in"])[None], a32(k["weight"]), a32(k["bias"]))
    np.testing.assert_allclose(y[0, :9], k["out_first9"], atol=k["tol"])


def test_kat_conv_with_stride(oracle):
    k = KATS["conv_with_stride"]
    d = conv_params(5, 5, 1, 3, 3, 1, False, True, 2, 2)
    y, dx, dW, db = orc_conv(oracle, d, a32(k["in"])[None], a32(k["weight"]), a32(k["bias"]),
                             a32(k["curr_delta"])[None])
    assert y[0].tolist() == k["out"]
    assert dx[0].tolist() == k["prev_delta"]
    assert dW[0].tolist() == k["dw"]
    assert db[0].tolist() == k["db"]


def test_kat_conv_with_dilation(oracle):
    k = KATS["conv_with_dilation"]
    d = conv_params(7, 7, 1, 3, 3, 1, False, True, 1, 1, 2, 2)
    x = np.arange(k["in_arange"], dtype=np.float32)[None]
    y = orc_conv(oracle, d, x, a32(k["weight"]), a32(k["bias"]))
    np.testing.assert_allclose(y[0], k["out"], atol=k["tol"])


@pytest.mark.parametrize("name", ["fc_forward", "fc_forward_nobias"])
def test_kat_fc(oracle, name):
    k = KATS[name]
    I, O = k["in_size"], k["out_size"]
    W = np.full(I * O, k["weight_const"], dtype=np.float32)
    b = np.full(O, k["bias_const"], dtype=np.float32) if "bias_const" in k else None
    y = o.f32(1, O)
    oracle.orc_fc_fwd(I, O, o.p(a32(k["in"])), o.p(W), o.p(b), o.p(y), 1)
    assert y[0].tolist() == k["out"]


def test_kat_max_pool(oracle):
    k = KATS["max_pool"]
    x = a32(k["in"])[None]
    for c in k["cases"]:
        d = maxpool_params(4, 4, 1, c["pool_w"], c["pool_h"], c["stride_w"], c["stride_h"], False,
                           c["pad_same"])
        n = d.out_w * d.out_h
        assert n == len(c["out"]), c["name"]
        y, arg = o.f32(1, n), np.zeros((1, n), dtype=np.int32)
        oracle.orc_maxpool_fwd(C.byref(d), o.p(x), o.p(y), o.p(arg), 1)
        assert y[0].tolist() == c["out"], c["name"]
    b = k["backward"]
    d = maxpool_params(4, 4, 1, b["pool"])
    y, arg, dx = o.f32(1, 4), np.zeros((1, 4), dtype=np.int32), o.f32(1, 16)
    oracle.orc_maxpool_fwd(C.byref(d), o.p(x), o.p(y), o.p(arg), 1)
    oracle.orc_maxpool_bwd(C.byref(d), o.p(a32(b["out_grad"])), o.p(arg), o.p(dx), 1)
    assert dx[0].tolist() == b["in_grad"]


def test_kat_ave_pool(oracle):
    k = KATS["ave_pool"]
    x = a32(k["in"])[None]
    for c in k["cases"]:
        d = maxpool_params(4, 4, 1, c["pool"], c["pool"], c["stride"], c["stride"])
        n = d.out_w * d.out_h
        W = np.ones(c["pool"] * c["pool"], dtype=np.float32)
        bias = np.zeros(1, dtype=np.float32)
        y = o.f32(1, n)
        oracle.orc_avgpool_fwd(C.byref(d), o.p(x), o.p(W), o.p(bias), o.p(y), 1)
        np.testing.assert_allclose(y[0], c["out"], rtol=1e-6)


@pytest.mark.parametrize("name,kind", [("adagrad", 0), ("adam", 1), ("momentum", 2)])
def test_kat_optimizers(oracle, name, kind):
    k = KATS["optimizers"][name]
    W, g = a32(k["weights"]).copy(), a32(k["gradients"])
    s0, s1 = np.zeros_like(W), np.zeros_like(W)
    h = hyper_for(kind)
    for expect in (k["first"], k["second"]):
        oracle.orc_opt_update(kind, C.byref(h), o.p(g), o.p(W), o.p(s0), o.p(s1), W.size)
        if kind == 1:  # adam::update advances its powers after every call
            h.b1_t = np.float32(h.b1_t) * np.float32(h.b1)
            h.b2_t = np.float32(h.b2_t) * np.float32(h.b2)
        np.testing.assert_allclose(W, expect, atol=KATS["optimizers"]["tol"])


def test_kat_quantization(oracle):
    q = KATS["quantization"]
    for x, mn, mx, want in q["float_to_quantized_u8"]:
        assert oracle.orc_f2q(8, x, mn, mx) == want
    for x, mn, mx, want in q["float_to_quantized_i32"]:
        assert oracle.orc_f2q(32, x, mn, mx) == want
    t = q["float_tensor_to_quantized"]
    assert [oracle.orc_f2q(8, v, t["min"], t["max"]) for v in t["in"]] == t["out"]
    t = q["quantized_tensor_to_float"]
    assert [oracle.orc_q2f(8, v, t["min"], t["max"]) for v in t["in"]] == t["out"]
    t = q["quantize_down_and_shrink_range"]
    src = np.asarray(t["in"], dtype=np.int32)
    dst = np.zeros(3, dtype=np.uint8)
    mn, mx = C.c_float(), C.c_float()
    oracle.orc_quantize_down_and_shrink_range(o.p(src), 3, t["min"], t["max"], C.byref(mn), C.byref(mx),
                                              o.p(dst))
    assert dst.tolist() == t["out"]
    assert abs(mn.value - t["min_new"]) < t["tol"] and abs(mx.value - t["max_new"]) < t["tol"]
    # requantize_many_in_new_range_32_to_8bit: the fixed-point path must agree with
    # the float path element by element
    t = q["requantize_32_to_8"]
    for imn, imx, omn, omx in t["ranges"]:
        vals = np.asarray([oracle.orc_f2q(32, v, imn, imx) for v in t["values"]], dtype=np.int32)
        want = [oracle.orc_f2q(8, oracle.orc_q2f(32, int(v), imn, imx), omn, omx) for v in vals]
        got = np.zeros(len(vals), dtype=np.uint8)
        oracle.orc_requantize_many_i32_u8(o.p(vals), len(vals), imn, imx, omn, omx, o.p(got))
        assert got.tolist() == want


@pytest.mark.parametrize("bias", [True, False])
def test_kat_quantized_fc(oracle, bias):
    k = KATS["quantized_fc"]
    W = np.full(8, k["weight_const"], dtype=np.float32)
    b = np.full(2, k["bias_const"], dtype=np.float32) if bias else None
    y = o.f32(1, 2)
    assert oracle.orc_qfc_fwd(4, 2, o.p(a32(k["in"])), o.p(W), o.p(b), o.p(y), 1) == 0
    want = 6.5 if bias else 6.0
    np.testing.assert_allclose(y[0], [want, want], atol=k["tol"])


# --------------------------------------------------------------------------- goldens
@pytest.mark.parametrize("name", list(CONV_CASES))
def test_gold_conv(oracle, gold, name):
    c = CONV_CASES[name]
    d = conv_desc(c)
    x, W, b, dy = gen_conv_inputs(c, d)
    y, dx, dW, db = orc_conv(oracle, d, x, W, b, dy)
    assert np.array_equal(y, gold[f"conv/{name}/y"])
    assert np.array_equal(dx, gold[f"conv/{name}/dx"])
    assert np.array_equal(merge_rows_np(dW), gold[f"conv/{name}/dW_sum"])
    if c["bias"]:
        assert np.array_equal(merge_rows_np(db), gold[f"conv/{name}/db_sum"])
    if f"conv/{name}/dW_rows" in gold:
        assert np.array_equal(dW, gold[f"conv/{name}/dW_rows"])
    # the merged form of the oracle equals merge_grads over its own rows
    _, _, dWs, dbs = orc_conv(oracle, d, x, W, b, dy, per_sample=0)
    assert np.array_equal(dWs[0], merge_rows_np(dW))
    if c["bias"]:
        assert np.array_equal(dbs[0], merge_rows_np(db))


@pytest.mark.parametrize("name", list(FC_CASES))
def test_gold_fc(oracle, gold, name):
    c = FC_CASES[name]
    rng = np.random.default_rng(c["seed"])
    B, I, O = c["B"], c["in"], c["out"]
    x = rng.uniform(0, 1, (B, I)).astype(np.float32)
    W = rng.uniform(-0.3, 0.3, I * O).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, O).astype(np.float32) if c["bias"] else None
    dy = rng.standard_normal((B, O)).astype(np.float32)
    y = o.f32(B, O)
    oracle.orc_fc_fwd(I, O, o.p(x), o.p(W), o.p(b), o.p(y), B)
    assert np.array_equal(y, gold[f"fc/{name}/y"])
    dx, dW, db = o.f32(B, I), o.f32(B, I * O), o.f32(B, O)
    oracle.orc_fc_bwd(I, O, o.p(x), o.p(W), o.p(dy), o.p(dx), o.p(dW), o.p(db) if c["bias"] else None, 1, B)
    assert np.array_equal(dx, gold[f"fc/{name}/dx"])
    assert np.array_equal(merge_rows_np(dW), gold[f"fc/{name}/dW_sum"])
    if c["bias"]:
        assert np.array_equal(merge_rows_np(db), gold[f"fc/{name}/db_sum"])


@pytest.mark.parametrize("name", list(MAXPOOL_CASES))
def test_gold_maxpool(oracle, gold, name):
    c = MAXPOOL_CASES[name]
    d = pool_desc(c)
    rng = np.random.default_rng(c["seed"])
    B = c["B"]
    x = rng.standard_normal((B, d.in_c * d.in_h * d.in_w)).astype(np.float32)
    n_out = d.in_c * d.out_h * d.out_w
    dy = rng.standard_normal((B, n_out)).astype(np.float32)
    y, arg, dx = o.f32(B, n_out), np.zeros((B, n_out), dtype=np.int32), o.f32(*x.shape)
    oracle.orc_maxpool_fwd(C.byref(d), o.p(x), o.p(y), o.p(arg), B)
    oracle.orc_maxpool_bwd(C.byref(d), o.p(dy), o.p(arg), o.p(dx), B)
    assert np.array_equal(y, gold[f"maxpool/{name}/y"])
    assert np.array_equal(dx, gold[f"maxpool/{name}/dx"])


@pytest.mark.parametrize("name", list(AVGPOOL_CASES))
def test_gold_avgpool(oracle, gold, name):
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
    y, dx, dW, db = o.f32(B, n_out), o.f32(*x.shape), o.f32(B, wlen), o.f32(B, d.in_c)
    oracle.orc_avgpool_fwd(C.byref(d), o.p(x), o.p(W), o.p(b), o.p(y), B)
    oracle.orc_avgpool_bwd(C.byref(d), o.p(x), o.p(W), o.p(dy), o.p(dx), o.p(dW), o.p(db), 1, B)
    assert np.array_equal(y, gold[f"avgpool/{name}/y"])
    assert np.array_equal(dx, gold[f"avgpool/{name}/dx"])
    assert np.array_equal(merge_rows_np(dW), gold[f"avgpool/{name}/dW_sum"])
    assert np.array_equal(merge_rows_np(db), gold[f"avgpool/{name}/db_sum"])


@pytest.mark.parametrize("name", list(ACT_CASES))
def test_gold_act_and_loss(oracle, gold, name):
    c = ACT_CASES[name]
    rng = np.random.default_rng(c["seed"])
    B, dim = c["B"], c["dim"]
    x = (rng.standard_normal((B, dim)) * c.get("scale", 1.0)).astype(np.float32)
    dy = rng.standard_normal((B, dim)).astype(np.float32)
    y, dx = o.f32(B, dim), o.f32(B, dim)
    if "param" in c:
        oracle.orc_act_param_fwd(c["kind"], c["param"], o.p(x), o.p(y), dim, B)
        oracle.orc_act_param_bwd(c["kind"], c["param"], o.p(y), o.p(dy), o.p(dx), dim, B)
    else:
        oracle.orc_act_fwd(c["kind"], o.p(x), o.p(y), dim, B)
        oracle.orc_act_bwd(c["kind"], o.p(y), o.p(dy), o.p(dx), dim, B)
    assert np.array_equal(y, gold[f"act/{name}/y"])
    assert np.array_equal(dx, gold[f"act/{name}/dx"])
    for loss in (0, 1, 2):
        yy, tt = gold[f"loss/{name}/{loss}/y"], gold[f"loss/{name}/{loss}/t"]
        g = o.f32(B, dim)
        oracle.orc_loss_grad(loss, o.p(yy), o.p(tt), o.p(g), dim, B)
        assert np.array_equal(g, gold[f"loss/{name}/{loss}/g"])


@pytest.mark.parametrize("name", list(BATCHNORM_CASES))
def test_gold_batchnorm(oracle, gold, name):
    """batch_normalization_layer forward (both phases) and backward: bit for bit."""
    c = BATCHNORM_CASES[name]
    x, dy, run_mean, run_var = gen_batchnorm_inputs(c)
    Cn, S, B = c["C"], c["S"], c["B"]
    for phase, train in (("train", 1), ("test", 0)):
        mean, var = (o.f32(Cn), o.f32(Cn)) if train else (run_mean.copy(), run_var.copy())
        sd, y, dx = o.f32(Cn), o.f32(*x.shape), o.f32(*x.shape)
        oracle.orc_batchnorm_fwd(Cn, S, c["eps"], o.p(x), o.p(mean), o.p(var), o.p(sd), o.p(y), B, train)
        oracle.orc_batchnorm_bwd(Cn, S, o.p(y), o.p(dy), o.p(sd), o.p(dx), B)
        assert np.array_equal(y, gold[f"batchnorm/{name}/{phase}/y"])
        assert np.array_equal(sd, gold[f"batchnorm/{name}/{phase}/stddev"])
        assert np.array_equal(dx, gold[f"batchnorm/{name}/{phase}/dx"])
        if train:
            assert np.array_equal(mean, gold[f"batchnorm/{name}/train/mean"])
            assert np.array_equal(var, gold[f"batchnorm/{name}/train/var"])


def test_batchnorm_post_update(oracle):
    """mean = m*mean + (1-m)*mean_cur (batch_normalization_layer.h:174-180)."""
    rng = np.random.default_rng(5)
    mean, var, mc, vc = (rng.standard_normal(7).astype(np.float32) for _ in range(4))
    want_m = np.float32(0.999) * mean + (np.float32(1) - np.float32(0.999)) * mc
    want_v = np.float32(0.999) * var + (np.float32(1) - np.float32(0.999)) * vc
    oracle.orc_batchnorm_post_update(7, 0.999, o.p(mean), o.p(var), o.p(mc), o.p(vc))
    assert np.array_equal(mean, want_m) and np.array_equal(var, want_v)


@pytest.mark.parametrize("name", list(LRN_CASES))
def test_gold_lrn(oracle, gold, name):
    c = LRN_CASES[name]
    rng = np.random.default_rng(c["seed"])
    x = rng.standard_normal((c["B"], c["C"] * c["w"] * c["h"])).astype(np.float32)
    y = o.f32(*x.shape)
    oracle.orc_lrn_fwd(o.p(x), o.p(y), c["C"], c["w"] * c["h"], c["size"], c["alpha"], c["beta"], c["B"])
    assert np.array_equal(y, gold[f"lrn/{name}/y"])


@pytest.mark.parametrize("name", list(DROPOUT_CASES))
def test_gold_dropout(oracle, gold, name):
    """With the mask the reference drew: forward mask*scale*x, backward mask*dy."""
    c = DROPOUT_CASES[name]
    rng = np.random.default_rng(c["seed"])
    x = rng.standard_normal((c["B"], c["dim"])).astype(np.float32)
    dy = rng.standard_normal((c["B"], c["dim"])).astype(np.float32)
    mask = gold[f"dropout/{name}/mask"]
    assert 0 < mask.mean() < 1
    scale = np.float32(1) / (np.float32(1) - np.float32(c["rate"]))
    y, dx = o.f32(*x.shape), o.f32(*x.shape)
    oracle.orc_dropout(o.p(x), o.p(mask), scale, o.p(y), x.size)
    oracle.orc_dropout(o.p(dy), o.p(mask), 1.0, o.p(dx), x.size)
    assert np.array_equal(y, gold[f"dropout/{name}/y"])
    assert np.array_equal(dx, gold[f"dropout/{name}/dx"])


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4, 5, 6])
def test_gold_optimizer_steps(oracle, gold, kind):
    W, g = gold["opt/W0"].copy(), gold["opt/g"]
    s0, s1 = np.zeros_like(W), np.zeros_like(W)
    h = hyper_for(kind)
    for _ in range(5):
        oracle.orc_opt_update(kind, C.byref(h), o.p(g), o.p(W), o.p(s0), o.p(s1), W.size)
        if kind in (1, 4):  # adam and adamax advance their powers after every call
            h.b1_t = np.float32(h.b1_t) * np.float32(h.b1)
            h.b2_t = np.float32(h.b2_t) * np.float32(h.b2)
    assert np.array_equal(W, gold[f"opt/{kind}/W5"])
    # a zero gradient leaves the weight exactly where it was (unconnected filter taps), weight decay aside
    if kind <= 4:
        assert np.array_equal(W[::7], gold["opt/W0"][::7])


@pytest.mark.parametrize("name", list(QCONV_CASES))
def test_gold_qconv(oracle, gold, name):
    c = QCONV_CASES[name]
    d = conv_desc(c)
    x, W, b, _ = gen_conv_inputs(c, d)
    B = x.shape[0]
    xp = o.f32(B, d.in_c * d.inp_h * d.inp_w)
    oracle.orc_conv_pad(C.byref(d), o.p(x), o.p(xp), B)
    y = o.f32(B, d.out_c * d.out_h * d.out_w)
    assert oracle.orc_qconv2d_fwd(C.byref(d), o.p(xp), o.p(W), o.p(b), o.p(y), B, None, None) == 0
    assert y.tobytes() == gold[f"qconv/{name}/y"].tobytes()


@pytest.mark.parametrize("name", list(QFC_CASES))
def test_gold_qfc(oracle, gold, name):
    c = QFC_CASES[name]
    rng = np.random.default_rng(c["seed"])
    B, I, O = c["B"], c["in"], c["out"]
    x = rng.uniform(-1, 1, (B, I)).astype(np.float32)
    W = rng.uniform(-0.5, 0.5, I * O).astype(np.float32)
    b = rng.uniform(-0.1, 0.1, O).astype(np.float32) if c["bias"] else None
    y = o.f32(B, O)
    assert oracle.orc_qfc_fwd(I, O, o.p(x), o.p(W), o.p(b), o.p(y), B) == 0
    assert y.tobytes() == gold[f"qfc/{name}/y"].tobytes()


@pytest.mark.parametrize("name", list(QEQ_CONV_CASES))
def test_gold_qconv_eq(oracle, gold, name):
    """The nine-argument quantized convolution kernel (uint8 values and ranges in and out): bit for bit."""
    d, x, W, bias, in_r, W_r, b_r = gen_qeq_conv_inputs(name)
    B = x.shape[0]
    y, yr = o.f32(B, d.out_c * d.out_h * d.out_w), o.f32(B, 2)
    assert oracle.orc_qconv2d_eq_fwd(C.byref(d), o.p(x), o.p(W), o.p(bias), o.p(in_r), o.p(W_r), o.p(b_r), o.p(y),
                                     o.p(yr), B) == 0
    assert y.tobytes() == gold[f"qconv_eq/{name}/y"].tobytes()
    assert yr.tobytes() == gold[f"qconv_eq/{name}/range"].tobytes()
    assert len(np.unique(y)) > 8  # the case exercises the requantizer, not a constant output


@pytest.mark.parametrize("name", list(QEQ_FC_CASES))
def test_gold_qfc_eq(oracle, gold, name):
    I, O, x, W, bias, in_r, W_r, b_r = gen_qeq_fc_inputs(name)
    B = x.shape[0]
    y, yr = o.f32(B, O), o.f32(B, 2)
    assert oracle.orc_qfc_eq_fwd(I, O, o.p(x), o.p(W), o.p(bias), o.p(in_r), o.p(W_r), o.p(b_r), o.p(y), o.p(yr), B) == 0
    assert y.tobytes() == gold[f"qfc_eq/{name}/y"].tobytes()
    assert yr.tobytes() == gold[f"qfc_eq/{name}/range"].tobytes()


@pytest.mark.parametrize("name", list(NET_CASES))
def test_gold_net_training(oracle, gold, name):
    """orc_net restates network::fit; after the same steps it holds the same weights."""
    c = NET_CASES[name]
    specs, keep = build_net_specs(c["net"])
    arr = (type(specs[0]) * len(specs))(*specs)
    net = oracle.orc_net_create(arr, len(specs), c["B"])
    assert net
    n = oracle.orc_net_param_count(net)
    p0 = xavier_params(specs, c["seed"])
    assert p0.size == n
    params = np.ctypeslib.as_array(oracle.orc_net_params(net), shape=(n,))
    params[:] = p0
    x, t = gen_net_data(c)
    B = c["B"]
    h = hyper_for(c["opt"])
    for s in range(c["steps"]):
        xs, ts = x[s * B:(s + 1) * B], t[s * B:(s + 1) * B]
        oracle.orc_net_train_step(net, o.p(xs), o.p(ts), B, c["loss"], c["opt"], C.byref(h))
    p1 = gold[f"net/{name}/p1"]
    assert np.array_equal(params, p1), float(np.abs(params - p1).max())
    for li in bn_layers(specs):  # the moving averages post_update kept
        cn = specs[li].bn_channels
        assert np.array_equal(np.ctypeslib.as_array(oracle.orc_net_bn_mean(net, li), shape=(cn,)),
                              gold[f"net/{name}/bn{li}/mean"])
        assert np.array_equal(np.ctypeslib.as_array(oracle.orc_net_bn_var(net, li), shape=(cn,)),
                              gold[f"net/{name}/bn{li}/var"])
    oracle.orc_net_set_phase(net, 0)  # network::predict runs in the test phase
    oracle.orc_net_forward(net, o.p(x[:B]), B)
    out = np.ctypeslib.as_array(oracle.orc_net_output(net), shape=(B, c["out_dim"]))
    assert np.array_equal(out, gold[f"net/{name}/predict"])
    if c["opt"] == 1:
        a, b = C.c_float(), C.c_float()
        oracle.orc_net_adam_powers(net, C.byref(a), C.byref(b))
        assert [a.value, b.value] == gold[f"net/{name}/adam_powers"].tolist()
    oracle.orc_net_destroy(net)


@pytest.mark.parametrize("name", ["lenet_165_b16_e2", "cifar_28_b8_e2", "lenet_33_b16_e1", "tiny_23_b5_e3"])
def test_gold_fit_with_ragged_last_batch(oracle, gold, name):
    """network::fit over a sample count that is not a multiple of the mini-batch: the restated
    loop (batch buffers that keep the previous step's rows, one-sample branch) ends with the
    reference's weights bit for bit."""
    from cases import gen_ragged_fit_data
    c, x, t, n_samples, B, epochs = gen_ragged_fit_data(name)
    specs, keep = build_net_specs(c["net"])
    arr = (type(specs[0]) * len(specs))(*specs)
    net = oracle.orc_net_create(arr, len(specs), B)
    p0 = xavier_params(specs, c["seed"])
    params = np.ctypeslib.as_array(oracle.orc_net_params(net), shape=(p0.size,))
    params[:] = p0
    h = hyper_for(c["opt"])
    assert oracle.orc_net_fit(net, o.p(x), o.p(t), n_samples, B, epochs, c["loss"], c["opt"], C.byref(h)) == 0
    assert np.array_equal(params, gold[f"fit_ragged/{name}/p1"])
    oracle.orc_net_destroy(net)
