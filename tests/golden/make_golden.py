"""Generate tests/golden/ref_outputs.npz by running the UNMODIFIED reference
(oracle/_ref/libtinydnn_ref.so, built by oracle/build_oracle.py where the
reference tree is present) on seeded inputs.

The fixture holds inputs and the reference's outputs for every operator on the
hot path plus short training runs, so that the oracle restatement and the CUDA
path can be checked on a machine that does not have the reference.

    python tests/golden/make_golden.py
"""
from __future__ import annotations

import ctypes as C
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import oracle_lib as o  # noqa: E402
from cases import (BATCHNORM_CASES, DROPOUT_CASES, LRN_CASES, QEQ_CONV_CASES, QEQ_FC_CASES,  # noqa: E402
                   bn_layers, gen_batchnorm_inputs, gen_qeq_conv_inputs, gen_qeq_fc_inputs,
                   ACT_CASES, AVGPOOL_CASES, CONV_CASES, DATA_CASES, FC_CASES, MAXPOOL_CASES, NET_CASES,  # noqa: E402
                   QCONV_CASES, QFC_CASES, build_net_specs, conv_desc, dataset_file_bytes, gen_conv_inputs,
                   gen_dataset_bytes, gen_net_data, hyper_for, merge_rows_np, pool_desc, xavier_params, OPT_KINDS,
                   RAGGED_FIT_CASES, gen_ragged_fit_data)

ROWS_LIMIT = 4096  # per-sample gradient rows are stored only when this small


def put_grads(out, key, dW, db):
    """Store the merged gradients, and the per-sample rows when they are small."""
    out[f"{key}/dW_sum"] = merge_rows_np(dW)
    out[f"{key}/db_sum"] = merge_rows_np(db)
    if dW.size <= ROWS_LIMIT:
        out[f"{key}/dW_rows"] = dW
        out[f"{key}/db_rows"] = db


def main():
    ref = o.load_reference()
    if ref is None:
        raise SystemExit("oracle/_ref/libtinydnn_ref.so is missing: run oracle/build_oracle.py first")
    out = {}

    for name, c in CONV_CASES.items():
        d = conv_desc(c)
        x, W, b, dy = gen_conv_inputs(c, d)
        B = x.shape[0]
        y = o.f32(B, d.out_c * d.out_h * d.out_w)
        assert ref.ref_conv2d_fwd(C.byref(d), o.p(x), o.p(W), o.p(b), o.p(y), B) == 0
        dx = o.f32(*x.shape)
        dW = o.f32(B, W.size)
        db = o.f32(B, d.out_c)
        assert ref.ref_conv2d_bwd(C.byref(d), o.p(x), o.p(W), o.p(dy), o.p(dx), o.p(dW), o.p(db), B) == 0
        out[f"conv/{name}/y"] = y
        out[f"conv/{name}/dx"] = dx
        put_grads(out, f"conv/{name}", dW, db)

    for name, c in FC_CASES.items():
        rng = np.random.default_rng(c["seed"])
        B, I, O = c["B"], c["in"], c["out"]
        x = rng.uniform(0, 1, (B, I)).astype(np.float32)
        W = rng.uniform(-0.3, 0.3, I * O).astype(np.float32)
        b = rng.uniform(-0.1, 0.1, O).astype(np.float32) if c["bias"] else None
        dy = rng.standard_normal((B, O)).astype(np.float32)
        y = o.f32(B, O)
        assert ref.ref_fc_fwd(I, O, o.p(x), o.p(W), o.p(b), o.p(y), B) == 0
        dx, dW, db = o.f32(B, I), o.f32(B, I * O), o.f32(B, O)
        assert ref.ref_fc_bwd(I, O, int(c["bias"]), o.p(x), o.p(W), o.p(dy), o.p(dx), o.p(dW), o.p(db), B) == 0
        out[f"fc/{name}/y"], out[f"fc/{name}/dx"] = y, dx
        put_grads(out, f"fc/{name}", dW, db)

    for name, c in MAXPOOL_CASES.items():
        d = pool_desc(c)
        rng = np.random.default_rng(c["seed"])
        B = c["B"]
        x = rng.standard_normal((B, d.in_c * d.in_h * d.in_w)).astype(np.float32)
        n_out = d.in_c * d.out_h * d.out_w
        dy = rng.standard_normal((B, n_out)).astype(np.float32)
        y, dx = o.f32(B, n_out), o.f32(*x.shape)
        assert ref.ref_maxpool_fwd_bwd(C.byref(d), int(c.get("ceil", 0)), int(c.get("same", 0)), o.p(x),
                                       o.p(y), o.p(dy), o.p(dx), B) == 0
        out[f"maxpool/{name}/y"], out[f"maxpool/{name}/dx"] = y, dx

    for name, c in AVGPOOL_CASES.items():
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
        assert ref.ref_avgpool_fwd_bwd(C.byref(d), o.p(x), o.p(W), o.p(b), o.p(y), o.p(dy), o.p(dx),
                                       o.p(dW), o.p(db), B) == 0
        out[f"avgpool/{name}/y"], out[f"avgpool/{name}/dx"] = y, dx
        put_grads(out, f"avgpool/{name}", dW, db)

    # quantized layers chained without dequantizing: the reference's nine- / eleven-argument kernels
    for name in QEQ_CONV_CASES:
        d, x, W, bias, in_r, W_r, b_r = gen_qeq_conv_inputs(name)
        B = x.shape[0]
        y, yr = o.f32(B, d.out_c * d.out_h * d.out_w), o.f32(B, 2)
        assert ref.ref_qconv2d_eq_fwd(C.byref(d), o.p(x), o.p(W), o.p(bias), o.p(in_r), o.p(W_r), o.p(b_r), o.p(y),
                                      o.p(yr), B) == 0
        out[f"qconv_eq/{name}/y"], out[f"qconv_eq/{name}/range"] = y, yr
    for name in QEQ_FC_CASES:
        I, O, x, W, bias, in_r, W_r, b_r = gen_qeq_fc_inputs(name)
        B = x.shape[0]
        y, yr = o.f32(B, O), o.f32(B, 2)
        assert ref.ref_qfc_eq_fwd(I, O, o.p(x), o.p(W), o.p(bias), o.p(in_r), o.p(W_r), o.p(b_r), o.p(y), o.p(yr),
                                  B) == 0
        out[f"qfc_eq/{name}/y"], out[f"qfc_eq/{name}/range"] = y, yr

    for name, c in BATCHNORM_CASES.items():
        x, dy, run_mean, run_var = gen_batchnorm_inputs(c)
        Cn, S, B = c["C"], c["S"], c["B"]
        y, dx = o.f32(*x.shape), o.f32(*x.shape)
        mean, var, sd = o.f32(Cn), o.f32(Cn), o.f32(Cn)
        assert ref.ref_batchnorm_fwd_bwd(Cn, S, c["eps"], o.p(x), o.p(mean), o.p(var), o.p(sd), o.p(y), o.p(dy), o.p(dx),
                                         B, 1) == 0
        for k, v in (("y", y), ("dx", dx), ("mean", mean), ("var", var), ("stddev", sd)):
            out[f"batchnorm/{name}/train/{k}"] = v
        y2, dx2, sd2 = o.f32(*x.shape), o.f32(*x.shape), o.f32(Cn)
        m2, v2 = run_mean.copy(), run_var.copy()
        assert ref.ref_batchnorm_fwd_bwd(Cn, S, c["eps"], o.p(x), o.p(m2), o.p(v2), o.p(sd2), o.p(y2), o.p(dy), o.p(dx2),
                                         B, 0) == 0
        for k, v in (("y", y2), ("dx", dx2), ("stddev", sd2)):
            out[f"batchnorm/{name}/test/{k}"] = v

    for name, c in LRN_CASES.items():
        rng = np.random.default_rng(c["seed"])
        x = rng.standard_normal((c["B"], c["C"] * c["w"] * c["h"])).astype(np.float32)
        y = o.f32(*x.shape)
        assert ref.ref_lrn_fwd(o.p(x), o.p(y), c["C"], c["w"], c["h"], c["size"], c["alpha"], c["beta"], c["B"]) == 0
        out[f"lrn/{name}/y"] = y

    for name, c in DROPOUT_CASES.items():
        rng = np.random.default_rng(c["seed"])
        x = rng.standard_normal((c["B"], c["dim"])).astype(np.float32)
        dy = rng.standard_normal((c["B"], c["dim"])).astype(np.float32)
        y, dx = o.f32(*x.shape), o.f32(*x.shape)
        mask = np.zeros(x.shape, np.uint8)
        assert ref.ref_dropout_fwd_bwd(c["dim"], c["rate"], o.p(x), o.p(y), o.p(mask), o.p(dy), o.p(dx), c["B"]) == 0
        out[f"dropout/{name}/mask"], out[f"dropout/{name}/y"], out[f"dropout/{name}/dx"] = mask, y, dx

    for name, c in ACT_CASES.items():
        rng = np.random.default_rng(c["seed"])
        B, dim = c["B"], c["dim"]
        x = (rng.standard_normal((B, dim)) * c.get("scale", 1.0)).astype(np.float32)
        dy = rng.standard_normal((B, dim)).astype(np.float32)
        y, dx = o.f32(B, dim), o.f32(B, dim)
        if "param" in c:
            assert ref.ref_act_param_fwd_bwd(c["kind"], c["param"], o.p(x), o.p(y), o.p(dy), o.p(dx), dim, B) == 0
        else:  # the layer's default constructor argument
            assert ref.ref_act_fwd_bwd(c["kind"], o.p(x), o.p(y), o.p(dy), o.p(dx), dim, B) == 0
        out[f"act/{name}/y"], out[f"act/{name}/dx"] = y, dx
        for loss in (0, 1, 2):
            yy = rng.uniform(0.05, 0.95, (B, dim)).astype(np.float32)
            tt = (rng.random((B, dim)) > 0.8).astype(np.float32)
            g = o.f32(B, dim)
            assert ref.ref_loss_grad(loss, o.p(yy), o.p(tt), o.p(g), dim, B) == 0
            out[f"loss/{name}/{loss}/y"], out[f"loss/{name}/{loss}/t"], out[f"loss/{name}/{loss}/g"] = yy, tt, g

    # optimizers: 5 consecutive updates with a fixed gradient
    rng = np.random.default_rng(77)
    W0 = rng.standard_normal(1000).astype(np.float32)
    g0 = rng.standard_normal(1000).astype(np.float32)
    g0[::7] = 0.0  # exact zeros must give exactly zero update
    out["opt/W0"], out["opt/g"] = W0, g0
    for kind in OPT_KINDS:
        W = W0.copy()
        h = hyper_for(kind)
        assert ref.ref_opt_steps(kind, C.byref(h), o.p(g0), o.p(W), W.size, 5) == 0
        out[f"opt/{kind}/W5"] = W

    for name, c in QCONV_CASES.items():
        d = conv_desc(c)
        x, W, b, _ = gen_conv_inputs(c, d)
        B = x.shape[0]
        y = o.f32(B, d.out_c * d.out_h * d.out_w)
        assert ref.ref_qconv2d_fwd(C.byref(d), o.p(x), o.p(W), o.p(b), o.p(y), B) == 0
        out[f"qconv/{name}/y"] = y

    for name, c in QFC_CASES.items():
        rng = np.random.default_rng(c["seed"])
        B, I, O = c["B"], c["in"], c["out"]
        x = rng.uniform(-1, 1, (B, I)).astype(np.float32)
        W = rng.uniform(-0.5, 0.5, I * O).astype(np.float32)
        b = rng.uniform(-0.1, 0.1, O).astype(np.float32) if c["bias"] else None
        y = o.f32(B, O)
        assert ref.ref_qfc_fwd(I, O, o.p(x), o.p(W), o.p(b), o.p(y), B) == 0
        out[f"qfc/{name}/y"] = y

    for name, c in NET_CASES.items():
        specs, keep = build_net_specs(c["net"])
        arr = (type(specs[0]) * len(specs))(*specs)
        h = ref.ref_net_create(arr, len(specs), c["seed"])
        assert h
        n = ref.ref_net_param_count(h)
        p0 = xavier_params(specs, c["seed"])
        assert p0.size == n
        ref.ref_net_set_params(h, o.p(p0))
        x, t = gen_net_data(c)
        B, steps = c["B"], c["steps"]
        hy = hyper_for(c["opt"])
        secs = ref.ref_net_fit(h, o.p(x), o.p(t), B, steps, c["loss"], c["opt"], C.byref(hy))
        assert secs >= 0
        p1 = o.f32(n)
        ref.ref_net_get_params(h, o.p(p1))
        yp = o.f32(B, c["out_dim"])
        assert ref.ref_net_predict(h, o.p(x[:B]), o.p(yp), B) == 0
        out[f"net/{name}/p1"], out[f"net/{name}/predict"] = p1, yp
        for li in bn_layers(specs):  # moving averages after the fit (predict above ran in the test phase)
            m, v = o.f32(specs[li].bn_channels), o.f32(specs[li].bn_channels)
            assert ref.ref_net_bn_stats(h, li, o.p(m), o.p(v)) == 0
            out[f"net/{name}/bn{li}/mean"], out[f"net/{name}/bn{li}/var"] = m, v
        if c["opt"] == 1:
            a, b2 = C.c_float(), C.c_float()
            ref.ref_net_adam_powers(h, C.byref(a), C.byref(b2))
            out[f"net/{name}/adam_powers"] = np.array([a.value, b2.value], dtype=np.float32)
        ref.ref_net_destroy(h)

    # network::fit with a ragged last mini-batch
    for name in RAGGED_FIT_CASES:
        c, x, t, n_samples, B, epochs = gen_ragged_fit_data(name)
        specs, keep = build_net_specs(c["net"])
        arr = (type(specs[0]) * len(specs))(*specs)
        h = ref.ref_net_create(arr, len(specs), c["seed"])
        p0 = xavier_params(specs, c["seed"])
        ref.ref_net_set_params(h, o.p(p0))
        hy = hyper_for(c["opt"])
        assert ref.ref_net_fit_n(h, o.p(x), o.p(t), n_samples, B, epochs, c["loss"], c["opt"], C.byref(hy)) >= 0
        p1 = o.f32(p0.size)
        ref.ref_net_get_params(h, o.p(p1))
        out[f"fit_ragged/{name}/p1"] = p1
        ref.ref_net_destroy(h)

    # dataset parsers on synthetic files in the datasets' own formats
    import tempfile
    for name, c in DATA_CASES.items():
        img, labels = gen_dataset_bytes(c)
        out_len = c["c"] * (c["h"] + 2 * c["yp"]) * (c["w"] + 2 * c["xp"])
        rows = o.f32(c["n"], out_len)
        with tempfile.NamedTemporaryFile(suffix=".bin") as f:
            f.write(dataset_file_bytes(c, img, labels))
            f.flush()
            if c["mode"] == 0:
                lab = np.zeros(c["n"], np.uint8)
                n = ref.ref_parse_cifar10(f.name.encode(), c["smin"], c["smax"], c["xp"], c["yp"], o.p(rows),
                                          o.p(lab), c["n"])
                assert np.array_equal(lab, labels)
            else:
                n = ref.ref_parse_mnist_images(f.name.encode(), c["smin"], c["smax"], c["xp"], c["yp"], o.p(rows),
                                               c["n"])
        assert n == c["n"], (name, n)
        out[f"data/{name}/rows"] = rows
    # network::train's targets for class labels: the output range of the net's last layer
    for net_name in ("lenet", "cifar"):
        specs, keep = build_net_specs(net_name)
        arr = (type(specs[0]) * len(specs))(*specs)
        h = ref.ref_net_create(arr, len(specs), 1)
        labels = np.arange(10, dtype=np.uint8)
        tg, rg = o.f32(10, 10), o.f32(2)
        assert ref.ref_net_label_targets(h, o.p(labels), 10, o.p(tg), o.p(rg)) == 0
        out[f"data/targets/{net_name}"] = tg
        out[f"data/target_range/{net_name}"] = rg
        ref.ref_net_destroy(h)

    path = HERE / "ref_outputs.npz"
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size / 1024:.1f} KiB, {len(out)} arrays)")


if __name__ == "__main__":
    main()
