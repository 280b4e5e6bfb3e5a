"""Generate tests/golden/ref_fullsize.npz: the UNMODIFIED reference
(oracle/_ref/libtinydnn_ref.so) run on every benchmark configuration at its
stated size, reduced to digests (strided samples, float64 sums, per-row sums;
byte hashes for the quantized outputs) so the fixture stays small.

    python tests/golden/make_golden_fullsize.py        # about ten minutes of CPU

Configurations: the CIFAR-10 net at batch 256 for 3 adam steps; the 3x3
single-layer sweep (56x56x64, 28x28x128, 14x14x256) at batch 256; the MLP
784-4096-4096-10 at batch 1024 with momentum (gradients computed 16 samples at
a time, because the reference's per-sample weight gradients of one such batch
would need 82 GB); the quantized convolution at batch 128 (stride 1 alone,
stride 2 followed by the quantized fully-connected layer 9216 -> 256).
"""
from __future__ import annotations

import ctypes as C
import hashlib
import sys
import time
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

import oracle_lib as o  # noqa: E402
from cases import (FULL_CONV_CASES, FULL_NET_CASES, FULL_Q_CASE, build_net_specs, conv_desc,  # noqa: E402
                   conv_params, digest, gen_full_conv_inputs, gen_full_q_inputs, gen_net_data, hyper_for,
                   merge_rows_np, net_layout, xavier_params)


def put(out, key, a, stride=101):
    for k, v in digest(a, stride).items():
        out[f"{key}/{k}"] = v


def sha(a):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(a).tobytes()).digest(), dtype=np.uint8).copy()


def main():
    ref = o.load_reference()
    if ref is None:
        raise SystemExit("oracle/_ref/libtinydnn_ref.so is missing: run oracle/build_oracle.py first")
    out = {}
    only = set(sys.argv[1:])

    def want(name):
        return not only or name in only

    # ---- single-layer sweep ---------------------------------------------------------------
    for name, c in FULL_CONV_CASES.items():
        if not want("conv"):
            break
        t0 = time.time()
        d = conv_desc(c)
        x, W, b, dy = gen_full_conv_inputs(c, d)
        B = x.shape[0]
        y = o.f32(B, d.out_c * d.out_h * d.out_w)
        assert ref.ref_conv2d_fwd(C.byref(d), o.p(x), o.p(W), o.p(b), o.p(y), B) == 0
        dx, dW, db = o.f32(*x.shape), o.f32(B, W.size), o.f32(B, d.out_c)
        assert ref.ref_conv2d_bwd(C.byref(d), o.p(x), o.p(W), o.p(dy), o.p(dx), o.p(dW), o.p(db), B) == 0
        put(out, f"conv/{name}/y", y, 10007)
        put(out, f"conv/{name}/dx", dx, 10007)
        put(out, f"conv/{name}/dW_sum", merge_rows_np(dW), 7)
        out[f"conv/{name}/db_sum"] = merge_rows_np(db)
        print(f"conv {name}: {time.time() - t0:.1f} s", flush=True)

    # ---- whole networks ---------------------------------------------------------------------
    for name, c in FULL_NET_CASES.items():
        if not want(name):
            continue
        t0 = time.time()
        specs, keep = build_net_specs(c["net"])
        arr = (type(specs[0]) * len(specs))(*specs)
        layout, n = net_layout(specs)
        h = ref.ref_net_create(arr, len(specs), c["seed"])
        assert h and ref.ref_net_param_count(h) == n
        p0 = xavier_params(specs, c["seed"])
        ref.ref_net_set_params(h, o.p(p0))
        x, t = gen_net_data(c)
        B, steps = c["B"], c["steps"]
        hy = hyper_for(c["opt"])
        for s in range(steps):
            xs, ts = x[s * B:(s + 1) * B], t[s * B:(s + 1) * B]
            g, y = o.f32(n), o.f32(B, c["out_dim"])
            assert ref.ref_net_grads_chunked(h, o.p(xs), o.p(ts), B, c["chunk"], c["loss"], o.p(g), o.p(y)) == 0
            assert ref.ref_net_apply_update(h, o.p(g), c["opt"], C.byref(hy)) == 0
            p = o.f32(n)
            ref.ref_net_get_params(h, o.p(p))
            out[f"net/{name}/step{s}/out"] = y
            for ti, (off, ln, _, _, _) in enumerate(layout):
                stride = 3 if ln <= 200000 else 1009
                put(out, f"net/{name}/step{s}/grad{ti}", g[off:off + ln], stride)
                put(out, f"net/{name}/step{s}/param{ti}", p[off:off + ln], stride)
            print(f"net {name} step {s}: {time.time() - t0:.1f} s", flush=True)
        if c["opt"] == 1:
            a, b2 = C.c_float(), C.c_float()
            ref.ref_net_adam_powers(h, C.byref(a), C.byref(b2))
            out[f"net/{name}/adam_powers"] = np.array([a.value, b2.value], dtype=np.float32)
        p_manual = o.f32(n)
        ref.ref_net_get_params(h, o.p(p_manual))
        ref.ref_net_destroy(h)
        if c["chunk"] == B:
            # the same steps through network::fit itself: identical weights, bit for bit
            h2 = ref.ref_net_create(arr, len(specs), c["seed"])
            ref.ref_net_set_params(h2, o.p(p0))
            assert ref.ref_net_fit(h2, o.p(x), o.p(t), B, steps, c["loss"], c["opt"], C.byref(hy)) >= 0
            p_fit = o.f32(n)
            ref.ref_net_get_params(h2, o.p(p_fit))
            ref.ref_net_destroy(h2)
            assert np.array_equal(p_fit, p_manual), "fprop/bprop/merge/update by hand differs from network::fit"
            print(f"net {name}: network::fit gives the same weights bit for bit", flush=True)

    # ---- how far two fp32 evaluation orders drift apart: the reference against itself ---------
    # The CIFAR-10 net at batch 256 trained by the reference twice from the same weights on the same
    # data: engine backend_t::internal, and the reference's own AVX kernels (backend_t::avx, built
    # from the same sources with -DCNN_USE_AVX).  Recorded after one fit of three adam steps and
    # after a second one: per parameter tensor the share of entries that agree to 1e-3 of the
    # largest magnitude and the worst difference.  This is the yardstick for what "the same result"
    # can mean for whole-net weights at this size (see tests/test_oracle_fullsize.py).
    if want("divergence"):
        avx = o.load_reference_avx()
        if avx is None:
            raise SystemExit("oracle/_ref/libtinydnn_ref_avx.so is missing")
        c = FULL_NET_CASES["cifar_adam_b256"]
        specs, keep = build_net_specs(c["net"])
        arr = (type(specs[0]) * len(specs))(*specs)
        layout, n = net_layout(specs)
        x, t = gen_net_data(c)
        hy = hyper_for(c["opt"])
        p0 = xavier_params(specs, c["seed"])
        runs = {}
        for label, lib in (("internal", ref), ("avx", avx)):
            h = lib.ref_net_create(arr, len(specs), 1)
            lib.ref_net_set_params(h, o.p(p0))
            runs[label] = []
            for fit in range(2):
                assert lib.ref_net_fit(h, o.p(x), o.p(t), c["B"], c["steps"], c["loss"], c["opt"], C.byref(hy)) >= 0
                p = o.f32(n)
                lib.ref_net_get_params(h, o.p(p))
                runs[label].append(p)
            lib.ref_net_destroy(h)
        table = np.zeros((2, len(layout), 2))
        for fit in range(2):
            for ti, (off, ln, _, _, _) in enumerate(layout):
                a, b = runs["internal"][fit][off:off + ln], runs["avx"][fit][off:off + ln]
                d, mx = np.abs(a.astype(np.float64) - b), float(np.abs(a).max())
                table[fit, ti] = [(d <= 1e-3 * mx).mean(), d.max() / mx]
        out["divergence/internal_vs_avx"] = table
        print("reference internal vs AVX engine, [fit][tensor](share within 1e-3, worst / max):")
        print(np.array2string(table, precision=4, suppress_small=True), flush=True)

    # ---- quantized inference ----------------------------------------------------------------
    if want("quant"):
        t0 = time.time()
        c = FULL_Q_CASE
        x, W, biases, Wf, bf = gen_full_q_inputs()
        B = c["B"]
        for bname, bias in biases.items():
            for stride in (1, 2):
                d = conv_params(c["w"], c["h"], c["c"], c["kw"], c["kh"], c["oc"], False, True, stride, stride)
                y = o.f32(B, d.out_c * d.out_h * d.out_w)
                assert ref.ref_qconv2d_fwd(C.byref(d), o.p(x), o.p(W), o.p(bias), o.p(y), B) == 0
                out[f"quant/{bname}/conv_s{stride}/sha256"] = sha(y)
                out[f"quant/{bname}/conv_s{stride}/samples"] = y.ravel()[::997].copy()
            assert y.shape[1] == 9216
            z = o.f32(B, c["fc_out"])
            assert ref.ref_qfc_fwd(9216, c["fc_out"], o.p(y), o.p(Wf), o.p(bf), o.p(z), B) == 0
            out[f"quant/{bname}/fc/sha256"] = sha(z)
            out[f"quant/{bname}/fc/samples"] = z.ravel()[::97].copy()
        print(f"quantized: {time.time() - t0:.1f} s", flush=True)

    path = HERE / "ref_fullsize.npz"
    if only and path.exists():
        old = dict(np.load(path))
        old.update(out)
        out = old
    np.savez_compressed(path, **out)
    print(f"wrote {path} ({path.stat().st_size / 1024:.1f} KiB, {len(out)} arrays)")


if __name__ == "__main__":
    main()
