"""GPU parity tests of the device-resident training step (b200_net_*): the
networks of the benchmark configurations are stepped through the C ABI and
compared with the oracle's restatement of network::fit, which test_oracle.py
ties bit for bit to the unmodified reference.

Tolerances: forward outputs 1e-4, gradients and updated weights 1e-3 (relative to
the largest reference magnitude)."""
import ctypes as C
import os
from pathlib import Path

import numpy as np
import pytest
import torch

import oracle_lib as o
from cases import NET_CASES, bn_layers, build_net_specs, null_gradient_biases, gen_net_data, hyper_for, net_layout, xavier_params
from test_ops_gpu import FWD_TOL, GRAD_TOL, assert_close, dev, host
from tiny_cnn_b200 import network as nw
from tiny_cnn_b200._lib import LayerSpec, check, ptr

pytestmark = pytest.mark.gpu
GOLD = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD / "ref_outputs.npz")


class DeviceNet:
    """Thin test harness over the C ABI net built from raw layer specs."""

    def __init__(self, ctx, specs, max_batch):
        self.ctx, self.lib = ctx, ctx.lib
        arr = (LayerSpec * len(specs))(*specs)
        h = C.c_void_p()
        check(self.lib.b200_net_create(ctx.handle, arr, len(specs), max_batch, C.byref(h)))
        self.h = h
        self.n = int(self.lib.b200_net_param_count(h))
        self.out_dim = int(self.lib.b200_net_out_dim(h))

    def set_params(self, p):
        check(self.lib.b200_net_set_params(self.h, ptr(np.ascontiguousarray(p, dtype=np.float32))))

    def params(self):
        p = np.empty(self.n, np.float32)
        check(self.lib.b200_net_get_params(self.h, ptr(p)))
        return p

    def grads(self):
        g = np.empty(self.n, np.float32)
        check(self.lib.b200_net_get_grads(self.h, ptr(g)))
        return g

    def output(self, B):
        out = np.empty((B, self.out_dim), np.float32)
        check(self.lib.b200_memcpy_d2h(self.ctx.handle, ptr(out), self.lib.b200_net_output_ptr(self.h),
                                       out.nbytes))
        return out

    def close(self):
        self.lib.b200_net_destroy(self.h)


def orc_net_for(oracle, specs, B, p0):
    arr = (LayerSpec * len(specs))(*specs)
    net = oracle.orc_net_create(arr, len(specs), B)
    n = oracle.orc_net_param_count(net)
    params = np.ctypeslib.as_array(oracle.orc_net_params(net), shape=(n,))
    params[:] = p0
    return net, params


@pytest.mark.parametrize("fuse", ["0", "1"])
@pytest.mark.parametrize("name", list(NET_CASES))
def test_net_steps_match_oracle(ctx, oracle, gold, name, fuse, monkeypatch):
    """Each step: outputs, batch-summed gradients and updated weights against the oracle;
    after the last step the weights against the reference's recorded run."""
    monkeypatch.setenv("B200_NET_NO_FUSE", "1" if fuse == "0" else "0")
    monkeypatch.setenv("B200_NET_NO_GRAPH", "1")
    c = NET_CASES[name]
    specs, keep = build_net_specs(c["net"])
    B = c["B"]
    p0 = xavier_params(specs, c["seed"])
    dnet = DeviceNet(ctx, specs, B)
    assert dnet.n == p0.size
    dnet.set_params(p0)
    onet, oparams = orc_net_for(oracle, specs, B, p0)
    x, t = gen_net_data(c)
    h = hyper_for(c["opt"])
    n = dnet.n
    null = null_gradient_biases(specs)
    for s in range(c["steps"]):
        xs, ts = x[s * B:(s + 1) * B], t[s * B:(s + 1) * B]
        dx, dt = dev(xs), dev(ts)
        check(dnet.lib.b200_net_forward(dnet.h, ptr(dx), B))
        oracle.orc_net_forward(onet, o.p(xs), B)
        out_ref = np.ctypeslib.as_array(oracle.orc_net_output(onet), shape=(B, c["out_dim"])).copy()
        assert_close(dnet.output(B), out_ref, FWD_TOL, f"{name} step {s} output")
        check(dnet.lib.b200_net_backward(dnet.h, ptr(dt), c["loss"]))
        oracle.orc_net_backward(onet, o.p(xs), o.p(ts), c["loss"], B)
        g_ref = np.ctypeslib.as_array(oracle.orc_net_grads(onet), shape=(n,)).copy()
        g = dnet.grads()
        gmax = float(np.abs(g_ref).max())
        for off, ln, _, _, _ in net_layout(specs)[0]:
            if off in null:  # exactly zero in exact arithmetic: both sides hold rounding noise
                assert np.abs(g[off:off + ln]).max() <= 1e-5 * gmax and np.abs(g_ref[off:off + ln]).max() <= 1e-5 * gmax
                continue
            assert_close(g[off:off + ln], g_ref[off:off + ln], GRAD_TOL, f"{name} step {s} grad@{off}")
        check(dnet.lib.b200_net_update(dnet.h, c["opt"], C.byref(h)))
        oracle.orc_net_update(onet, c["opt"], C.byref(h))
        p = dnet.params()
        for off, ln, _, _, _ in net_layout(specs)[0]:
            if off in null:  # driven by noise only: stays tiny on both sides
                assert np.abs(p[off:off + ln]).max() <= 1e-4 and np.abs(oparams[off:off + ln]).max() <= 1e-4
                continue
            assert_close(p[off:off + ln], oparams[off:off + ln], GRAD_TOL, f"{name} step {s} weights@{off}")
    p1 = gold[f"net/{name}/p1"]
    p = dnet.params()
    for off, ln, _, _, _ in net_layout(specs)[0]:
        if off in null:
            assert np.abs(p[off:off + ln]).max() <= 1e-4 and np.abs(p1[off:off + ln]).max() <= 1e-4
            continue
        assert_close(p[off:off + ln], p1[off:off + ln], GRAD_TOL, f"{name} final weights@{off} vs reference")
    if c["opt"] == 1:
        a, b = C.c_float(), C.c_float()
        check(dnet.lib.b200_net_adam_powers(dnet.h, C.byref(a), C.byref(b)))
        # Adam's powers advance once per parameter tensor: identical float products
        assert [a.value, b.value] == gold[f"net/{name}/adam_powers"].tolist()
    # batch normalization: the moving averages against the reference's, then predict in the test phase
    for li in bn_layers(specs):
        cn = specs[li].bn_channels
        m, v = np.empty(cn, np.float32), np.empty(cn, np.float32)
        check(dnet.lib.b200_net_bn_stats(dnet.h, li, ptr(m), ptr(v), 0))
        assert_close(m, gold[f"net/{name}/bn{li}/mean"], GRAD_TOL, f"{name} moving mean of layer {li}")
        assert_close(v, gold[f"net/{name}/bn{li}/var"], GRAD_TOL, f"{name} moving variance of layer {li}")
    check(dnet.lib.b200_net_set_phase(dnet.h, 0))
    dx0 = dev(x[:B])
    check(dnet.lib.b200_net_forward(dnet.h, ptr(dx0), B))
    # after training the weights agree to GRAD_TOL, and so do the outputs they give
    assert_close(dnet.output(B), gold[f"net/{name}/predict"], GRAD_TOL, f"{name} predict after the fit")
    dnet.close()
    oracle.orc_net_destroy(onet)


@pytest.mark.parametrize("name", ["lenet_adagrad", "cifar_adam"])
def test_train_step_graph_and_host_path(ctx, oracle, gold, name, monkeypatch):
    """b200_net_train_step (captured graph after the first two calls) and the HOST
    entry point reach the reference's weights too, and return the forward output."""
    monkeypatch.setenv("B200_NET_NO_FUSE", "0")
    monkeypatch.setenv("B200_NET_NO_GRAPH", "0")
    c = NET_CASES[name]
    specs, keep = build_net_specs(c["net"])
    B = c["B"]
    p0 = xavier_params(specs, c["seed"])
    x, t = gen_net_data(c)
    h = hyper_for(c["opt"])
    p1 = gold[f"net/{name}/p1"]
    for mode in ("device", "host"):
        dnet = DeviceNet(ctx, specs, B)
        dnet.set_params(p0)
        # fixed device staging so every step reuses one captured graph
        dx = torch.empty(B, c["in_dim"], device="cuda")
        dt = torch.empty(B, c["out_dim"], device="cuda")
        first_out = None
        for s in range(c["steps"]):
            xs, ts = x[s * B:(s + 1) * B], t[s * B:(s + 1) * B]
            if mode == "device":
                dx.copy_(torch.from_numpy(xs))
                dt.copy_(torch.from_numpy(ts))
                torch.cuda.synchronize()
                check(dnet.lib.b200_net_train_step(dnet.h, ptr(dx), ptr(dt), B, c["loss"], c["opt"],
                                                   C.byref(h)))
            else:
                out = np.empty((B, c["out_dim"]), np.float32)
                check(dnet.lib.b200_net_train_step_host(dnet.h, ptr(np.ascontiguousarray(xs)),
                                                        ptr(np.ascontiguousarray(ts)), B, c["loss"],
                                                        c["opt"], C.byref(h), ptr(out)))
                if s == 0:
                    first_out = out
        ctx.sync()
        p = dnet.params()
        for off, ln, _, _, _ in net_layout(specs)[0]:
            assert_close(p[off:off + ln], p1[off:off + ln], GRAD_TOL, f"{name} {mode} weights@{off}")
        if mode == "host":
            onet, _ = orc_net_for(oracle, specs, B, p0)
            oracle.orc_net_forward(onet, o.p(x[:B]), B)
            out_ref = np.ctypeslib.as_array(oracle.orc_net_output(onet), shape=(B, c["out_dim"]))
            assert_close(first_out, out_ref, FWD_TOL, f"{name} host step output")
            oracle.orc_net_destroy(onet)
        dnet.close()


@pytest.mark.parametrize("graph", ["0", "1"])
def test_without_the_input_gradient_the_weights_are_the_same_bits(ctx, graph, monkeypatch):
    """b200_net_set_input_grad(net, 0) drops the first layer's dX (which network::fit never reads):
    four adam steps of the CIFAR net end in bit-identical weights, and turning it back on works."""
    monkeypatch.setenv("B200_NET_NO_GRAPH", "0" if graph == "1" else "1")
    specs, keep = build_net_specs("cifar")
    B = 16
    p0 = xavier_params(specs, 11)
    rng = np.random.default_rng(12)
    x = torch.from_numpy(rng.standard_normal((B, 3072)).astype(np.float32)).cuda()
    t = torch.zeros(B, 10, device="cuda")
    t[torch.arange(B), torch.from_numpy(rng.integers(0, 10, B)).cuda()] = 1.0
    h = hyper_for(1)
    results = []
    for on in (1, 0):
        dnet = DeviceNet(ctx, specs, B)
        dnet.set_params(p0)
        check(ctx.lib.b200_net_set_input_grad(dnet.h, on))
        for s in range(4):
            if s == 3:  # back on for the last step: the graphs are rebuilt
                check(ctx.lib.b200_net_set_input_grad(dnet.h, 1))
            check(ctx.lib.b200_net_train_step(dnet.h, ptr(x), ptr(t), B, 1, 1, C.byref(h)))
        ctx.sync()
        results.append(dnet.params())
        dnet.close()
    assert not np.array_equal(results[0], p0)
    assert results[0].tobytes() == results[1].tobytes()


def test_sequential_mirror_lenet_100_steps(ctx, oracle):
    """Benchmark configuration 1 through the Python mirror of network<sequential>:
    LeNet-5, batch 16, 100 adagrad steps on +-1 targets; weights within 1e-3 of the oracle."""
    net = nw.lenet5().build(16, ctx)
    rng = np.random.default_rng(1001)
    p0 = net.init_weight(rng)
    specs, keep = build_net_specs("lenet")
    assert net.n_params == net_layout(specs)[1] == 52012  # incl. unused average-pool slots
    onet, oparams = orc_net_for(oracle, specs, 16, p0)
    x = rng.uniform(-1, 1, (1600, 1024)).astype(np.float32)
    labels = rng.integers(0, 10, 1600)
    t = np.full((1600, 10), -1.0, np.float32)
    t[np.arange(1600), labels] = 1.0
    opt = nw.adagrad(0.01)
    net.fit(opt, x, t, 16, 1, nw.LOSS_MSE)
    h = opt.hyper()
    for s in range(100):
        oracle.orc_net_train_step(onet, o.p(x[s * 16:(s + 1) * 16]), o.p(t[s * 16:(s + 1) * 16]), 16, 0, 0,
                                  C.byref(h))
    p = net.get_params()
    for off, ln, _, _, _ in net_layout(specs)[0]:
        assert_close(p[off:off + ln], oparams[off:off + ln], GRAD_TOL, f"lenet 100 steps weights@{off}")
    oracle.orc_net_destroy(onet)
    net.close()


def test_fit_host_equals_step_by_step(ctx):
    """b200_net_fit_host (uploads overlapped with the steps, two epochs, a last mini-batch of 4 new
    samples completed with the previous step's rows as network::fit does) ends with exactly the
    weights of one b200_net_train_step_host call per mini-batch on explicitly assembled rows, and
    returns the forward output of every step's new samples."""
    specs, keep = build_net_specs("cifar")
    B, n = 8, 28  # 3 full mini-batches and one of 4 new samples per epoch
    rng = np.random.default_rng(5)
    x = rng.standard_normal((n, 3072)).astype(np.float32)
    t = np.zeros((n, 10), np.float32)
    t[np.arange(n), rng.integers(0, 10, n)] = 1.0
    p0 = xavier_params(specs, 11)
    h = hyper_for(1)
    a, b = DeviceNet(ctx, specs, B), DeviceNet(ctx, specs, B)
    a.set_params(p0)
    b.set_params(p0)
    outs_a = np.zeros((n, 10), np.float32)
    outs_b = np.zeros((n, 10), np.float32)
    xp, tp = torch.from_numpy(x).pin_memory(), torch.from_numpy(t).pin_memory()
    check(a.lib.b200_net_fit_host(a.h, ptr(xp), ptr(tp), n, B, 2, 1, 1, C.byref(h), ptr(outs_a)))
    xb, tb = np.zeros((B, 3072), np.float32), np.zeros((B, 10), np.float32)  # in_batch_ / t_batch_
    for epoch in range(2):
        for i in range(0, n, B):
            nb = min(B, n - i)
            xb[:nb], tb[:nb] = x[i:i + nb], t[i:i + nb]
            out = np.empty((B, 10), np.float32)
            check(b.lib.b200_net_train_step_host(b.h, ptr(xb), ptr(tb), B, 1, 1, C.byref(h), ptr(out)))
            outs_b[i:i + nb] = out[:nb]
    assert np.array_equal(a.params(), b.params())
    assert np.array_equal(outs_a, outs_b)
    a.close()
    b.close()


@pytest.mark.parametrize("name", ["lenet_165_b16_e2", "cifar_28_b8_e2", "lenet_33_b16_e1", "tiny_23_b5_e3"])
def test_fit_host_ragged_last_batch_vs_reference(ctx, gold, name):
    """network::fit over a sample count that is not a multiple of the mini-batch (short last step
    completed with the previous step's rows; a single left-over sample as a one-sample step):
    b200_net_fit_host against the weights the reference ends with."""
    from cases import gen_ragged_fit_data
    c, x, t, n_samples, B, epochs = gen_ragged_fit_data(name)
    specs, keep = build_net_specs(c["net"])
    dnet = DeviceNet(ctx, specs, B)
    dnet.set_params(xavier_params(specs, c["seed"]))
    h = hyper_for(c["opt"])
    check(dnet.lib.b200_net_fit_host(dnet.h, ptr(x), ptr(t), n_samples, B, epochs, c["loss"], c["opt"], C.byref(h),
                                     None))
    p, p1 = dnet.params(), gold[f"fit_ragged/{name}/p1"]
    for off, ln, _, _, _ in net_layout(specs)[0]:
        assert_close(p[off:off + ln], p1[off:off + ln], GRAD_TOL, f"{name} weights@{off} vs reference")
    dnet.close()


def test_fit_host_refuses_a_short_first_batch(ctx):
    """Fewer samples than one mini-batch (and more than one): the reference would read rows of its
    batch buffers that were never set; the library says so instead."""
    specs, keep = build_net_specs("tiny_conv")
    dnet = DeviceNet(ctx, specs, 8)
    x, t = np.zeros((3, 288), np.float32), np.zeros((3, 6), np.float32)
    h = hyper_for(0)
    assert dnet.lib.b200_net_fit_host(dnet.h, ptr(x), ptr(t), 3, 8, 1, 2, 0, C.byref(h), None) != 0
    assert b"no earlier full mini-batch" in dnet.lib.b200_last_error()
    dnet.close()


def test_net_rejects_bad_input(ctx):
    specs, keep = build_net_specs("tiny_conv")
    dnet = DeviceNet(ctx, specs, 4)
    x = torch.zeros(8, 288, device="cuda")
    with pytest.raises(Exception):
        check(dnet.lib.b200_net_forward(dnet.h, ptr(x), 8))  # batch above max_batch
    bad = list(specs)
    bad[5].fc_in = 81  # does not match the 80 outputs of the layer before
    arr = (LayerSpec * len(bad))(*bad)
    h = C.c_void_p()
    assert dnet.lib.b200_net_create(ctx.handle, arr, len(bad), 4, C.byref(h)) != 0
    dnet.close()


def test_second_fit_resets_state_and_keeps_adam_powers(ctx, oracle, monkeypatch):
    """What a second network::fit call with the same adam object means (fit calls
    optimizer.reset(): the per-weight state is cleared, b1_t / b2_t carry on, network.h:856,
    optimizer.h:36-38): b200_net_opt_reset + b200_net_set_adam_powers against the oracle."""
    monkeypatch.setenv("B200_NET_NO_GRAPH", "0")
    c = NET_CASES["cifar_adam"]
    specs, keep = build_net_specs(c["net"])
    B, steps = c["B"], c["steps"]
    p0 = xavier_params(specs, 31)
    x, t = gen_net_data(c)
    h = hyper_for(1)
    dnet = DeviceNet(ctx, specs, B)
    dnet.set_params(p0)
    onet, oparams = orc_net_for(oracle, specs, B, p0)
    dx = torch.empty(B, c["in_dim"], device="cuda")
    dt = torch.empty(B, c["out_dim"], device="cuda")
    for rep in range(2):
        if rep == 1:
            a, b = C.c_float(), C.c_float()
            check(dnet.lib.b200_net_adam_powers(dnet.h, C.byref(a), C.byref(b)))
            oa, ob = C.c_float(), C.c_float()
            oracle.orc_net_adam_powers(onet, C.byref(oa), C.byref(ob))
            assert (a.value, b.value) == (oa.value, ob.value)
            check(dnet.lib.b200_net_opt_reset(dnet.h, 1))
            check(dnet.lib.b200_net_set_adam_powers(dnet.h, h.b1, h.b2, a.value, b.value))
            oracle.orc_net_opt_reset(onet, 1)
        for s in range(steps):
            xs, ts = x[s * B:(s + 1) * B], t[s * B:(s + 1) * B]
            dx.copy_(torch.from_numpy(xs))
            dt.copy_(torch.from_numpy(ts))
            torch.cuda.synchronize()
            check(dnet.lib.b200_net_train_step(dnet.h, ptr(dx), ptr(dt), B, c["loss"], 1, C.byref(h)))
            oracle.orc_net_train_step(onet, o.p(np.ascontiguousarray(xs)), o.p(np.ascontiguousarray(ts)), B, c["loss"],
                                      1, C.byref(h))
        ctx.sync()
        p = dnet.params()
        for off, ln, _, _, _ in net_layout(specs)[0]:
            assert_close(p[off:off + ln], oparams[off:off + ln], GRAD_TOL, f"fit {rep} weights@{off}")
    # optimizer state export equals the oracle's view of mt / vt within the gradient tolerance
    s0 = np.empty(dnet.n, np.float32)
    check(dnet.lib.b200_net_get_opt_state(dnet.h, 0, ptr(s0)))
    check(dnet.lib.b200_net_set_opt_state(dnet.h, 0, ptr(s0)))
    s0b = np.empty(dnet.n, np.float32)
    check(dnet.lib.b200_net_get_opt_state(dnet.h, 0, ptr(s0b)))
    assert np.array_equal(s0, s0b) and np.abs(s0).max() > 0
    dnet.close()
    oracle.orc_net_destroy(onet)
