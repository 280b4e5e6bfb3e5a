"""The gradient sum over data-parallel replicas (csrc/peer_reduce.cu) on ONE GPU.

Two "ranks" are two nets of the same process whose exchange buffers both live in this GPU's
memory.  Kernels that wait for one another must never be separate launches on one GPU, so
the ranks run one after the other and every rank pushes before any rank sums
(b200_net_peer_push / b200_net_peer_sum): by the time a summing kernel starts, every flag it
looks at is already set.  The result is compared with the CPU oracle's step on the
concatenated mini-batch -- what a reduction over replicas must equal (gradients are summed,
tiny_dnn/layers/layer.h:663-673) -- at the 1e-3 gradient / weight tolerance.

The bounded wait is tested with a flag that nothing sets: a world of two whose second rank
never runs, time limit 20 ms; the step must end, report code 7 through b200_ctx_sync and
leave the parameters unchanged."""
import ctypes as C

import numpy as np
import pytest
import torch

import oracle_lib as o
from cases import build_net_specs, hyper_for, net_layout, xavier_params
from test_net_gpu import DeviceNet, orc_net_for
from test_ops_gpu import GRAD_TOL, assert_close
from tiny_cnn_b200 import ops
from tiny_cnn_b200._lib import check, ptr

pytestmark = pytest.mark.gpu


def exchange_buffers(ctx, net, world):
    nbytes = int(ctx.lib.b200_net_peer_reduce_bytes(net.h, world))
    bufs = [torch.zeros((nbytes + 3) // 4, dtype=torch.float32, device="cuda") for _ in range(world)]
    torch.cuda.synchronize()
    return bufs, (C.c_ulonglong * world)(*[b.data_ptr() for b in bufs])


@pytest.mark.parametrize("netname,B,in_dim,out_dim,loss,opt", [
    ("cifar", 16, 3072, 10, 1, 1),
    ("tiny_conv", 5, 288, 6, 2, 0),
])
def test_two_ranks_on_one_gpu_equal_the_oracle_on_the_concatenated_batch(ctx, oracle, netname, B, in_dim, out_dim,
                                                                         loss, opt, monkeypatch):
    monkeypatch.setenv("B200_NET_NO_GRAPH", "1")
    world, steps = 2, 3  # both halves of the exchange buffer, and the first one again
    specs, keep = build_net_specs(netname)
    layout, n = net_layout(specs)
    p0 = xavier_params(specs, 77)
    nets = [DeviceNet(ctx, specs, B) for _ in range(world)]
    bufs, addrs = exchange_buffers(ctx, nets[0], world)
    for r, net in enumerate(nets):
        net.set_params(p0)
        check(ctx.lib.b200_net_peer_reduce_init(net.h, r, world, addrs, 1000))
    onet, oparams = orc_net_for(oracle, specs, B * world, p0)
    rng = np.random.default_rng(78)
    h = hyper_for(opt)
    for s in range(steps):
        x = rng.standard_normal((world * B, in_dim)).astype(np.float32)
        t = np.zeros((world * B, out_dim), np.float32)
        t[np.arange(world * B), rng.integers(0, out_dim, world * B)] = 1.0
        xd, td = torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda()
        for r, net in enumerate(nets):
            check(ctx.lib.b200_net_forward(net.h, ptr(xd[r * B:(r + 1) * B]), B))
            check(ctx.lib.b200_net_backward(net.h, ptr(td[r * B:(r + 1) * B]), loss))
        for net in nets:
            check(ctx.lib.b200_net_peer_push(net.h))
        for net in nets:
            check(ctx.lib.b200_net_peer_sum(net.h))
        ctx.sync()
        oracle.orc_net_forward(onet, o.p(x), world * B)
        oracle.orc_net_backward(onet, o.p(x), o.p(t), loss, world * B)
        g_ref = np.ctypeslib.as_array(oracle.orc_net_grads(onet), shape=(n,)).copy()
        g0, g1 = nets[0].grads(), nets[1].grads()
        assert np.array_equal(g0, g1), "the ranks summed to different buckets"
        for off, ln, _, _, _ in layout:
            assert_close(g0[off:off + ln], g_ref[off:off + ln], GRAD_TOL, f"{netname} step {s} summed grad@{off}")
        for net in nets:
            check(ctx.lib.b200_net_update(net.h, opt, C.byref(h)))
        oracle.orc_net_update(onet, opt, C.byref(h))
        ctx.sync()
        pa, pb = nets[0].params(), nets[1].params()
        assert np.array_equal(pa, pb), "replicas differ after the update"
        for off, ln, _, _, _ in layout:
            assert_close(pa[off:off + ln], oparams[off:off + ln], GRAD_TOL, f"{netname} step {s} weights@{off}")
    for net in nets:
        net.close()
    oracle.orc_net_destroy(onet)
    del bufs


@pytest.mark.parametrize("graph", ["0", "1"])
def test_wait_for_a_rank_that_never_comes_times_out(ctx, graph, monkeypatch):
    """World of two, only rank 0 runs: the summing kernel's wait (20 ms limit) runs out, the
    update of that step is skipped, and b200_ctx_sync reports code 7."""
    monkeypatch.setenv("B200_NET_NO_GRAPH", "0" if graph == "1" else "1")
    specs, keep = build_net_specs("tiny_conv")
    B = 4
    p0 = xavier_params(specs, 5)
    net = DeviceNet(ctx, specs, B)
    net.set_params(p0)
    bufs, addrs = exchange_buffers(ctx, net, 2)
    check(ctx.lib.b200_net_peer_reduce_init(net.h, 0, 2, addrs, 20))
    rng = np.random.default_rng(6)
    x = torch.from_numpy(rng.standard_normal((B, 288)).astype(np.float32)).cuda()
    t = torch.zeros(B, 6, device="cuda")
    t[:, 0] = 1.0
    h = hyper_for(1)
    ctx.sync()
    check(ctx.lib.b200_net_train_step(net.h, ptr(x), ptr(t), B, 2, 1, C.byref(h)))
    with pytest.raises(ops.B200Error, match="code 7"):
        ctx.sync()
    assert np.array_equal(net.params(), p0), "a step whose reduction timed out must not change the parameters"
    ctx.sync()  # the error word was cleared by the report
    net.close()
    del bufs


def test_peer_reduce_rejects_bad_arguments(ctx):
    specs, keep = build_net_specs("tiny_conv")
    net = DeviceNet(ctx, specs, 4)
    bufs, addrs = exchange_buffers(ctx, net, 2)
    lib = ctx.lib
    assert lib.b200_net_peer_reduce_init(net.h, 2, 2, addrs, 0) != 0      # rank outside the world
    assert lib.b200_net_peer_reduce_init(net.h, 0, 1, addrs, 0) != 0      # a world of one has nothing to sum
    assert lib.b200_net_peer_reduce_init(net.h, 0, 2, addrs, -5) != 0     # negative time limit
    bad = (C.c_ulonglong * 2)(bufs[0].data_ptr(), bufs[1].data_ptr() + 4)  # not 16-byte aligned
    assert lib.b200_net_peer_reduce_init(net.h, 0, 2, bad, 0) != 0
    assert lib.b200_net_peer_sum(net.h) != 0                               # never initialised
    net.close()
