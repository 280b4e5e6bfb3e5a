"""World-size-2 gloo test of the data-parallel host logic on CPU.

Two processes each step the oracle's network on half of a batch, SUM-all-reduce
the flat gradient bucket through tiny_cnn_b200.parallel.DataParallel and update;
the result must equal one process stepping the whole batch (up to the float
re-association of the batch sum)."""
import ctypes as C
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from tiny_cnn_b200.parallel import DataParallel, shard_bounds  # noqa: E402


def test_shard_bounds_cover_the_batch():
    for n, w in [(256, 8), (10, 3), (7, 8), (0, 2), (2048, 8)]:
        got = [shard_bounds(n, w, r) for r in range(w)]
        assert got[0][0] == 0 and got[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(got, got[1:]))
        sizes = [hi - lo for lo, hi in got]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def test_peer_reduce_is_off_without_gpus():
    """On CPU buckets (and for a single rank) the peer-memory reduction declines without touching
    the library or the process group; the driver keeps the all-reduce of torch.distributed."""
    from tiny_cnn_b200.parallel import DataParallel

    class Net:
        def grads_tensor(self):
            return torch.zeros(8)

    dp = DataParallel(Net())
    assert dp.world == 1 and dp.peer is False
    assert dp.enable_peer_reduce() is False and dp.peer is False
    dp.world = 2  # a CPU bucket never takes the peer path either
    assert dp.enable_peer_reduce() is False and dp.peer is False


class OracleNet:
    """The oracle's CPU network behind the interface DataParallel drives."""

    def __init__(self, case_name, batch):
        import oracle_lib as o
        from cases import NET_CASES, build_net_specs, xavier_params
        self.o, self.lib = o, o.load_oracle()
        c = NET_CASES[case_name]
        specs, self.keep = build_net_specs(c["net"])
        arr = (type(specs[0]) * len(specs))(*specs)
        self.h = self.lib.orc_net_create(arr, len(specs), batch)
        self.n = self.lib.orc_net_param_count(self.h)
        self.params = np.ctypeslib.as_array(self.lib.orc_net_params(self.h), shape=(self.n,))
        self.params[:] = xavier_params(specs, c["seed"])
        self.grads = np.ctypeslib.as_array(self.lib.orc_net_grads(self.h), shape=(self.n,))
        self.x = None

    def grads_tensor(self):
        return torch.from_numpy(self.grads)

    def forward(self, x):
        self.x = np.ascontiguousarray(x)
        self.lib.orc_net_forward(self.h, self.o.p(self.x), self.x.shape[0])

    def backward(self, t, loss):
        t = np.ascontiguousarray(t)
        self.lib.orc_net_backward(self.h, self.o.p(self.x), self.o.p(t), loss, t.shape[0])

    def update(self, opt_and_hyper):
        kind, h = opt_and_hyper
        self.lib.orc_net_update(self.h, kind, C.byref(h))


def _worker(rank, world, port, case_name, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cases import NET_CASES, gen_net_data, hyper_for
    c = NET_CASES[case_name]
    x, t = gen_net_data(c)
    B = c["B"]
    lo, hi = shard_bounds(B, world, rank)
    net = OracleNet(case_name, B)
    dp = DataParallel(net)
    h = hyper_for(c["opt"])
    for s in range(c["steps"]):
        xs, ts = x[s * B:(s + 1) * B], t[s * B:(s + 1) * B]
        dp.train_onebatch((c["opt"], h), xs[lo:hi], ts[lo:hi], c["loss"])
    q.put((rank, net.params.copy()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("case_name", ["tiny_conv_adam", "mlp_momentum"])
def test_two_rank_data_parallel_equals_single_process(case_name):
    from cases import NET_CASES, gen_net_data, hyper_for
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, case_name, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # replicas hold bit-identical parameters
    assert np.array_equal(results[0], results[1])
    # and they match one process on the whole batch
    c = NET_CASES[case_name]
    x, t = gen_net_data(c)
    B = c["B"]
    net = OracleNet(case_name, B)
    h = hyper_for(c["opt"])
    for s_ in range(c["steps"]):
        net.forward(x[s_ * B:(s_ + 1) * B])
        net.backward(t[s_ * B:(s_ + 1) * B], c["loss"])
        net.update((c["opt"], h))
    scale = np.abs(net.params).max()
    assert np.abs(results[0] - net.params).max() <= 1e-3 * scale
