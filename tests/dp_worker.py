"""Worker of test_parallel_gpu.py: one process per GPU under torch.distributed.run.

Trains the small convolutional test network for a few data-parallel steps twice from the same
weights -- once with the gradient bucket summed by the library's peer-memory kernel inside the
step's graph, once with the NCCL all-reduce between forward_backward and update -- and checks that
the replicas agree bit for bit with each other and (two ranks: a + b in either order) with the
NCCL run, and that rank 0's weights equal -- within the 1e-3 weight tolerance -- what the CPU
oracle reaches in the same steps on the concatenated mini-batch (gradients are summed over the
batch with no 1/N, so sharding the batch must not change the result).  Both runs use the model's
fixed tile choices (B200_AUTOTUNE unset) and end with Context.sync(), which raises when a bounded
wait of the reduction ran out.  Prints `DP_WORKER_OK` on rank 0 when everything held.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from tiny_cnn_b200 import network as nw  # noqa: E402
from tiny_cnn_b200 import ops  # noqa: E402
from tiny_cnn_b200._lib import LOSS_CROSS_ENTROPY  # noqa: E402
from tiny_cnn_b200.parallel import DataParallel  # noqa: E402


def batch_of(rank, step, B):
    """Rank `rank`'s shard of step `step`: the same bytes wherever they are generated."""
    rng = np.random.default_rng(100 + 1000 * step + rank)
    x = rng.uniform(-1, 1, (B, 3072)).astype(np.float32)
    t = np.zeros((B, 10), np.float32)
    t[np.arange(B), rng.integers(0, 10, B)] = 1.0
    return x, t


def oracle_params(world, steps, B):
    """The CPU oracle's weights after the same steps on the concatenated mini-batches."""
    import oracle_lib as o
    from cases import build_net_specs, hyper_for, xavier_params  # noqa: F401
    from tiny_cnn_b200._lib import LayerSpec
    orc = o.load_oracle()
    specs, keep = build_net_specs("cifar")
    arr = (LayerSpec * len(specs))(*specs)
    net = orc.orc_net_create(arr, len(specs), B * world)
    n = orc.orc_net_param_count(net)
    params = np.ctypeslib.as_array(orc.orc_net_params(net), shape=(n,))
    return orc, net, params


def run(rank, world, local, use_peer, steps, B):
    ctx = ops.Context(local)
    net = nw.cifar10_net(local).build(B, ctx)
    p0 = net.init_weight(np.random.default_rng(3))
    opt = nw.adam(1e-3)
    dp = DataParallel(net)
    if use_peer:
        assert dp.enable_peer_reduce(rendezvous=use_peer), f"peer mapping by {use_peer} unavailable"
        assert dp.rendezvous == use_peer
    for s in range(steps):
        xh, th = batch_of(rank, s, B)
        x, t = torch.from_numpy(xh).cuda(), torch.from_numpy(th).cuda()
        dp.train_onebatch(opt, x, t, LOSS_CROSS_ENTROPY)
    dp.check()  # raises if a wait of the reduction for another rank ran out (code 7)
    p = torch.from_numpy(net.get_params()).cuda()
    net.close()
    return p, p0


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    steps, B = 4, 16  # step 1 eager, step 2 captured, steps 3-4 replayed; both halves of the buffer twice
    # the exchange buffers mapped by the library's own inter-process handles, then by torch symmetric memory
    p_peer, p0 = run(rank, world, local, "ipc", steps, B)
    p_symm, _ = run(rank, world, local, "symm", steps, B)
    p_nccl, _ = run(rank, world, local, None, steps, B)
    gathered = [torch.empty_like(p_peer) for _ in range(world)]
    dist.all_gather(gathered, p_peer)
    ok = all(torch.equal(gathered[0], g) for g in gathered) and torch.equal(p_peer, p_symm)
    if world == 2:
        ok = ok and torch.equal(p_peer, p_nccl)
    else:
        ok = ok and torch.allclose(p_peer, p_nccl, rtol=1e-4, atol=1e-6)
    moved = not torch.equal(p_peer, torch.from_numpy(p0).cuda())
    if rank == 0:
        # the oracle on the concatenated mini-batch
        import oracle_lib as o
        from cases import build_net_specs, hyper_for, net_layout
        orc, onet, oparams = oracle_params(world, steps, B)
        oparams[:] = p0
        h = hyper_for(1)
        for s in range(steps):
            parts = [batch_of(r, s, B) for r in range(world)]
            x = np.ascontiguousarray(np.concatenate([p[0] for p in parts]))
            t = np.ascontiguousarray(np.concatenate([p[1] for p in parts]))
            orc.orc_net_train_step(onet, o.p(x), o.p(t), B * world, 1, 1, C.byref(h))
        got = p_peer.cpu().numpy()
        specs, keep = build_net_specs("cifar")
        worst = 0.0
        for off, ln, _, _, _ in net_layout(specs)[0]:
            a, b = got[off:off + ln], oparams[off:off + ln]
            worst = max(worst, float(np.abs(a - b).max() / max(float(np.abs(b).max()), 1e-30)))
        print(f"data-parallel weights vs the oracle on the concatenated batch: worst {worst:.2e} of a tensor's "
              f"largest magnitude", flush=True)
        ok = ok and worst <= 1e-3
        orc.orc_net_destroy(onet)
    flag = torch.tensor([1 if (ok and moved) else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print("DP_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
