"""Worker of test_parallel_gpu.py: one process per GPU under torch.distributed.run.

Trains the small convolutional test network for a few data-parallel steps twice from the same
weights -- once with the gradient bucket summed by the library's peer-memory kernel inside the
step's graph, once with the NCCL all-reduce between forward_backward and update -- and checks that
the replicas agree bit for bit with each other and (two ranks: a + b in either order) with the
NCCL run.  Prints `DP_WORKER_OK` on rank 0 when everything held.
"""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from tiny_cnn_b200 import network as nw  # noqa: E402
from tiny_cnn_b200 import ops  # noqa: E402
from tiny_cnn_b200._lib import LOSS_CROSS_ENTROPY  # noqa: E402
from tiny_cnn_b200.parallel import DataParallel  # noqa: E402


def run(rank, world, local, use_peer, steps, B):
    ctx = ops.Context(local)
    net = nw.cifar10_net(local).build(B, ctx)
    net.init_weight(np.random.default_rng(3))
    opt = nw.adam(1e-3)
    dp = DataParallel(net)
    if use_peer:
        assert dp.enable_peer_reduce(), "peer mapping unavailable"
    rng = np.random.default_rng(100 + rank)
    for s in range(steps):
        x = torch.from_numpy(rng.uniform(-1, 1, (B, 3072)).astype(np.float32)).cuda()
        t_host = np.zeros((B, 10), np.float32)
        t_host[np.arange(B), rng.integers(0, 10, B)] = 1.0
        t = torch.from_numpy(t_host).cuda()
        dp.train_onebatch(opt, x, t, LOSS_CROSS_ENTROPY)
    torch.cuda.synchronize()
    p = torch.from_numpy(net.get_params()).cuda()
    net.close()
    return p


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    steps, B = 4, 16  # step 1 eager, step 2 captured, steps 3-4 replayed; both halves of the buffer twice
    p_peer = run(rank, world, local, True, steps, B)
    p_nccl = run(rank, world, local, False, steps, B)
    gathered = [torch.empty_like(p_peer) for _ in range(world)]
    dist.all_gather(gathered, p_peer)
    ok = all(torch.equal(gathered[0], g) for g in gathered)
    if world == 2:
        ok = ok and torch.equal(p_peer, p_nccl)
    else:
        ok = ok and torch.allclose(p_peer, p_nccl, rtol=1e-4, atol=1e-6)
    moved = not torch.equal(p_peer, torch.from_numpy(np.zeros(1, np.float32)).cuda().expand_as(p_peer))
    flag = torch.tensor([1 if (ok and moved) else 0], device="cuda", dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and int(flag.item()) == 1:
        print("DP_WORKER_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
