"""Data-parallel driver: the mini-batch is split contiguously over the ranks,
every rank runs forward/backward on its shard, the batch-summed weight
gradients are SUM-all-reduced (the reference sums per-sample gradients and
applies no 1/B factor: tiny_dnn/layers/layer.h:663-673, tiny_dnn/node.h:89-103),
and every rank then applies the identical optimizer update, so replicas stay
bit-identical without a parameter broadcast after step 0.

`torch.distributed` is the plumbing (NCCL over NVLink on GPUs, gloo in CPU
tests); the collective operates in place on the net's flat gradient bucket.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def shard_bounds(n_total: int, world: int, rank: int):
    """Contiguous [lo, hi) rows of rank `rank` when `n_total` rows are split over `world`
    ranks; the first n_total % world ranks take one extra row."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError(f"bad rank {rank} of {world}")
    base, extra = divmod(n_total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


class DataParallel:
    """Wraps a net exposing forward(x), backward(t, loss), update(opt) and
    grads_tensor() (a torch view of its flat gradient bucket)."""

    def __init__(self, net, group: Optional[dist.ProcessGroup] = None):
        self.net = net
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.bucket = net.grads_tensor()

    def allreduce_grads(self):
        """In-place SUM over ranks of the gradient bucket (no averaging)."""
        if self.world > 1:
            dist.all_reduce(self.bucket, op=dist.ReduceOp.SUM, group=self.group)

    def train_onebatch(self, opt, x_shard, t_shard, loss: int):
        """One data-parallel step on this rank's shard."""
        self.net.forward(x_shard)
        self.net.backward(t_shard, loss)
        self.allreduce_grads()
        self.net.update(opt)

    def broadcast_params(self, params: torch.Tensor, src: int = 0):
        """Make every replica start from rank `src`'s parameters."""
        if self.world > 1:
            dist.broadcast(params, src=src, group=self.group)
        return params
