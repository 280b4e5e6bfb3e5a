"""Data-parallel driver: the mini-batch is split contiguously over the ranks,
every rank runs forward/backward on its shard, the batch-summed weight
gradients are SUM-all-reduced (the reference sums per-sample gradients and
applies no 1/B factor: tiny_dnn/layers/layer.h:663-673, tiny_dnn/node.h:89-103),
and every rank then applies the identical optimizer update, so replicas stay
bit-identical without a parameter broadcast after step 0.

`torch.distributed` is the plumbing (NCCL over NVLink on GPUs, gloo in CPU
tests); the collective operates in place on the net's flat gradient bucket.

On GPUs `enable_peer_reduce()` moves the sum into the step itself: every rank
maps every rank's exchange buffer (the library's own inter-process handles, or torch
symmetric memory, do the rendezvous),
and the library's own kernel pushes the bucket over NVLink and adds the copies in
rank order inside the captured graph of `train_onebatch`, which is then one graph
launch per step with no collective call between two graphs.
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
        self.peer = False
        self._symm = None  # keeps the exchange buffer and its rendezvous handle alive
        self.rendezvous = None  # "ipc" or "symm" once the peer reduction is on

    def enable_peer_reduce(self, timeout_ms: int = 0, rendezvous: Optional[str] = None) -> bool:
        """Map every rank's exchange buffer into every rank and hand the addresses to the net
        (b200_net_peer_reduce_init).  Returns True when EVERY rank succeeded; otherwise all
        ranks keep the NCCL all-reduce.  Collective: every rank must call it.  `timeout_ms` bounds
        every wait of the reduction for another rank (0 = the library's default, 10 s); call
        `check()` now and then to learn of a wait that ran out.

        `rendezvous` (or the environment variable B200_PEER_RENDEZVOUS): "ipc" = the library's own
        b200_peer_buffer_create / _open with the handles gathered over the process group (what a
        C++ launcher would do), "symm" = torch symmetric memory; the default tries them in that order."""
        if self.world <= 1 or not self.bucket.is_cuda:
            return False
        import ctypes as C
        import os

        from ._lib import check
        lib, h = self.net.lib, self.net.handle
        nbytes = int(lib.b200_net_peer_reduce_bytes(h, self.world))
        mode = rendezvous or os.environ.get("B200_PEER_RENDEZVOUS", "")
        order = {"ipc": ("ipc",), "symm": ("symm",), "": ("ipc", "symm")}.get(mode)
        if order is None:
            raise ValueError(f"unknown rendezvous {mode!r}: 'ipc' or 'symm'")
        for how in order:
            ok, why, ptrs, keep = 1, "", None, None
            try:
                ptrs, keep = (self._rendezvous_ipc if how == "ipc" else self._rendezvous_symm)(nbytes)
                torch.cuda.synchronize()
            except Exception as e:  # no peer mapping this way on this system
                ok, why = 0, f"{type(e).__name__}: {e}"
            flag = torch.tensor([ok], device=self.bucket.device, dtype=torch.int32)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)  # also: every buffer is zeroed
            if int(flag.item()) == 1:
                arr = (C.c_ulonglong * self.world)(*ptrs)
                check(lib.b200_net_peer_reduce_init(h, self.rank, self.world, arr, int(timeout_ms)))
                self._symm = keep
                self.peer = True
                self.rendezvous = how
                return True
            if keep is not None and how == "ipc":
                self._release_ipc(keep)
            if why and self.rank == 0:
                import sys
                print(f"[tiny_cnn_b200] peer mapping by {how} unavailable ({why})", file=sys.stderr, flush=True)
        return False

    def _rendezvous_symm(self, nbytes):
        import torch.distributed._symmetric_memory as symm_mem
        buf = symm_mem.empty((nbytes + 3) // 4, dtype=torch.float32, device=self.bucket.device)
        buf.zero_()
        grp = self.group if self.group is not None else dist.group.WORLD
        hdl = symm_mem.rendezvous(buf, grp)
        return [int(p) for p in hdl.buffer_ptrs], (buf, hdl)

    def _rendezvous_ipc(self, nbytes):
        """Every rank creates its buffer in the library, the opaque handles travel through the
        process group, every rank opens the others'.  A rank whose creation failed still takes
        part in the gather (with None) so that no rank is left waiting."""
        import ctypes as C

        from ._lib import B200Error, check
        lib, ctx = self.net.lib, self.net.ctx.handle
        own, handle, err = C.c_void_p(), (C.c_ubyte * 64)(), None
        try:
            check(lib.b200_peer_buffer_create(ctx, nbytes, C.byref(own), handle))
        except B200Error as e:
            err = e
        handles = [None] * self.world
        dist.all_gather_object(handles, None if err else bytes(handle), group=self.group)
        keep = {"own": own.value, "opened": []}
        if err is not None or any(hb is None for hb in handles):
            self._release_ipc(keep)
            raise err if err is not None else RuntimeError("another rank could not create its buffer")
        ptrs = []
        try:
            for r, hb in enumerate(handles):
                if r == self.rank:
                    ptrs.append(own.value)
                    continue
                q = C.c_void_p()
                check(lib.b200_peer_buffer_open(ctx, (C.c_ubyte * 64).from_buffer_copy(hb), C.byref(q)))
                keep["opened"].append(q.value)
                ptrs.append(q.value)
        except B200Error:
            self._release_ipc(keep)
            raise
        return ptrs, keep

    def _release_ipc(self, keep):
        """Unmap the other ranks' buffers.  The own buffer stays allocated until the process ends:
        another rank may still have it mapped."""
        lib, ctx = self.net.lib, self.net.ctx.handle
        for q in keep.get("opened", []):
            lib.b200_peer_buffer_close(ctx, q)
        keep["opened"] = []

    def check(self):
        """Wait for this rank's queued work and raise if a kernel gave up a bounded wait (a reduction
        over the replicas that timed out: this rank skipped the update, the replicas now differ)."""
        ctx = getattr(self.net, "ctx", None)
        if ctx is not None:
            ctx.sync()

    def allreduce_grads(self):
        """In-place SUM over ranks of the gradient bucket (no averaging)."""
        if self.world > 1:
            if self.peer:
                from ._lib import check
                check(self.net.lib.b200_net_peer_reduce(self.net.handle))
            else:
                dist.all_reduce(self.bucket, op=dist.ReduceOp.SUM, group=self.group)

    def train_onebatch(self, opt, x_shard, t_shard, loss: int):
        """One data-parallel step on this rank's shard."""
        if self.peer and hasattr(self.net, "train_onebatch"):
            # the reduction is part of the net's captured step: one graph launch
            self.net.train_onebatch(opt, x_shard, t_shard, loss)
            return
        self.net.forward(x_shard)
        self.net.backward(t_shard, loss)
        self.allreduce_grads()
        self.net.update(opt)

    def broadcast_params(self, params: torch.Tensor, src: int = 0):
        """Make every replica start from rank `src`'s parameters."""
        if self.world > 1:
            dist.broadcast(params, src=src, group=self.group)
        return params
