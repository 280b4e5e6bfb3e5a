"""Kernel timeline of graph-replayed training steps of the CIFAR-10 network.

`python -m tiny_cnn_b200.step_timeline [--batch 256] [--steps 5]` prints, for the last of `steps`
replayed steps, every kernel with its start offset and duration in microseconds.  The times come
from CUPTI through `torch.profiler`, which records the kernels of every library in the process, so
kernels inside a replayed CUDA graph and on both of the step's streams are seen as they really
overlap (a per-kernel profiler serialises them).  Needs a GPU; there is no CPU path.
"""
from __future__ import annotations

import argparse
import re

import numpy as np
import torch

from . import network as nw
from . import ops
from ._lib import LOSS_CROSS_ENTROPY


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--steps", type=int, default=5)
    args = ap.parse_args()
    ctx = ops.Context(0)
    net = nw.cifar10_net(0).build(args.batch, ctx)
    net.init_weight(np.random.default_rng(42))
    opt = nw.adam(1e-3)
    rng = np.random.default_rng(7)
    x = torch.from_numpy(rng.uniform(-1, 1, (args.batch, 3 * 32 * 32)).astype(np.float32)).cuda()
    t_host = np.zeros((args.batch, 10), np.float32)
    t_host[np.arange(args.batch), rng.integers(0, 10, args.batch)] = 1.0
    t = torch.from_numpy(t_host).cuda()
    loss_ce = LOSS_CROSS_ENTROPY  # as the benchmark step
    for _ in range(10):  # warm-up: tile choices, graph capture
        net.train_onebatch(opt, x, t, loss_ce)
    torch.cuda.synchronize()
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(max(2, args.steps)):
            net.train_onebatch(opt, x, t, loss_ce)
        torch.cuda.synchronize()
    evs = [e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA]
    evs.sort(key=lambda e: e.time_range.start)
    marks = [i for i, e in enumerate(evs) if "opt_advance_powers" in e.name]  # first kernel of a step
    if len(marks) < 2:
        raise SystemExit("fewer than two steps were recorded")
    a, b = marks[-2], marks[-1]
    t0 = evs[a].time_range.start
    print(f"step span {evs[b].time_range.start - t0:.1f} us, {b - a} kernels")
    for e in evs[a:b]:
        m = re.search(r"(\w+_kernel)", e.name)
        name = m.group(1) if m else e.name[:48]
        print(f"{e.time_range.start - t0:8.1f} {e.time_range.end - e.time_range.start:7.1f}  {name}")


if __name__ == "__main__":
    main()
