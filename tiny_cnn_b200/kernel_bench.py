"""Single-layer timing of the convolution kernels through the C ABI.

    python -m tiny_cnn_b200.kernel_bench --layer conv2 --batch 256 --reps 5 --passes fwd,bwd

Prints one JSON line with the CUDA-event time per pass and the achieved
TFLOP/s (2*B*oh*ow*oc*ic*kh*kw flop per pass: forward, dX and dW each).
It is also the small, self-terminating program used for `ncu` captures.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from . import ops
from ._lib import check, ptr

# name -> (width, in_c, out_c, window), all stride 1, padding same
LAYERS = {
    "conv1": (32, 3, 32, 5), "conv2": (16, 32, 32, 5), "conv3": (8, 32, 64, 5),   # CIFAR-10 net
    "lenet_c1": (32, 1, 6, 5), "lenet_c3": (14, 6, 16, 5),
    "sweep56": (56, 64, 64, 3), "sweep28": (28, 128, 128, 3), "sweep14": (14, 256, 256, 3),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layer", default="conv2", choices=sorted(LAYERS))
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--passes", default="fwd,bwd")
    ap.add_argument("--algo", type=int, default=0)
    args = ap.parse_args()
    w, c, oc, k = LAYERS[args.layer]
    B = args.batch
    ctx = ops.Context(0)
    d = ops.conv_params(w, w, c, k, k, oc, True, True, algo=args.algo)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(B, c * w * w, device="cuda", generator=g)
    W = (torch.rand(oc * c * k * k, device="cuda", generator=g) - 0.5) * 0.2
    b = torch.zeros(oc, device="cuda")
    dy = torch.randn(B, oc * w * w, device="cuda", generator=g)
    y, dx = torch.empty_like(dy), torch.empty_like(x)
    dW, db = torch.zeros_like(W), torch.zeros_like(b)
    lib, h = ctx.lib, ctx.handle
    fns = {
        "fwd": lambda: check(lib.b200_conv2d_fwd(h, C.byref(d), ptr(x), ptr(W), ptr(b), ptr(y), B)),
        "bwd": lambda: check(lib.b200_conv2d_bwd(h, C.byref(d), ptr(x), ptr(W), ptr(dy), ptr(dx), ptr(dW),
                                                 ptr(db), 0, B)),
        "dw": lambda: check(lib.b200_conv2d_bwd(h, C.byref(d), ptr(x), ptr(W), ptr(dy), None, ptr(dW),
                                                ptr(db), 0, B)),
    }
    flop = 2.0 * B * w * w * oc * c * k * k
    out = {"layer": args.layer, "batch": B, "flop_per_pass": flop}
    for name in args.passes.split(","):
        fn = fns[name]
        for _ in range(args.warmup):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / args.reps
        npass = 2 if name == "bwd" else 1
        out[name] = {"ms": round(ms, 4), "tflops": round(npass * flop / (ms * 1e-3) / 1e12, 3)}
    print(json.dumps(out))


if __name__ == "__main__":
    main()
