"""Single-layer timing of the kernels through the C ABI.

    python bench_layers.py --layer conv2 --batch 256 --reps 5 --passes fwd,bwd
    python bench_layers.py --layer fc4096 --batch 1024        (MLP configuration layers)
    python bench_layers.py --layer qconv --batch 128          (quantized configuration)

Prints one JSON line with the CUDA-event time per pass and the achieved
TFLOP/s (2*B*oh*ow*oc*ic*kh*kw flop per pass: forward, dX and dW each).
It is also the small, self-terminating program used for `ncu` captures.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json

import torch

from tiny_cnn_b200 import ops
from tiny_cnn_b200._lib import check, ptr

# name -> (width, in_c, out_c, window), all stride 1, padding same
LAYERS = {
    "conv1": (32, 3, 32, 5), "conv2": (16, 32, 32, 5), "conv3": (8, 32, 64, 5),   # CIFAR-10 net
    "lenet_c1": (32, 1, 6, 5), "lenet_c3": (14, 6, 16, 5),
    "sweep56": (56, 64, 64, 3), "sweep28": (28, 128, 128, 3), "sweep14": (14, 256, 256, 3),
}


# name -> (in, out) of the fully-connected layers of the MLP configuration
FC_LAYERS = {"fc784": (784, 4096), "fc4096": (4096, 4096), "fc10": (4096, 10)}


def timed(fn, reps, warmup):
    for _ in range(warmup):
        fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def other_layers(args, ctx):
    """Fully-connected layers of the MLP configuration and the quantized forward layers."""
    B = args.batch
    g = torch.Generator(device="cuda").manual_seed(2)
    out = {"layer": args.layer, "batch": B}
    if args.layer in FC_LAYERS:
        I, O = FC_LAYERS[args.layer]
        x = torch.rand(B, I, device="cuda", generator=g)
        W = (torch.rand(I * O, device="cuda", generator=g) - 0.5) * 0.05
        b = torch.zeros(O, device="cuda")
        dy = torch.randn(B, O, device="cuda", generator=g)
        y = torch.empty(B, O, device="cuda")
        dW, db = torch.empty_like(W), torch.empty_like(b)
        flop = 2.0 * B * I * O
        ms = timed(lambda: ops.fully_connected_op(ctx, I, O, x, W, b, out=y), args.reps, args.warmup)
        out["fwd"] = {"ms": round(ms, 4), "tflops": round(flop / ms / 1e9, 3)}
        ms = timed(lambda: ops.fully_connected_grad_op(ctx, I, O, x, W, dy, dW=dW, db=db), args.reps, args.warmup)
        out["bwd"] = {"ms": round(ms, 4), "tflops": round(2 * flop / ms / 1e9, 3)}
    elif args.layer == "qconv":  # 32 x 28 x 28 -> 64 maps, 5x5, valid (stride from --stride)
        d = ops.conv_params(28, 28, 32, 5, 5, 64, False, True, args.stride, args.stride)
        x = torch.rand(B, 32 * 28 * 28, device="cuda", generator=g) * 2 - 1
        W = torch.rand(64 * 32 * 25, device="cuda", generator=g) - 0.5
        b = torch.zeros(64, device="cuda")
        ms = timed(lambda: ops.quantized_conv2d(ctx, d, x, W, b), args.reps, args.warmup)
        macs = B * 64 * d.out_w * d.out_h * 32 * 25
        out["fwd"] = {"ms": round(ms, 4), "int_tops": round(2.0 * macs / ms / 1e9, 3)}
    elif args.layer == "bn":  # batch normalization, 64 channels x 32 x 32 (an HBM-bound layer: bytes, not flops)
        Cn, S = 64, 1024
        x = torch.randn(B, Cn * S, device="cuda", generator=g)
        dy = torch.randn(B, Cn * S, device="cuda", generator=g)
        y, mean, var, sd = ops.batch_normalization_forward(ctx, Cn, S, 1e-5, x)
        nbytes = 4.0 * B * Cn * S
        ms = timed(lambda: ops.batch_normalization_forward(ctx, Cn, S, 1e-5, x), args.reps, args.warmup)
        # two reduction passes and the normalising pass read x; one write
        out["fwd"] = {"ms": round(ms, 4), "algorithmic_gbs": round(2 * nbytes / ms / 1e6, 1),
                      "touched_gbs": round(4 * nbytes / ms / 1e6, 1)}
        ms = timed(lambda: ops.batch_normalization_backward(ctx, Cn, S, y, dy, sd), args.reps, args.warmup)
        out["bwd"] = {"ms": round(ms, 4), "algorithmic_gbs": round(3 * nbytes / ms / 1e6, 1),
                      "touched_gbs": round(5 * nbytes / ms / 1e6, 1)}
    elif args.layer == "lrn":  # across 64 channels of 32 x 32, window 5
        Cn, area = 64, 1024
        x = torch.randn(B, Cn * area, device="cuda", generator=g)
        nbytes = 4.0 * B * Cn * area
        ms = timed(lambda: ops.lrn_forward(ctx, x, Cn, area, 5, 1e-4, 0.75), args.reps, args.warmup)
        out["fwd"] = {"ms": round(ms, 4), "algorithmic_gbs": round(2 * nbytes / ms / 1e6, 1)}
    else:  # qfc 9216 -> 256
        x = torch.rand(B, 9216, device="cuda", generator=g) * 2 - 1
        W = torch.rand(9216 * 256, device="cuda", generator=g) - 0.5
        b = torch.zeros(256, device="cuda")
        ms = timed(lambda: ops.quantized_fully_connected(ctx, 9216, 256, x, W, b), args.reps, args.warmup)
        out["fwd"] = {"ms": round(ms, 4), "int_tops": round(2.0 * B * 9216 * 256 / ms / 1e9, 3)}
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--layer", default="conv2", choices=sorted(LAYERS) + sorted(FC_LAYERS) + ["qconv", "qfc", "bn", "lrn"])
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--batch", type=int, default=256)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--passes", default="fwd,bwd")
    ap.add_argument("--algo", type=int, default=0)
    args = ap.parse_args()
    ctx = ops.Context(0)
    if args.layer not in LAYERS:
        return other_layers(args, ctx)
    w, c, oc, k = LAYERS[args.layer]
    B = args.batch
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
