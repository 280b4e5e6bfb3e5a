"""GPU test of b200_conv2d_dw_noalloc, the weight-gradient entry point for hosts
that may not allocate device memory while they run (all HBM already handed to
their own pools, or a loop that cannot afford the device-wide synchronisation an
allocation implies).  The entry point keeps its partial sums in a fixed array
inside the library instead of a buffer grown with cudaMalloc.

It is called through the C ABI twice in a row, with different layer shapes so the
second call finds the first call's partial sums still in the array, and each
result is compared with the regular entry point b200_conv2d_bwd -- and, for the
calls that start from zero, with the CPU oracle's batch-summed weight gradient --
within the gradient tolerance of the other GPU tests.  The file sorts last so that a run
stopping at the first failure has already run every other test."""
import ctypes as C

import numpy as np
import pytest
import torch

from tiny_cnn_b200 import ops
from tiny_cnn_b200._lib import check, load, ptr

pytestmark = pytest.mark.gpu
GRAD_TOL = 1e-3


def close(got, want, tol, what):
    got, want = got.double().cpu().numpy(), want.double().cpu().numpy()
    scale = max(float(np.abs(want).max()), 1e-30)
    err = np.abs(got - want)
    assert (err <= tol * (np.abs(want) + scale)).all(), f"{what}: max err {err.max():g} (scale {scale:g})"


def oracle_dw(d, x, W, dy, batch):
    """batch-summed dW / db of the CPU restatement (oracle.c: conv2d_op_internal.h:130-179)."""
    import oracle_lib as o
    orc = o.load_oracle()
    xh, dyh = x.cpu().numpy(), dy.cpu().numpy()
    xp = o.f32(batch, d.in_c * d.inp_h * d.inp_w)
    orc.orc_conv_pad(C.byref(d), o.p(xh), o.p(xp), batch)
    dxp, dW, db = o.f32(*xp.shape), o.f32(W.numel()), o.f32(d.out_c)
    Wh = W.cpu().numpy()
    orc.orc_conv2d_bwd(C.byref(d), o.p(xp), o.p(Wh), o.p(dyh), o.p(dxp), o.p(dW), o.p(db), 0, batch)
    return torch.from_numpy(dW), torch.from_numpy(db)


def run_pair(ctx, lib, w, c, oc, k, batch, same, accumulate, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    d = ops.conv_params(w, w, c, k, k, oc, same, True)
    x = torch.randn(batch, ops.conv_in_len(d), device="cuda", generator=g)
    W = (torch.rand(ops.conv_w_len(d), device="cuda", generator=g) - 0.5) * 0.2
    dy = torch.randn(batch, ops.conv_out_len(d), device="cuda", generator=g)
    base_W = torch.full((ops.conv_w_len(d),), 0.25, device="cuda") if accumulate else None
    base_b = torch.full((oc,), -0.5, device="cuda") if accumulate else None
    _, dW_ref, db_ref = ops.conv2d_grad_op(ctx, d, x, W, dy, need_dx=False,
                                           dW=None if base_W is None else base_W.clone(),
                                           db=None if base_b is None else base_b.clone(),
                                           accumulate=accumulate)
    dW = base_W.clone() if accumulate else torch.empty(ops.conv_w_len(d), device="cuda")
    db = base_b.clone() if accumulate else torch.empty(oc, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    check(lib.b200_conv2d_dw_noalloc(C.c_void_p(stream), C.byref(d), ptr(x), ptr(dy), ptr(dW), ptr(db),
                                     int(accumulate), batch))
    torch.cuda.synchronize()
    close(dW, dW_ref, GRAD_TOL, f"dW {w}x{w}x{c}->{oc} k{k}")
    close(db, db_ref, GRAD_TOL, f"db {w}x{w}x{c}->{oc} k{k}")
    if not accumulate:
        dW_orc, db_orc = oracle_dw(d, x, W, dy, batch)
        close(dW.cpu(), dW_orc, GRAD_TOL, f"dW {w}x{w}x{c}->{oc} k{k} vs oracle")
        close(db.cpu(), db_orc, GRAD_TOL, f"db {w}x{w}x{c}->{oc} k{k} vs oracle")


def test_noalloc_weight_gradient_matches_regular_entry_point(ctx):
    lib = load()
    # two calls in a row: a 5x5 layer with long partial rows, then a 3x3 layer whose
    # shorter rows overlay what the first call left in the fixed array
    run_pair(ctx, lib, 8, 32, 64, 5, 48, True, False, 1)
    run_pair(ctx, lib, 14, 16, 24, 3, 9, True, True, 2)
    # and the first shape again, accumulating onto existing gradients
    run_pair(ctx, lib, 8, 32, 64, 5, 48, True, True, 3)


def test_noalloc_refuses_what_it_cannot_hold(ctx):
    lib = load()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    z = torch.zeros(16, device="cuda")
    # a partial row of 2048*2048*9 floats is far beyond the 4 Mi-float array
    d = ops.conv_params(8, 8, 2048, 3, 3, 2048, True, True)
    assert lib.b200_conv2d_dw_noalloc(stream, C.byref(d), ptr(z), ptr(z), ptr(z), ptr(z), 0, 1) != 0
    assert b"fixed scratch" in lib.b200_last_error()
    # strided windows are outside what this entry point supports
    d = ops.conv_params(9, 9, 2, 3, 3, 3, False, True, 2, 2)
    assert lib.b200_conv2d_dw_noalloc(stream, C.byref(d), ptr(z), ptr(z), ptr(z), ptr(z), 0, 1) != 0
    assert b"stride 1" in lib.b200_last_error()
