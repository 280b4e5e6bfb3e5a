"""The callers' data formats: raw CIFAR-10 / MNIST bytes scaled and padded into the first layer's
float rows, class labels into target rows.  The oracle restatement is pinned to the reference's
parsers (outputs recorded from parse_cifar10 / parse_mnist_images on synthetic files in the
datasets' own formats); the CUDA kernels must give the same bits, and a fit from the raw bytes
must end with exactly the weights of a fit from the converted floats."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

import oracle_lib as o
from cases import (DATA_CASES, build_net_specs, gen_dataset_bytes, hyper_for, image_desc, xavier_params)

GOLD = Path(__file__).parent / "golden"


@pytest.fixture(scope="module")
def gold():
    return np.load(GOLD / "ref_outputs.npz")


@pytest.mark.parametrize("name", list(DATA_CASES))
def test_oracle_image_scaling_equals_the_reference_parsers(oracle, gold, name):
    c = DATA_CASES[name]
    img, labels = gen_dataset_bytes(c)
    d = image_desc(c)
    want = gold[f"data/{name}/rows"]
    got = o.f32(*want.shape)
    oracle.orc_images_u8_to_float(C.byref(d), o.p(img), c["n"], o.p(got))
    assert got.tobytes() == want.tobytes()


def test_oracle_label_targets_equal_the_reference(oracle, gold):
    labels = np.arange(10, dtype=np.uint8)
    for net in ("lenet", "cifar"):
        lo, hi = gold[f"data/target_range/{net}"]
        got = o.f32(10, 10)
        oracle.orc_labels_to_targets(o.p(labels), 10, 10, float(lo), float(hi), o.p(got))
        assert np.array_equal(got, gold[f"data/targets/{net}"])


@pytest.mark.gpu
@pytest.mark.parametrize("name", list(DATA_CASES))
def test_device_image_scaling_bit_exact(ctx, gold, name):
    import torch
    from tiny_cnn_b200._lib import check, ptr
    c = DATA_CASES[name]
    img, labels = gen_dataset_bytes(c)
    d = image_desc(c)
    want = gold[f"data/{name}/rows"]
    src = torch.from_numpy(img).cuda()
    dst = torch.empty(want.shape, dtype=torch.float32, device="cuda")
    check(ctx.lib.b200_images_u8_to_float(ctx.handle, C.byref(d), ptr(src), c["n"], ptr(dst)))
    ctx.sync()
    assert dst.cpu().numpy().tobytes() == want.tobytes()


@pytest.mark.gpu
def test_device_label_targets_and_bad_descriptors(ctx, gold):
    import torch
    from tiny_cnn_b200._lib import ImageDesc, check, ptr
    labels = torch.arange(10, dtype=torch.uint8, device="cuda")
    dst = torch.empty(10, 10, device="cuda")
    check(ctx.lib.b200_labels_to_targets(ctx.handle, ptr(labels), 10, 10, 0.0, 1.0, ptr(dst)))
    ctx.sync()
    assert np.array_equal(dst.cpu().numpy(), gold["data/targets/cifar"])
    # the parsers' own argument checks (cifar10_parser.h:43-46)
    src = torch.zeros(3072, dtype=torch.uint8, device="cuda")
    out = torch.empty(3072, device="cuda")
    bad_pad = ImageDesc(0, 3, 32, 32, -1, 0, 0.0, 1.0)
    assert ctx.lib.b200_images_u8_to_float(ctx.handle, C.byref(bad_pad), ptr(src), 1, ptr(out)) != 0
    assert b"padding" in ctx.lib.b200_last_error()
    bad_scale = ImageDesc(0, 3, 32, 32, 0, 0, 1.0, 1.0)
    assert ctx.lib.b200_images_u8_to_float(ctx.handle, C.byref(bad_scale), ptr(src), 1, ptr(out)) != 0
    assert b"scale_max" in ctx.lib.b200_last_error()
    empty = ImageDesc(0, 3, 32, 32, 0, 0, 0.0, 1.0)
    check(ctx.lib.b200_images_u8_to_float(ctx.handle, C.byref(empty), None, 0, None))  # no images: nothing to do


@pytest.mark.gpu
def test_fit_from_raw_bytes_equals_fit_from_parsed_floats(ctx, oracle):
    """b200_net_fit_u8_host (uint8 upload, device scaling, labels to targets) against
    b200_net_fit_host on the oracle's float rows: identical weights and outputs; ragged last batch."""
    import torch
    from test_net_gpu import DeviceNet
    from tiny_cnn_b200._lib import ImageDesc, check, ptr
    specs, keep = build_net_specs("cifar")
    B, n = 8, 28
    rng = np.random.default_rng(91)
    img = rng.integers(0, 256, (n, 3072), dtype=np.uint8)
    labels = rng.integers(0, 10, n, dtype=np.uint8)
    d = ImageDesc(0, 3, 32, 32, 0, 0, -1.0, 1.0)
    x = o.f32(n, 3072)
    oracle.orc_images_u8_to_float(C.byref(d), o.p(img), n, o.p(x))
    t = o.f32(n, 10)
    oracle.orc_labels_to_targets(o.p(labels), n, 10, 0.0, 1.0, o.p(t))
    p0 = xavier_params(specs, 12)
    h = hyper_for(1)
    a, b = DeviceNet(ctx, specs, B), DeviceNet(ctx, specs, B)
    a.set_params(p0)
    b.set_params(p0)
    outs_a, outs_b = np.zeros((n, 10), np.float32), np.zeros((n, 10), np.float32)
    ip, lp = torch.from_numpy(img).pin_memory(), torch.from_numpy(labels).pin_memory()
    check(a.lib.b200_net_fit_u8_host(a.h, C.byref(d), ptr(ip), ptr(lp), n, B, 2, 0.0, 1.0, 1, 1, C.byref(h),
                                     ptr(outs_a)))
    check(b.lib.b200_net_fit_host(b.h, ptr(x), ptr(t), n, B, 2, 1, 1, C.byref(h), ptr(outs_b)))  # same ragged rule
    assert np.array_equal(a.params(), b.params())
    assert np.array_equal(outs_a, outs_b)
    # a label beyond the network's outputs is refused before anything runs
    labels_bad = labels.copy()
    labels_bad[3] = 10
    assert a.lib.b200_net_fit_u8_host(a.h, C.byref(d), ptr(ip), ptr(labels_bad), n, B, 1, 0.0, 1.0, 1, 1, C.byref(h),
                                      None) != 0
    # and an image size the network does not read
    d_pad = ImageDesc(0, 3, 32, 32, 2, 2, -1.0, 1.0)
    assert a.lib.b200_net_fit_u8_host(a.h, C.byref(d_pad), ptr(ip), ptr(lp), n, B, 1, 0.0, 1.0, 1, 1, C.byref(h),
                                      None) != 0
    a.close()
    b.close()
