"""CPU checks of the C ABI boundary: the library builds, loads, exports every
symbol include/tinycnn_b200.h declares, fills descriptors like the reference,
and refuses to compute without a GPU (there is no CPU path)."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

from tiny_cnn_b200 import _lib as L

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "tinycnn_b200.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    decl = declared_symbols()
    assert len(decl) > 60
    assert sorted(L.SIGNATURES) == decl


def test_library_exports_every_declared_symbol():
    lib = L.load()  # raises if the .so is missing or lacks a typed symbol
    for name in declared_symbols():
        assert hasattr(lib, name), name
    out = subprocess.run(["nm", "-D", "--defined-only", str(L.LIB_PATH)], capture_output=True, text=True)
    exported = set(re.findall(r" T (b200_[a-z0-9_]+)", out.stdout))
    assert exported == set(declared_symbols())
    assert lib.b200_version() == b"0.1"


def test_conv_descriptor_matches_reference_shape_rules():
    lib = L.load()
    d = L.ConvDesc()
    # same padding: in_padded = in + k - 1, out = ceil(in / stride) (convolutional_layer.h:404-438)
    assert lib.b200_conv_desc_init(C.byref(d), 32, 32, 3, 5, 5, 32, 1, 1, 1, 1, 1, 1) == 0
    assert (d.inp_w, d.inp_h, d.out_w, d.out_h) == (36, 36, 32, 32)
    assert lib.b200_conv_desc_init(C.byref(d), 9, 8, 2, 3, 3, 3, 1, 1, 2, 2, 1, 1) == 0
    assert (d.inp_w, d.inp_h, d.out_w, d.out_h) == (11, 10, 5, 4)
    # valid with dilation: out = in - dil*k + dil (util.h:329-344)
    assert lib.b200_conv_desc_init(C.byref(d), 7, 7, 1, 3, 3, 1, 0, 1, 1, 1, 2, 2) == 0
    assert (d.inp_w, d.out_w, d.out_h) == (7, 3, 3)
    assert lib.b200_conv_desc_init(C.byref(d), 28, 28, 32, 5, 5, 64, 0, 1, 2, 2, 1, 1) == 0
    assert d.out_w * d.out_h * d.out_c == 9216
    assert lib.b200_conv_desc_init(C.byref(d), 2, 2, 1, 5, 5, 1, 0, 1, 1, 1, 1, 1) != 0
    assert b"empty" in lib.b200_last_error()


def test_pool_descriptor_matches_reference_shape_rules():
    lib = L.load()
    d = L.PoolDesc()
    assert lib.b200_pool_desc_init(C.byref(d), 4, 4, 1, 2, 2, 1, 1, 0, 1) == 0  # same, stride 1
    assert (d.out_w, d.out_h) == (4, 4)
    assert lib.b200_pool_desc_init(C.byref(d), 4, 4, 1, 2, 2, 1, 1, 0, 0) == 0  # valid, stride 1
    assert (d.out_w, d.out_h) == (3, 3)
    assert lib.b200_pool_desc_init(C.byref(d), 7, 7, 1, 2, 2, 2, 2, 1, 0) == 0  # ceil mode
    assert (d.out_w, d.out_h) == (4, 4)
    assert lib.b200_pool_desc_init(C.byref(d), 7, 7, 1, 2, 2, 2, 2, 0, 0) == 0
    assert (d.out_w, d.out_h) == (3, 3)


def test_python_descriptor_restatement_equals_the_library():
    """tests/cases.py restates the descriptor arithmetic so that fixtures and CPU baselines need no
    CUDA library; it must agree with b200_conv_desc_init / b200_pool_desc_init field for field."""
    import cases
    lib = L.load()
    skip = {"tbl", "algo", "input_is_padded"}
    for c in list(cases.CONV_CASES.values()) + list(cases.QCONV_CASES.values()):
        d = L.ConvDesc()
        assert lib.b200_conv_desc_init(C.byref(d), c["w"], c["h"], c["c"], c["kw"], c["kh"], c["oc"],
                                       int(c["same"]), int(c["bias"]), c.get("sw", 1), c.get("sh", 1),
                                       c.get("dw", 1), c.get("dh", 1)) == 0
        p = cases.conv_desc(c)
        for name, _ in L.ConvDesc._fields_:
            if name not in skip:
                assert getattr(d, name) == getattr(p, name), (c, name)
    for c in list(cases.MAXPOOL_CASES.values()) + list(cases.AVGPOOL_CASES.values()):
        d = L.PoolDesc()
        assert lib.b200_pool_desc_init(C.byref(d), c["w"], c["h"], c["c"], c["pw"], c["ph"], c["sw"], c["sh"],
                                       int(c.get("ceil", 0)), int(c.get("same", 0))) == 0
        p = cases.pool_desc(c)
        for name, _ in L.PoolDesc._fields_:
            assert getattr(d, name) == getattr(p, name), (c, name)


def test_no_cpu_fallback():
    """Without a GPU the context cannot be created and says why."""
    lib = L.load()
    if lib.b200_device_count() > 0:
        pytest.skip("a GPU is present")
    h = C.c_void_p()
    assert lib.b200_ctx_create(0, None, C.byref(h)) != 0
    assert b"no CPU path" in lib.b200_last_error()
    from tiny_cnn_b200.ops import Context
    with pytest.raises(L.B200Error):
        Context(0)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setenv("TINYCNN_B200_LIB", str(tmp_path / "absent.so"))
    monkeypatch.setattr(L, "_lib", None)
    with pytest.raises(L.B200Error, match="no CPU fallback"):
        L.load()
    monkeypatch.setattr(L, "_lib", None)


def test_product_never_touches_the_oracle():
    """The package and the native sources must not import, link or name the oracle."""
    for path in list((ROOT / "tiny_cnn_b200").rglob("*.py")) + list((ROOT / "tiny_cnn_b200").rglob("*.cu")) + \
            list((ROOT / "tiny_cnn_b200").rglob("*.cuh")) + [HEADER]:
        text = path.read_text()
        assert "oracle" not in text.lower(), path
        assert "liboracle" not in text and "orc_" not in text, path
