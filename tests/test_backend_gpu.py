"""Runs the C++ A/B test of the engine core::backend_t::b200 inside tiny-dnn.

oracle/_ref/bin/test_backend_b200 is tests/cpp/test_backend_b200.cpp compiled
(oracle/build_oracle.py, where the reference tree is present) against the
overlay of tiny_cnn_b200/host/make_overlay.py and linked with the native
library: stock tiny-dnn layer classes and a network<sequential> run with
backend_t::internal and with backend_t::b200 and are compared."""
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "oracle" / "_ref" / "bin" / "test_backend_b200"
DP_BIN = ROOT / "oracle" / "_ref" / "bin" / "test_dp_b200"


@pytest.mark.gpu
def test_backend_b200_inside_tiny_dnn():
    if not BIN.exists():
        pytest.skip("the C++ A/B binary has not been built (reference tree absent at build time)")
    res = subprocess.run([str(BIN)], capture_output=True, text=True, timeout=600)
    print(res.stdout)
    print(res.stderr)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-2000:]
    assert "RESULT: all passed" in res.stdout


@pytest.mark.gpu
def test_data_parallel_fit_from_cpp_on_two_gpus():
    """tests/cpp/test_dp_b200.cpp: two processes, one GPU each, network<sequential>::fit on backend_t::b200 with
    the gradients summed over the processes (buffer handles exchanged over pipes, no framework)."""
    import torch
    if not DP_BIN.exists():
        pytest.skip("the C++ data-parallel binary has not been built (reference tree absent at build time)")
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    res = subprocess.run([str(DP_BIN), "2"], capture_output=True, text=True, timeout=600)
    print(res.stdout)
    print(res.stderr)
    assert res.returncode == 0, res.stdout[-4000:] + res.stderr[-2000:]
    assert "RESULT: all passed" in res.stdout


def test_overlay_patches_fit_the_reference(tmp_path):
    """Where the reference tree is present, every anchored edit of the overlay applies."""
    import os
    ref = Path(os.environ.get("TINYDNN_REFERENCE", str(ROOT.parent / "reference")))
    if not (ref / "tiny_dnn" / "tiny_dnn.h").exists():
        pytest.skip("reference tree not present")
    from tiny_cnn_b200.host.make_overlay import PATCHES, make_overlay
    out = make_overlay(ref, tmp_path / "overlay")
    for rel in PATCHES:
        assert "b200" in (out / rel).read_text()
    assert (out / "tiny_dnn/core/kernels/b200_glue.h").exists()
    assert (out / "tiny_dnn/core/b200_backend.h").exists()
