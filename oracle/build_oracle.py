"""Build recipe of the test oracle.

`build_oracle()`      gcc  oracle/oracle.c      -> oracle/liboracle.so
                      (plain C restatement; -ffp-contract=off so the compiler
                      never fuses a multiply with an add)
`build_reference()`   g++  oracle/ref_shim.cpp + oracle/ref_qfc.cpp against the
                      reference's own headers -> oracle/_ref/libtinydnn_ref.so
                      (only where the reference tree is present; flags follow
                      the reference's OpenMP configuration: -O3 -fopenmp
                      -DCNN_USE_OMP, default serialization, no AVX macros, so
                      every kernel runs as backend_t::internal)
                      and, from the same ref_shim.cpp with -DCNN_USE_SSE
                      -DCNN_USE_AVX -mavx -DREF_ENGINE=core::backend_t::avx,
                      oracle/_ref/libtinydnn_ref_avx.so: the reference's AVX
                      kernels (5x5 convolutions, fully connected), only ever
                      timed as an informational CPU column, never a parity target

Outputs are git-ignored build products; no reference source is copied.
"""
from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
# the reference tree: beside this repository unless TINYDNN_REFERENCE says otherwise
REF_ROOT = Path(os.environ.get("TINYDNN_REFERENCE", str(ROOT.parent / "reference")))
ORACLE_SO = HERE / "liboracle.so"
REF_DIR = HERE / "_ref"
REF_SO = REF_DIR / "libtinydnn_ref.so"
REF_AVX_SO = REF_DIR / "libtinydnn_ref_avx.so"


def _run(cmd):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(map(str, cmd)) + "\n" + res.stdout + res.stderr)


def _stale(target: Path, sources) -> bool:
    if not target.exists():
        return True
    t = target.stat().st_mtime
    return any(Path(s).stat().st_mtime > t for s in sources)


def build_oracle(force: bool = False) -> Path:
    srcs = [HERE / "oracle.c", ROOT / "include" / "tinycnn_b200.h"]
    if force or _stale(ORACLE_SO, srcs):
        _run(["gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-fvisibility=hidden",
              f"-I{ROOT / 'include'}", "-o", str(ORACLE_SO), str(HERE / "oracle.c"), "-lm"])
    return ORACLE_SO


def reference_available() -> bool:
    return (REF_ROOT / "tiny_dnn" / "tiny_dnn.h").exists()


def build_reference(force: bool = False) -> Path | None:
    """Compile the unmodified reference behind the C doors; None if it is absent."""
    if not reference_available():
        return REF_SO if REF_SO.exists() else None
    REF_DIR.mkdir(exist_ok=True)
    srcs = [HERE / "ref_shim.cpp", HERE / "ref_qfc.cpp", ROOT / "include" / "tinycnn_b200.h",
            HERE / "ref_stub" / "tiny_dnn" / "core" / "kernels" / "tiny_quantized_matmul_kernel.h"]
    if not (force or _stale(REF_SO, srcs) or _stale(REF_AVX_SO, srcs)):
        return REF_SO
    common = ["g++", "-std=c++14", "-O3", "-fopenmp", "-DCNN_USE_OMP", "-ffp-contract=off", "-fPIC",
              "-fvisibility=hidden", "-w", f"-I{ROOT / 'include'}"]
    o1 = REF_DIR / "ref_shim.o"
    o2 = REF_DIR / "ref_qfc.o"
    p1 = subprocess.Popen(common + [f"-I{REF_ROOT}", "-c", str(HERE / "ref_shim.cpp"), "-o", str(o1)],
                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    p2 = subprocess.Popen(common + [f"-I{HERE / 'ref_stub'}", f"-I{REF_ROOT}", "-c",
                                    str(HERE / "ref_qfc.cpp"), "-o", str(o2)],
                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    o3 = REF_DIR / "ref_shim_avx.o"
    p3 = subprocess.Popen(common + ["-DCNN_USE_SSE", "-DCNN_USE_AVX", "-mavx",
                                    "-DREF_ENGINE=core::backend_t::avx", f"-I{REF_ROOT}", "-c",
                                    str(HERE / "ref_shim.cpp"), "-o", str(o3)],
                          stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    out1, _ = p1.communicate()
    out2, _ = p2.communicate()
    out3, _ = p3.communicate()
    if p1.returncode or p2.returncode or p3.returncode:
        raise RuntimeError("reference build failed:\n" + out1 + out2 + out3)
    _run(["g++", "-shared", "-fopenmp", "-o", str(REF_SO), str(o1), str(o2)])
    _run(["g++", "-shared", "-fopenmp", "-o", str(REF_AVX_SO), str(o3)])
    return REF_SO


OVERLAY_DIR = REF_DIR / "overlay"
BACKEND_TEST = REF_DIR / "bin" / "test_backend_b200"
FIT_BENCH = REF_DIR / "bin" / "bench_fit_b200"
DP_TEST = REF_DIR / "bin" / "test_dp_b200"


def build_backend_test(force: bool = False) -> Path | None:
    """Generate the backend_t::b200 overlay from the reference tree and compile the
    C++ A/B test (tests/cpp/test_backend_b200.cpp) against it; None if the reference
    is absent.  The binary links tiny_cnn_b200/csrc/libtinycnn_b200.so by relative rpath."""
    if not reference_available():
        return BACKEND_TEST if BACKEND_TEST.exists() else None
    import sys as _sys
    _sys.path.insert(0, str(ROOT))
    from tiny_cnn_b200.host.make_overlay import make_overlay
    src = ROOT / "tests" / "cpp" / "test_backend_b200.cpp"
    dp_src = ROOT / "tests" / "cpp" / "test_dp_b200.cpp"  # data-parallel fit, one process per GPU
    host = ROOT / "tiny_cnn_b200" / "host"
    bench_src = host / "bench_fit.cpp"
    deps = [src, dp_src, bench_src, host / "b200_glue.h", host / "b200_backend.h", host / "b200_net.h",
            host / "make_overlay.py", ROOT / "include" / "tinycnn_b200.h"]
    if not (force or _stale(BACKEND_TEST, deps) or _stale(FIT_BENCH, deps) or _stale(DP_TEST, deps)):
        return BACKEND_TEST
    make_overlay(REF_ROOT, OVERLAY_DIR)
    BACKEND_TEST.parent.mkdir(parents=True, exist_ok=True)
    libdir = ROOT / "tiny_cnn_b200" / "csrc"
    procs = []
    for s, out in ((src, BACKEND_TEST), (bench_src, FIT_BENCH), (dp_src, DP_TEST)):  # the A/B test, and the timed fit bench.py runs
        procs.append(subprocess.Popen(
            ["g++", "-std=c++14", "-O2", "-fopenmp", "-DCNN_USE_OMP", "-w", f"-I{OVERLAY_DIR}", f"-I{REF_ROOT}",
             f"-I{ROOT / 'include'}", str(s), "-o", str(out), f"-L{libdir}", "-ltinycnn_b200",
             "-Wl,-rpath,$ORIGIN/../../../tiny_cnn_b200/csrc", "-ldl", "-lpthread", "-lrt"],
            stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    logs = [p.communicate()[0] for p in procs]
    if any(p.returncode for p in procs):
        raise RuntimeError("backend test build failed:\n" + "".join(logs))
    return BACKEND_TEST


if __name__ == "__main__":
    print(build_oracle(force="-f" in sys.argv))
    print(build_reference(force="-f" in sys.argv))
    print(build_backend_test(force="-f" in sys.argv))
