"""Build recipe of the native library (nvcc, sm_100a only).

`build_native()` compiles every `csrc/*.cu` to an object file and links
`csrc/libtinycnn_b200.so` in-tree.  nvcc cross-compiles, so this works on a
machine without a GPU.  Object files are rebuilt only when a source or header
is newer than them.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
INCLUDE = PKG_DIR.parent / "include"
LIB_PATH = CSRC / "libtinycnn_b200.so"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = [
    "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
    f"-I{INCLUDE}", f"-I{CSRC}",
]
# files whose float arithmetic must not be contracted into fused multiply-adds
NO_FMAD = {"quant.cu"}


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; the native library cannot be built")
    return exe


def _newest_header() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in hs)


# Role-timing diagnostics of the tensor-core kernels (cycle counters per warp role, printed when
# the environment variable B200_TC_TIMING is set) exist only in a library built with
# `python -m tiny_cnn_b200.build --tc-timing`, which goes to csrc/libtinycnn_b200_timing.so; load it
# with TINYCNN_B200_LIB.  The default library carries none of it.
TIMING_LIB_PATH = CSRC / "libtinycnn_b200_timing.so"


def _compile(src: Path, verbose: bool, ptxas_info: bool, tc_timing: bool = False) -> Path:
    obj = src.with_suffix(".timing.o" if tc_timing else ".o")
    newest = max(src.stat().st_mtime, _newest_header(), Path(__file__).stat().st_mtime)
    if obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    cmd = [_nvcc(), *ARCH_FLAGS, *COMMON_FLAGS, "-c", str(src), "-o", str(obj)]
    if src.name in NO_FMAD:
        cmd.append("-fmad=false")
    if tc_timing:
        cmd.append("-DB200_TC_TIMING")
    if ptxas_info:
        cmd += ["-Xptxas", "-v"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    if ptxas_info or verbose:
        sys.stderr.write(res.stderr)
    return obj


def build_native(verbose: bool = False, force: bool = False, ptxas_info: bool = False,
                 tc_timing: bool = False) -> Path:
    """Compile and link the CUDA library; returns the path of the .so."""
    lib_path = TIMING_LIB_PATH if tc_timing else LIB_PATH
    srcs = sorted(CSRC.glob("*.cu"))
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    if force:
        for s in srcs:
            o = s.with_suffix(".timing.o" if tc_timing else ".o")
            if o.exists():
                o.unlink()
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose, ptxas_info, tc_timing), srcs))
    newest_obj = max(o.stat().st_mtime for o in objs)
    if lib_path.exists() and lib_path.stat().st_mtime >= newest_obj and not force:
        return lib_path
    cmd = [_nvcc(), *ARCH_FLAGS, "-shared", "-o", str(lib_path), *map(str, objs),
           "-Xcompiler", "-fPIC", "-cudart", "static"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return lib_path


if __name__ == "__main__":
    p = build_native(verbose="-v" in sys.argv, force="-f" in sys.argv,
                     ptxas_info="--ptxas" in sys.argv, tc_timing="--tc-timing" in sys.argv)
    print(p)
