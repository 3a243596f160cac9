"""Builds the UNMODIFIED reference (mikex86/flashlstm_poc) for sm_100 as an on-GPU comparison arm.

    python -m baseline.build_reference [--reference /path/to/flashlstm_poc]

Nothing of the reference is copied or patched: its own source files are compiled where they lie, with
compiler flags only, into two shared libraries under baseline/_ref/ (git-ignored):

    libflashlstm_v1.so   src/lstm.cu + src/kernels.cu                    (C ABI of include/flashlstm/lstm_api.h)
    libflashlstm_v2.so   flashlstm_v2/src/{lstm_forward,lstm_backward,gemm}.cu  (C ABI of flashlstm_v2/include/lstm.hpp)

What the reference's CMake files would need and how each is met here:
  * CUTLASS headers (un-vendored: an empty submodule in v2, a network fetch in v1, scripts/ensure_cutlass.py):
    the header tree that ships inside this image's flashinfer wheel (CUTLASS 4.x keeps the 2.x device::Gemm API
    the reference instantiates);
  * NVTX (hard requirement of CMakeLists.txt:25-90): compiled out with the reference's own switches
    NVTX_DISABLE (src/nvtx_profinst.h:3) and GPUTX_DISABLE_NVTX (flashlstm_v2/src/gputx.h:3);
  * cuDNN / cuBLAS: only the benchmark executables link them, the two libraries do not;
  * architecture: sm_100 instead of sm_89 (CMakeLists.txt:10); FLASHLSTM_CUDA_ARCH=100 as
    flashlstm_v2/CMakeLists.txt:21-22 would define it.
The product never links or imports these libraries; baseline/reference_gpu.py loads them for comparison runs.
"""
from __future__ import annotations

import argparse
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
V1_LIB = os.path.join(OUT, "libflashlstm_v1.so")
V2_LIB = os.path.join(OUT, "libflashlstm_v2.so")


def find_cutlass() -> str:
    """A CUTLASS include directory: $CUTLASS_INCLUDE, else the copy inside an installed Python package."""
    cand = [os.environ.get("CUTLASS_INCLUDE")]
    for sp in sys.path:
        cand += glob.glob(os.path.join(sp, "flashinfer", "data", "cutlass", "include"))
        cand += glob.glob(os.path.join(sp, "tilelang", "3rdparty", "cutlass", "include"))
    for c in cand:
        if c and os.path.exists(os.path.join(c, "cutlass", "gemm", "device", "gemm.h")):
            return c
    raise RuntimeError("no CUTLASS header tree found (set CUTLASS_INCLUDE)")


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def build(reference: str = "/root/reference", force: bool = False) -> dict:
    """Returns {"v1": path-or-error, "v2": path-or-error}."""
    os.makedirs(OUT, exist_ok=True)
    cutlass = find_cutlass()
    common = [_nvcc(), "-std=c++17", "-O3", "-gencode", "arch=compute_100,code=sm_100", "--expt-relaxed-constexpr",
              "-shared", "-Xcompiler", "-fPIC", "-I", cutlass]
    jobs = {
        "v1": (V1_LIB, ["-DNVTX_DISABLE", "-I", os.path.join(reference, "include"), "-I", os.path.join(reference, "src"),
                        os.path.join(reference, "src", "lstm.cu"), os.path.join(reference, "src", "kernels.cu")]),
        "v2": (V2_LIB, ["-DGPUTX_DISABLE_NVTX", "-DFLASHLSTM_CUDA_ARCH=100",
                        "-I", os.path.join(reference, "flashlstm_v2", "include"), "-I", os.path.join(reference, "flashlstm_v2", "src"),
                        *[os.path.join(reference, "flashlstm_v2", "src", f) for f in ("lstm_forward.cu", "lstm_backward.cu", "gemm.cu")]]),
    }
    result = {}
    for name, (lib, args) in jobs.items():
        if os.path.exists(lib) and not force:
            result[name] = lib
            continue
        proc = subprocess.run(common + args + ["-o", lib], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
        result[name] = lib if proc.returncode == 0 else "build failed:\n" + proc.stdout[-2000:]
    return result


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    for k, v in build(a.reference, a.force).items():
        print(k, v)
