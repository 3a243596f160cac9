"""In-tree build of the native library and the CPython extension (nvcc, sm_100a only).

    python -m flashlstm_poc_b200._build            # build if sources changed
    python -m flashlstm_poc_b200._build --force

Outputs, next to this file:
    libflashlstm_b200.so                      the C-ABI library (include/*.h)
    _flashlstm.<abi>.so                       CPython extension with the reference's two entry points
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIB = os.path.join(PKG, "libflashlstm_b200.so")
EXT = os.path.join(PKG, "_flashlstm" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))
STAMP = os.path.join(OBJ, "stamp.txt")

CU_SOURCES = [
    "engine.cu", "simt_kernels.cu", "simt_persistent.cu", "tc_engine.cu", "tc_gemm.cu", "tc_lstm_fwd.cu", "tc_lstm_bwd.cu", "tc_lstm_step.cu", "comm.cu", "static_scratch.cu", "api_v1.cu", "api_v2.cu",
]

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; set NVCC or install the CUDA toolkit")


def _cuda_home() -> str:
    return os.path.dirname(os.path.dirname(os.path.realpath(_nvcc())))


def _fingerprint() -> str:
    h = hashlib.sha256()
    paths = []
    for d in (CSRC, os.path.join(ROOT, "include")):
        for base, _, files in os.walk(d):
            paths += [os.path.join(base, f) for f in files]
    for p in sorted(paths) + [os.path.abspath(__file__)]:
        h.update(os.path.relpath(p, ROOT).encode())  # the tree may sit elsewhere on another machine
        with open(p, "rb") as f:
            h.update(f.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current() -> bool:
    if not (os.path.exists(LIB) and os.path.exists(EXT) and os.path.exists(STAMP)):
        return False
    with open(STAMP) as f:
        return f.read().strip() == _fingerprint()


def _run(cmd):
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build step failed:\n  " + " ".join(cmd) + "\n" + proc.stdout)
    return proc.stdout


def build(force: bool = False, verbose: bool = False) -> str:
    if not force and is_current():
        return LIB
    os.makedirs(OBJ, exist_ok=True)
    nvcc = _nvcc()
    inc = ["-I", os.path.join(ROOT, "include"), "-I", CSRC]
    extra = ["-Xptxas", "-v"] if verbose else []

    def compile_one(src):
        obj = os.path.join(OBJ, src.replace(".cu", ".o"))
        out = _run([nvcc, *NVCC_FLAGS, *extra, *inc, "-c", os.path.join(CSRC, src), "-o", obj])
        return obj, out

    with ThreadPoolExecutor(max_workers=min(8, len(CU_SOURCES))) as pool:
        results = list(pool.map(compile_one, CU_SOURCES))
    if verbose:
        for _, out in results:
            sys.stdout.write(out)
    objs = [o for o, _ in results]
    _run([nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-ldl",
          "-Xlinker", "--no-undefined"])
    py_inc = sysconfig.get_paths()["include"]
    _run(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", os.path.join(CSRC, "pyext.cpp"), "-o", EXT,
          "-I", py_inc, "-I", os.path.join(ROOT, "include"), "-I", os.path.join(_cuda_home(), "include"),
          "-L", PKG, "-lflashlstm_b200", "-Wl,-rpath,$ORIGIN"])
    with open(STAMP, "w") as f:
        f.write(_fingerprint())
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
