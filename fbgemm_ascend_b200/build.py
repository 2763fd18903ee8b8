"""In-tree build of the two shared libraries of this package (sm_100a only).

``lib/libtbe_b200.so``      CUDA kernels + the C ABI of ``include/tbe_b200.h``; no torch in it.
``lib/libtbe_b200_torch.so``  the ``torch.ops.fbgemm.*`` registrations, calling the C ABI.

One architecture, one ``nvcc`` invocation per source file: this replaces the
reference's chip detection and per-SoC operator packages
(FbgemmAscend.cmake:5-183, fbgemm_ascend/__init__.py:55-231).

Run ``python -m fbgemm_ascend_b200.build`` or call :func:`build`.
"""
from __future__ import annotations

import importlib.util
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG_DIR)
CSRC = os.path.join(PKG_DIR, "csrc")
LIB_DIR = os.path.join(PKG_DIR, "lib")
OBJ_DIR = os.path.join(PKG_DIR, "build")
INCLUDE = os.path.join(ROOT, "include")

CABI_LIB = os.path.join(LIB_DIR, "libtbe_b200.so")
TORCH_LIB = os.path.join(LIB_DIR, "libtbe_b200_torch.so")

CUDA_SOURCES = ["tbe_common.cu", "tbe_lookup.cu", "tbe_quant.cu", "tbe_permute.cu", "tbe_sparse.cu", "tbe_exchange.cu"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-I" + INCLUDE]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; this package builds only with the CUDA toolkit")


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n" + " ".join(cmd) + "\n" + r.stdout)
    return r.stdout


def build_cabi(force: bool = False, verbose: bool = False, extra_flags=()) -> str:
    os.makedirs(LIB_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, "tbe_common.cuh"), os.path.join(INCLUDE, "tbe_b200.h")]
    nvcc = _nvcc()
    jobs, objs = [], []
    for src in CUDA_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _newer(o, [s] + headers):
            jobs.append([nvcc] + NVCC_FLAGS + list(extra_flags) + ["-c", s, "-o", o])
    with ThreadPoolExecutor(max_workers=4) as ex:
        list(ex.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _newer(CABI_LIB, objs):
        _run([nvcc, "-shared", "-o", CABI_LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"], verbose)
    return CABI_LIB


def build_torch(force: bool = False, verbose: bool = False) -> str:
    src = os.path.join(CSRC, "torch_ops.cpp")
    if not (force or _newer(TORCH_LIB, [src, os.path.join(INCLUDE, "tbe_b200.h"), CABI_LIB])):
        return TORCH_LIB
    torch_dir = os.path.dirname(importlib.util.find_spec("torch").origin)
    cuda_home = os.path.dirname(os.path.dirname(_nvcc()))
    cxx = shutil.which("g++") or "g++"
    cmd = [cxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=1",
           "-I" + INCLUDE, "-I" + os.path.join(torch_dir, "include"),
           "-I" + os.path.join(torch_dir, "include", "torch", "csrc", "api", "include"),
           "-I" + os.path.join(cuda_home, "include"),
           src, "-o", TORCH_LIB,
           "-L" + LIB_DIR, "-ltbe_b200", "-L" + os.path.join(torch_dir, "lib"),
           "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(torch_dir, "lib")]
    _run(cmd, verbose)
    return TORCH_LIB


def build(force: bool = False, verbose: bool = False) -> None:
    build_cabi(force, verbose)
    build_torch(force, verbose)


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print("built", CABI_LIB, TORCH_LIB)
