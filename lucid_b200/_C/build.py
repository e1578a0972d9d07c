"""Builds liblucid_cuda.so (sm_100a) next to this file with nvcc, and the small CPython module
``_fastcall`` (gcc) that binds a few of its entry points without ctypes' per-call cost.

    python -m lucid_b200._C.build [--force]

nvcc cross-compiles without a GPU.  The shared object is kept in-tree so that it
travels with the source tree; it is not installed into site-packages.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(ROOT, "include")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "liblucid_cuda.so")
FASTCALL_SRC = os.path.join(CSRC, "fastcall.c")
FASTCALL_PATH = os.path.join(HERE, "_fastcall" + (sysconfig.get_config_var("EXT_SUFFIX") or ".so"))

SOURCES = ["api.cu", "quant_kernels.cu", "hist_kernels.cu", "embed_kernels.cu", "qlinear_tcgen05.cu", "wo_kernels.cu",
           "wo_prep_kernels.cu", "peer_kernels.cu", "qgemv_kernels.cu"]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-I", INCLUDE, "-I", CSRC,
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found; liblucid_cuda.so cannot be built")
    return exe


def _newer(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every .cu and link the shared library; returns its path."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    headers.append(os.path.join(INCLUDE, "lucid_cuda.h"))
    nvcc = _nvcc()
    objs, jobs = [], []
    for src in SOURCES:
        src_path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
        objs.append(obj)
        if force or not _newer(obj, [src_path] + headers):
            jobs.append([nvcc, *NVCC_FLAGS, "-c", src_path, "-o", obj])

    def run(cmd: list[str]) -> None:
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compiler failed:\n{' '.join(cmd)}\n{r.stdout}\n{r.stderr}")

    with ThreadPoolExecutor(max_workers=4) as pool:
        list(pool.map(run, jobs))
    if force or jobs or not _newer(LIB_PATH, objs):
        run([nvcc, "-shared", "-o", LIB_PATH, *objs, "-gencode", "arch=compute_100a,code=sm_100a"])
    if force or not _newer(FASTCALL_PATH, [FASTCALL_SRC, os.path.join(INCLUDE, "lucid_cuda.h")]):
        cc = shutil.which("gcc") or shutil.which("cc")
        if cc is None:
            raise RuntimeError("gcc not found; the _fastcall module cannot be built")
        run([cc, "-O2", "-shared", "-fPIC", "-Wall", "-I", sysconfig.get_paths()["include"], "-I", INCLUDE,
             FASTCALL_SRC, "-o", FASTCALL_PATH])
    return LIB_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
