"""Build the in-tree native library ``chocosgd_b200/lib/libchoco_b200.so``.

All CUDA sources are compiled for sm_100a only
(``nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo``); nvcc cross-compiles without
a GPU.  The kernels expose a plain C ABI (raw pointers + ``cudaStream_t``) and are bound
with ctypes (``ops/_lib.py``), so no PyTorch header is compiled and a full rebuild takes
seconds.  Usage: ``python -m chocosgd_b200.build_ext [--force] [--verbose]``."""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "lib")
OBJ_DIR = os.path.join(OUT_DIR, "obj")
LIB = os.path.join(OUT_DIR, "libchoco_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--use_fast_math" if False else "-DCHOCO_NO_FAST_MATH", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-fopenmp"]


def nvcc_path():
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    return None


def sources():
    cu = sorted(f for f in os.listdir(SRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(SRC) if f.endswith(".cpp"))
    return cu, cpp


def _digest():
    h = hashlib.sha256()
    for f in sorted(os.listdir(SRC)):
        if f.endswith((".cu", ".cuh", ".cpp", ".h")):
            with open(os.path.join(SRC, f), "rb") as fh:
                h.update(f.encode())
                h.update(fh.read())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def is_current():
    stamp = os.path.join(OUT_DIR, "build.stamp")
    return os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read().strip() == _digest()


def build(force=False, verbose=False):
    """Compile every source for sm_100a and link the shared library.  Returns its path."""
    if not force and is_current():
        return LIB
    nvcc = nvcc_path()
    if nvcc is None:
        if os.path.exists(LIB):
            return LIB
        raise RuntimeError("nvcc not found and no prebuilt library present")
    os.makedirs(OBJ_DIR, exist_ok=True)
    cu, cpp = sources()
    log = {}

    def compile_one(f):
        obj = os.path.join(OBJ_DIR, f + ".o")
        if f.endswith(".cu"):
            cmd = [nvcc] + NVCC_FLAGS + ["-I", SRC, "-c", os.path.join(SRC, f), "-o", obj]
        else:
            cmd = [nvcc, "-x", "c++", "-std=c++17", "-O3", "-Xcompiler", "-fPIC,-fopenmp", "-I", SRC, "-c",
                   os.path.join(SRC, f), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        log[f] = r.stderr + r.stdout
        if r.returncode != 0:
            raise RuntimeError(f"compiling {f} failed:\n{r.stderr}\n{r.stdout}")
        return obj

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as ex:
        objs = list(ex.map(compile_one, cu + cpp))
    link = [nvcc, "-shared", "-o", LIB] + objs + ["-Xcompiler", "-fopenmp", "-lgomp"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("link failed:\n" + r.stderr + r.stdout)
    with open(os.path.join(OUT_DIR, "build.stamp"), "w") as fh:
        fh.write(_digest())
    with open(os.path.join(OUT_DIR, "ptxas.log"), "w") as fh:
        for f in cu:
            fh.write(f"==== {f}\n{log.get(f, '')}\n")
    if verbose:
        print(open(os.path.join(OUT_DIR, "ptxas.log")).read())
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="--verbose" in sys.argv)
    print(path)
