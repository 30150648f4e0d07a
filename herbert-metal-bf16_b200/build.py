"""Builds libhb200.so (CUDA kernels + C ABI + host selection library) in-tree for sm_100a.

    python herbert-metal-bf16_b200/build.py [--force]

nvcc cross-compiles without a GPU. Objects go to build/ (ignored), the library to
herbert-metal-bf16_b200/lib/libhb200.so.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
LIB_DIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIB_DIR, "libhb200.so")
OBJ_DIR = os.path.join(ROOT, "build", "hb200")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC",
]


def _nvcc() -> str:
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built (there is no CPU fallback)")


def sources() -> list[str]:
    out = []
    for d in (CSRC, HOST):
        for f in sorted(os.listdir(d)):
            if f.endswith((".cu", ".cpp")):
                out.append(os.path.join(d, f))
    return out


def _deps() -> list[str]:
    deps = [os.path.join(ROOT, "include", "hb200.h")]
    for d in (CSRC, HOST):
        deps += [os.path.join(d, f) for f in os.listdir(d) if f.endswith((".hpp", ".cuh", ".h"))]
    return deps


def _stale(target: str, inputs: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(i) > t for i in inputs)


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = sources()
    deps = _deps()
    if not force and not _stale(LIB, srcs + deps):
        return LIB
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    os.makedirs(LIB_DIR, exist_ok=True)

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src) + ".o")
        if force or _stale(obj, [src] + deps):
            cmd = [nvcc, *NVCC_FLAGS, "-x", "cu", "-c", src, "-o", obj]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"nvcc failed for {src}:\n{r.stdout}\n{r.stderr}")
            if verbose and r.stderr.strip():
                print(r.stderr)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(compile_one, srcs))
    # linked beside the target and renamed over it: a reader never sees a half-written library
    tmp = LIB + ".partial"
    cmd = [nvcc, "-shared", "-o", tmp, *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    os.replace(tmp, LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
