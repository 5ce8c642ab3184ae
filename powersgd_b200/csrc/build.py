"""Builds the native library in-tree: `python -m powersgd_b200.csrc.build`.

Every translation unit is compiled for sm_100a only (`-gencode arch=compute_100a,code=sm_100a`)
and linked into `libpsgd_b200.so` next to the sources, with the CUDA runtime linked statically
so that the library loads beside any PyTorch build. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from typing import List

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libpsgd_b200.so")
OBJ_DIR = os.path.join(HERE, "build")
# the same sources with -DPSGD_BOUNDS_CHECK (see psgd_bounds.cuh): kernels validate their tiles and
# record violations instead of accessing memory; loaded through PSGD_B200_LIB by the checked tests
DEBUG_LIB = os.path.join(HERE, "libpsgd_b200_debug.so")
DEBUG_OBJ_DIR = os.path.join(HERE, "build_debug")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden", "--use_fast_math=false"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def sources() -> List[str]:
    return sorted(f for f in os.listdir(HERE) if f.endswith((".cu", ".cpp")))


def _digest(paths: List[str]) -> str:
    h = hashlib.sha256()
    for p in sorted(paths):
        with open(p, "rb") as fp:
            h.update(p.encode())
            h.update(fp.read())
    return h.hexdigest()


def _compile_one(nvcc: str, src: str, verbose: bool, debug: bool = False) -> str:
    obj = os.path.join(DEBUG_OBJ_DIR if debug else OBJ_DIR, os.path.splitext(src)[0] + ".o")
    cmd = [nvcc, *ARCH, *[c for c in COMMON if c != "--use_fast_math=false"], "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
    if debug:
        cmd.insert(1, "-DPSGD_BOUNDS_CHECK")
    if src.endswith(".cpp"):
        cmd.insert(1, "-x")
        cmd.insert(2, "cu")
    if verbose:
        cmd[1:1] = ["-Xptxas", "-v"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return obj


def build(force: bool = False, verbose: bool = False, debug: bool = False) -> str:
    """`debug=True` builds the bounds-checked variant (libpsgd_b200_debug.so) instead."""
    srcs = sources()
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".h", ".cuh"))]
    obj_dir, lib = (DEBUG_OBJ_DIR, DEBUG_LIB) if debug else (OBJ_DIR, LIB)
    stamp_path = os.path.join(obj_dir, "stamp.txt")
    digest = _digest([os.path.join(HERE, s) for s in srcs] + headers)
    if not force and os.path.exists(lib) and os.path.exists(stamp_path):
        with open(stamp_path) as fp:
            if fp.read().strip() == digest:
                return lib
    os.makedirs(obj_dir, exist_ok=True)
    nvcc = _nvcc()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile_one(nvcc, s, verbose, debug), srcs))
    link = [nvcc, *ARCH, "-shared", "-cudart", "static", "-o", lib, *objs, "-lpthread", "-ldl", "-lrt"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    with open(stamp_path, "w") as fp:
        fp.write(digest)
    return lib


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug="--debug" in sys.argv)
    print(path)
