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


def _compile_one(nvcc: str, src: str, verbose: bool) -> str:
    obj = os.path.join(OBJ_DIR, os.path.splitext(src)[0] + ".o")
    cmd = [nvcc, *ARCH, *[c for c in COMMON if c != "--use_fast_math=false"], "-I", HERE, "-c", os.path.join(HERE, src), "-o", obj]
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


def build(force: bool = False, verbose: bool = False) -> str:
    srcs = sources()
    headers = [os.path.join(HERE, f) for f in os.listdir(HERE) if f.endswith((".h", ".cuh"))]
    stamp_path = os.path.join(OBJ_DIR, "stamp.txt")
    digest = _digest([os.path.join(HERE, s) for s in srcs] + headers)
    if not force and os.path.exists(LIB) and os.path.exists(stamp_path):
        with open(stamp_path) as fp:
            if fp.read().strip() == digest:
                return LIB
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
        objs = list(pool.map(lambda s: _compile_one(nvcc, s, verbose), srcs))
    link = [nvcc, *ARCH, "-shared", "-cudart", "static", "-o", LIB, *objs, "-lpthread", "-ldl", "-lrt"]
    res = subprocess.run(link, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    with open(stamp_path, "w") as fp:
        fp.write(digest)
    return LIB


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
