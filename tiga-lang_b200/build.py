"""Builds libtiga_b200.so (hand-written CUDA for sm_100a) in-tree with nvcc.

    python tiga-lang_b200/build.py [--force]

Every ``csrc/*.cu`` is compiled for sm_100a only and linked into
``tiga-lang_b200/tiga/_native/libtiga_b200.so`` (git-ignored).  nvcc
cross-compiles, so no GPU is needed to build.
"""
from __future__ import annotations

import concurrent.futures
import glob
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OUT_DIR = os.path.join(HERE, "tiga", "_native")
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(OUT_DIR, "libtiga_b200.so")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
    "-I", os.path.join(ROOT, "include"), "-I", CSRC,
]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and os.path.exists(candidate):
            return candidate
    raise RuntimeError("nvcc not found; set NVCC=/path/to/nvcc")


def _newest(paths) -> float:
    return max(os.path.getmtime(p) for p in paths)


def build(force: bool = False, verbose: bool = False) -> str:
    sources = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not sources:
        raise RuntimeError("no CUDA sources found")
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest(sources + headers + [__file__]):
        return LIB
    os.makedirs(OUT_DIR, exist_ok=True)
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    header_time = _newest(headers + [__file__])

    def compile_one(src: str) -> str:
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        if force or not os.path.exists(obj) or os.path.getmtime(obj) < max(os.path.getmtime(src), header_time):
            cmd = [nvcc, *NVCC_FLAGS, "-c", src, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            result = subprocess.run(cmd, capture_output=True, text=True)
            if verbose:
                sys.stderr.write(result.stderr)
            if result.returncode:
                raise RuntimeError(f"nvcc failed for {src}:\n{result.stderr}")
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(compile_one, sources))
    link = [nvcc, "-shared", "-o", LIB, *objects, "-gencode", "arch=compute_100a,code=sm_100a",
            "-Xcompiler", "-fPIC"]
    result = subprocess.run(link, capture_output=True, text=True)
    if result.returncode:
        raise RuntimeError(f"link failed:\n{result.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
