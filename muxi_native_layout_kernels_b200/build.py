"""Builds libmlk_b200.so (the C-ABI library of hand-written sm_100a kernels) next to this file.

Usage: ``python muxi_native_layout_kernels_b200/build.py [--force] [--verbose]`` (run it as a script: importing the
package would try to load the library that is about to be built).
Plays the role of the reference's ``setup.py`` (setup.py:56-103: one extension, 21 sources), but the
result is a plain shared library with an ``extern "C"`` surface and no dependency on torch headers.
nvcc cross-compiles without a GPU, so this also runs on a CPU-only machine.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR / "csrc"
OBJ_DIR = PKG_DIR / "build"
LIB_PATH = PKG_DIR / "libmlk_b200.so"

SOURCES = [
    "abi.cu",
    "dense.cu",
    "dense_umma.cu",
    "dense_umma_f8.cu",
    "dense_umma_f8n.cu",
    "hgemm_umma.cu",
    "prepack.cu",
    "moe_router.cu",
    "moe_align.cu",
    "moe_experts.cu",
    "moe_umma.cu",
    "moe_umma_f8n.cu",
    "moe_decode.cu",
    "ep_reduce.cu",
    "moe_exchange.cu",
    "selector.cpp",
]

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
]


def _nvcc() -> str:
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(cand):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build libmlk_b200.so")
    return cand


def _stamp() -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.iterdir()) + [PKG_DIR.parent / "include" / "mlk_b200.h"]):
        if p.is_file():
            h.update(p.name.encode())
            h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def _compile(src: str, verbose: bool) -> str:
    obj = OBJ_DIR / (src + ".o")
    cmd = [_nvcc(), *NVCC_FLAGS, "-x", "cu", "-c", str(CSRC / src), "-o", str(obj)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    (OBJ_DIR / (src + ".log")).write_text(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src}:\n{res.stdout}\n{res.stderr}")
    if verbose:
        sys.stderr.write(res.stderr)
    return str(obj)


def build(force: bool = False, verbose: bool = False) -> Path:
    """Compiles every source for sm_100a and links libmlk_b200.so; no-op when sources are unchanged."""
    OBJ_DIR.mkdir(exist_ok=True)
    stamp_file = OBJ_DIR / "stamp"
    stamp = _stamp()
    if not force and LIB_PATH.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return LIB_PATH
    with cf.ThreadPoolExecutor(max_workers=min(len(SOURCES), os.cpu_count() or 4)) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), SOURCES))
    cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *objs, "-gencode", "arch=compute_100a,code=sm_100a"]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    stamp_file.write_text(stamp)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true", help="print ptxas register / shared-memory usage")
    a = ap.parse_args()
    print(build(force=a.force, verbose=a.verbose))
