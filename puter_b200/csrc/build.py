"""Builds libputer_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m puter_b200.csrc.build [--force]

Objects go to puter_b200/csrc/build/, the library to puter_b200/libputer_b200.so.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
OBJ_DIR = os.path.join(HERE, "build")
LIB = os.path.join(PKG, "libputer_b200.so")

SOURCES = [
    "runtime.cu",
    "convert.cu",
    "elementwise.cu",
    "norm.cu",
    "layernorm.cu",
    "softmax.cu",
    "rope.cu",
    "pages.cu",
    "attention_exact.cu",
    "decode_attention.cu",
    "prefill_attention.cu",
    "attention.cu",
]

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--extended-lambda",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", shutil.which("nvcc")):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _headers_mtime() -> float:
    m = 0.0
    for d in (HERE, os.path.join(os.path.dirname(PKG), "include")):
        for f in os.listdir(d):
            if f.endswith((".cuh", ".h")):
                m = max(m, os.path.getmtime(os.path.join(d, f)))
    return m


def _compile(nvcc: str, src: str, force: bool, hdr_mtime: float) -> str:
    obj = os.path.join(OBJ_DIR, src.replace(".cu", ".o"))
    path = os.path.join(HERE, src)
    if not force and os.path.exists(obj) and os.path.getmtime(obj) >= max(os.path.getmtime(path), hdr_mtime):
        return obj
    cmd = [nvcc, *NVCC_FLAGS, "-c", path, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src}:\n{res.stdout}\n{res.stderr}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    hdr = _headers_mtime()
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as pool:
        objs = list(pool.map(lambda s: _compile(nvcc, s, force, hdr), SOURCES))
    if force or not os.path.exists(LIB) or any(os.path.getmtime(o) > os.path.getmtime(LIB) for o in objs):
        cmd = [nvcc, "-shared", "-o", LIB, *objs, "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static", "-lcuda"]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
        if verbose:
            print("linked", LIB)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
