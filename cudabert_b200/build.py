"""Build libcudaBERT.so (and the unit_test program) in-tree with nvcc for sm_100a.

    python -m cudabert_b200.build [--force]

Objects go to cudabert_b200/csrc/build/, the library to cudabert_b200/cuda_bert/libcudaBERT.so
(the place the reference's binding looks for it, cuda_bert/pybert.py:10-11).  nvcc
cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(CSRC, "build")
LIB = os.path.join(HERE, "cuda_bert", "libcudaBERT.so")
UNIT_TEST = os.path.join(HERE, "cuda_bert", "unit_test")

CUDA_SOURCES = ["gemm_tcgen05.cu", "gemm_f32.cu", "attention.cu", "attention_tc.cu", "rowwise.cu", "model.cu", "abi.cu"]
CXX_SOURCES = ["npy.cc", "batcher.cc", "tokenizer.cc", "reader.cc"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found")
    return exe


def _newer(target: str, deps) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(d) <= t for d in deps)


def _headers():
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    hs.append(os.path.join(os.path.dirname(HERE), "include", "cudabert.h"))
    return hs


def _compile(src: str, force: bool) -> str:
    obj = os.path.join(OBJ, os.path.splitext(src)[0] + ".o")
    path = os.path.join(CSRC, src)
    if not force and _newer(obj, [path] + _headers()):
        return obj
    if src.endswith(".cu"):
        cmd = [nvcc()] + NVCC_FLAGS + ["-c", path, "-o", obj]
    else:
        cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-c", path, "-o", obj]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("compile failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(os.path.dirname(LIB), exist_ok=True)
    srcs = CUDA_SOURCES + CXX_SOURCES
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, force), srcs))
    if force or not _newer(LIB, objs):
        cmd = [nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", LIB] + objs
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("link failed: %s\n%s\n%s" % (" ".join(cmd), r.stdout, r.stderr))
    ut_src = os.path.join(CSRC, "unit_test.cpp")
    if os.path.exists(ut_src) and (force or not _newer(UNIT_TEST, [ut_src, LIB])):
        cmd = ["g++", "-O2", "-std=c++17", ut_src, "-o", UNIT_TEST, "-L" + os.path.dirname(LIB), "-lcudaBERT",
               "-Wl,-rpath,$ORIGIN"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("unit_test link failed:\n%s\n%s" % (r.stdout, r.stderr))
    if verbose:
        print("built", LIB)
    return LIB


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
