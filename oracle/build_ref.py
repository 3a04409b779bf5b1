"""Build the reference's own CUDA library (fp32, cuBLAS) for sm_100a into oracle/_ref/.

    python oracle/build_ref.py [--reference <checkout of the reference>]

TEST INFRASTRUCTURE: the result, oracle/_ref/libcudaBERT_ref.so, is a second checker for the
GPU parity tests and the "reference CUDA on the same box" line of the benchmark notes.  The
product never loads it.  Sources are compiled where they lie in the reference tree (nothing is
copied into this repository); the reference's CMake project is not used (it needs the removed
find_package(CUDA) and the CUDA-samples headers), only its source list
(cuda_bert/CMakeLists.txt:33-46) with two small stand-in headers from oracle/shim/.

Differences from the reference's own flags (cuda_bert/CMakeLists.txt:26-31): an explicit
-arch=sm_100a (the reference passes none), C++17 instead of C++11 (needed by the toolkit's
headers), and NO -use_fast_math, so that tanh / exp / division are the accurate versions and the
library can serve as a numerical reference.
"""
import argparse
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SOURCES = ["utils/bert.cu", "utils/common.cc", "utils/load_model.cc", "utils/manager.cu", "ops/elementwise.cu",
           "ops/embedding.cu", "ops/layernorm.cu", "ops/linear.cu", "ops/matmul.cu", "ops/softmax.cu",
           "ops/batch_matmul.cu", "cuda_bert.cu", "ops/crossEntropyLoss.cu"]


def default_reference_dir():
    env = os.environ.get("CUDABERT_REFERENCE")
    return env if env else os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=default_reference_dir(),
                    help="checkout of the reference project (default: $CUDABERT_REFERENCE, else the "
                         "directory 'reference' beside this repository)")
    args = ap.parse_args()
    src_root = os.path.join(args.reference, "cuda_bert")
    if not os.path.isdir(src_root):
        sys.exit("reference tree not found at %s" % src_root)
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    os.makedirs(os.path.join(OUT, "obj"), exist_ok=True)
    lib = os.path.join(OUT, "libcudaBERT_ref.so")
    if os.path.exists(lib) and "--force" not in sys.argv:
        print("up to date:", lib)
        return

    def compile_one(rel):
        obj = os.path.join(OUT, "obj", rel.replace("/", "_") + ".o")
        cmd = [nvcc, "-x", "cu", "-arch=sm_100a", "-std=c++17", "--expt-relaxed-constexpr", "-O3", "-Xcompiler",
               "-fPIC", "-w", "-I" + os.path.join(HERE, "shim"), "-I" + src_root, "-DHAVE_CUDA", "-rdc=true", "-c",
               os.path.join(src_root, rel), "-o", obj]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode:
            raise RuntimeError("%s\n%s" % (" ".join(cmd), r.stderr[-2000:]))
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    cnpy_obj = os.path.join(OUT, "obj", "cnpy.o")
    r = subprocess.run(["g++", "-O2", "-fPIC", "-w", "-c", os.path.join(src_root, "cnpy", "cnpy.cpp"), "-o", cnpy_obj],
                       capture_output=True, text=True)
    if r.returncode:
        sys.exit("cnpy: " + r.stderr[-2000:])
    r = subprocess.run([nvcc, "-arch=sm_100a", "-shared", "-o", lib] + objs + [cnpy_obj, "-lcublas", "-lz"],
                       capture_output=True, text=True)
    if r.returncode:
        sys.exit("link: " + r.stderr[-2000:])
    print("built", lib)


if __name__ == "__main__":
    main()
