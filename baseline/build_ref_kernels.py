"""Builds the reference's self-contained CUDA kernels into baseline/ref_kernels/libref_kernels.so.

    python baseline/build_ref_kernels.py [--reference /path/to/onnxruntime-genai]

The reference's end-to-end runtime cannot be built offline (its build downloads ONNX Runtime), but three of its CUDA
translation units depend only on its own headers: src/cuda/cuda_topk.cu (eight top-k algorithms + the online selector),
src/cuda/beam_search_topk.cu and src/cuda/model_kernels.cu.  They are compiled here UNMODIFIED, straight from the reference
tree, for sm_100a with the flags of the reference's own build (cmake/check_cuda.cmake:45: --expt-relaxed-constexpr, C++20),
and linked with baseline/ref_kernels/harness.cu (C entry points).  benchmark/benchmark_tail_kernels.py times them next to this
framework's kernels on the same GPU.  The library is not committed; it travels with the working tree.
"""
import argparse
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "ref_kernels", "libref_kernels.so")
UNITS = ["cuda_topk.cu", "beam_search_topk.cu", "model_kernels.cu"]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    a = ap.parse_args()
    src = os.path.join(a.reference, "src", "cuda")
    if not os.path.isdir(src):
        print("reference tree not found at", a.reference)
        return 1
    build = os.path.join(HERE, "ref_kernels", "build")
    os.makedirs(build, exist_ok=True)
    flags = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++20", "--expt-relaxed-constexpr", "-Xcudafe", "--diag_suppress=2803",
             "-Xcompiler", "-fPIC", "-I" + src, "-I" + os.path.join(a.reference, "src")]

    def one(path):
        obj = os.path.join(build, os.path.basename(path) + ".o")
        r = subprocess.run(["nvcc", *flags, "-c", path, "-o", obj], capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(r.stderr[-3000:])
        return obj

    with ThreadPoolExecutor(4) as ex:
        objs = list(ex.map(one, [os.path.join(src, u) for u in UNITS] + [os.path.join(HERE, "ref_kernels", "harness.cu")]))
    r = subprocess.run(["nvcc", "-shared", "-o", OUT, *objs], capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(r.stderr[-3000:])
    print("built", OUT)
    return 0


if __name__ == "__main__":
    sys.exit(main())
