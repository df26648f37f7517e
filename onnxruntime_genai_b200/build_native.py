"""In-tree builders for the native artefacts.

* `_og_native.*.so` — C++17 runtime core (config, search, engine scheduler ...) with pybind11 bindings,
  compiled by g++.
* `libogb200_kernels.so` — hand-written sm_100a CUDA kernels with `extern "C"` launchers, compiled by
  nvcc (`-gencode arch=compute_100a,code=sm_100a`) and loaded through ctypes.  The launchers take raw
  device pointers and a stream, so no torch headers are needed and a full rebuild takes seconds.

* `native/c_api/libogb200_genai.so` — the C API over the package (g++, links libpython).

Each is rebuilt only when a source is newer than the artefact.  Usage: `python -m
onnxruntime_genai_b200.build_native [--force] [--verbose]`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
NATIVE_DIR = os.path.join(PKG_DIR, "native")
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
BUILD_DIR = os.path.join(PKG_DIR, "build")

NATIVE_SO = os.path.join(PKG_DIR, "_og_native" + sysconfig.get_config_var("EXT_SUFFIX"))
KERNELS_SO = os.path.join(PKG_DIR, "libogb200_kernels.so")
C_API_DIR = os.path.join(NATIVE_DIR, "c_api")
C_API_SO = os.path.join(C_API_DIR, "libogb200_genai.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr", "-Xptxas", "-v"]


def _newer(sources, target) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _run(cmd, verbose):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if verbose:
        sys.stderr.write(r.stdout + r.stderr)
    return r.stdout + r.stderr


def build_native(force=False, verbose=False) -> str:
    import pybind11
    srcs = sorted(os.path.join(NATIVE_DIR, f) for f in os.listdir(NATIVE_DIR) if f.endswith(".cpp"))
    hdrs = sorted(os.path.join(NATIVE_DIR, f) for f in os.listdir(NATIVE_DIR) if f.endswith(".h"))
    if not force and not _newer(srcs + hdrs, NATIVE_SO):
        return NATIVE_SO
    os.makedirs(os.path.join(BUILD_DIR, "native"), exist_ok=True)
    inc = ["-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"], "-I" + NATIVE_DIR]
    flags = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wno-unused-variable"]

    def compile_one(src):
        obj = os.path.join(BUILD_DIR, "native", os.path.basename(src) + ".o")
        if force or _newer([src] + hdrs, obj):
            _run(["g++", *flags, *inc, "-c", src, "-o", obj], verbose)
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    _run(["g++", "-shared", "-o", NATIVE_SO, *objs], verbose)
    return NATIVE_SO


def build_kernels(force=False, verbose=False) -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    srcs = sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith(".cu"))
    hdrs = sorted(os.path.join(CSRC_DIR, f) for f in os.listdir(CSRC_DIR) if f.endswith((".cuh", ".h")))
    if not srcs:
        raise RuntimeError("no CUDA sources found")
    if not force and not _newer(srcs + hdrs, KERNELS_SO):
        return KERNELS_SO
    os.makedirs(os.path.join(BUILD_DIR, "csrc"), exist_ok=True)
    logs = []

    def compile_one(src):
        obj = os.path.join(BUILD_DIR, "csrc", os.path.basename(src) + ".o")
        if force or _newer([src] + hdrs, obj):
            logs.append((src, _run([nvcc, *NVCC_FLAGS, "-I" + CSRC_DIR, "-c", src, "-o", obj], verbose)))
        return obj

    with ThreadPoolExecutor(max_workers=8) as ex:
        objs = list(ex.map(compile_one, srcs))
    _run([nvcc, "-shared", "-o", KERNELS_SO, *objs, "-lcuda"], verbose)
    with open(os.path.join(BUILD_DIR, "ptxas.log"), "a") as f:
        for src, log in logs:
            f.write(f"==== {os.path.basename(src)}\n{log}\n")
    return KERNELS_SO


def build_c_api(force=False, verbose=False) -> str:
    """libogb200_genai.so: the C API (native/c_api/ogb_genai_c.h), linked against libpython so that a program without an
    interpreter of its own can host the runtime."""
    import pybind11
    src = os.path.join(C_API_DIR, "ogb_genai_c.cpp")
    hdr = os.path.join(C_API_DIR, "ogb_genai_c.h")
    if not force and not _newer([src, hdr], C_API_SO):
        return C_API_SO
    libdir = sysconfig.get_config_var("LIBDIR") or "/usr/lib"
    ver = sysconfig.get_config_var("LDVERSION") or sysconfig.get_python_version()
    _run(["g++", "-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-Wall", "-I" + pybind11.get_include(),
          "-I" + sysconfig.get_paths()["include"], "-I" + C_API_DIR, "-shared", "-o", C_API_SO, src,
          "-L" + libdir, "-lpython" + ver, "-ldl", "-Wl,-rpath," + libdir], verbose)
    return C_API_SO


def build_all(force=False, verbose=False):
    return build_native(force, verbose), build_kernels(force, verbose)


if __name__ == "__main__":
    force = "--force" in sys.argv
    verbose = "--verbose" in sys.argv
    for p in build_all(force, verbose) + (build_c_api(force, verbose),):
        print("built", p)
