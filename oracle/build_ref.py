"""Test infrastructure: compile the reference's own CPU implementation of the transformer-layer path.

The reference sources are compiled where they lie (nothing is copied); only the built module is written,
to ``oracle/_ref/``.  The reference's CMake build cannot run on this image (its third-party submodules
are empty directories and it fetches others from the network), so the translation units of its CPU path
are handed to g++ directly:

    turbo_transformers/core/{enforce,memory,tensor,config,profiler,tensor_copy}.cpp
    turbo_transformers/core/allocator/*.cpp          (non-test)
    turbo_transformers/layers/kernels/*.cpp          (non-test)
    turbo_transformers/layers/*.cpp                  (non-test)
    turbo_transformers/python/pybind.cpp

against the stand-in headers under ``oracle/shim`` (abseil, loguru, dlpack's old names, cblas.h),
``oracle/blas_shim.cpp`` (replaces core/blas_openblas.cpp, which needs Eigen) and an OpenBLAS shared
object found in site-packages.  No ``TT_WITH_CUDA``: this is the fp32 OpenMP + cblas_sgemm path.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--force]
"""
import argparse
import glob
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT_DIR = os.path.join(HERE, "_ref")
MODULE = "turbo_transformers_cxx"


def _site_packages():
    import numpy  # any package that lives in site-packages
    return os.path.dirname(os.path.dirname(numpy.__file__))


def find_openblas():
    """An OpenBLAS .so that exports unprefixed LP64 cblas_sgemm (the opencv wheel bundles one)."""
    sp = _site_packages()
    hits = sorted(glob.glob(os.path.join(sp, "opencv_python_headless.libs", "libopenblas*.so*")))
    hits += sorted(glob.glob(os.path.join(sp, "opencv_python.libs", "libopenblas*.so*")))
    for h in hits:
        return h
    for d in ("/usr/lib/x86_64-linux-gnu", "/usr/lib64", "/usr/local/lib"):
        for h in sorted(glob.glob(os.path.join(d, "libopenblas*.so*"))):
            return h
    return None


def find_dlpack_header():
    sp = _site_packages()
    cands = [os.path.join(sp, "tvm_ffi", "include", "dlpack", "dlpack.h"),
             os.path.join(sp, "torch", "include", "ATen", "dlpack.h")]
    for c in cands:
        if os.path.exists(c):
            return c
    return None


def module_path():
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    return os.path.join(OUT_DIR, MODULE + suffix)


def blas_dir_file():
    return os.path.join(OUT_DIR, "blas_dir.txt")


def build(reference="/root/reference", force=False, verbose=True):
    """Build oracle/_ref/turbo_transformers_cxx*.so. Returns its path, or None when it cannot be built."""
    out = module_path()
    if os.path.exists(out) and not force:
        return out
    tt = os.path.join(reference, "turbo_transformers")
    if not os.path.isdir(tt):
        if verbose:
            print(f"[oracle] reference tree not found at {reference}; using the prebuilt module if any")
        return out if os.path.exists(out) else None
    blas = find_openblas()
    dlpack = find_dlpack_header()
    if blas is None or dlpack is None:
        if verbose:
            print(f"[oracle] cannot build: openblas={blas} dlpack={dlpack}")
        return None
    import pybind11
    import torch
    os.makedirs(OUT_DIR, exist_ok=True)

    def nontest(pattern):
        return [f for f in sorted(glob.glob(os.path.join(tt, pattern)))
                if not f.endswith("_test.cpp") and "catch2" not in f and "benchmark" not in f]

    core = [os.path.join(tt, "core", f + ".cpp") for f in
            ("enforce", "memory", "tensor", "config", "profiler", "tensor_copy")]
    core = [c for c in core if os.path.exists(c)]
    srcs = (core + nontest("core/allocator/*.cpp") + nontest("layers/kernels/*.cpp") + nontest("layers/*.cpp")
            + [os.path.join(HERE, "blas_shim.cpp"), os.path.join(tt, "python", "pybind.cpp")])
    torch_inc = os.path.join(os.path.dirname(torch.__file__), "include")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-fopenmp", "-march=native", "-shared", "-w",
           "-DTT_BLAS_USE_OPENBLAS", f'-DORACLE_DLPACK_HEADER="{dlpack}"',
           "-include", "functional", "-include", "algorithm", "-include", "numeric",
           "-I", os.path.join(HERE, "shim"), "-I", reference, "-I", torch_inc,
           "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
           *srcs, f"-l:{os.path.basename(blas)}", "-L", os.path.dirname(blas),
           f"-Wl,-rpath,{os.path.dirname(blas)}", "-o", out]
    if verbose:
        print("[oracle] compiling the reference CPU path:", len(srcs), "translation units")
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        if verbose:
            print(r.stdout[-4000:], r.stderr[-4000:], file=sys.stderr)
        return None
    with open(blas_dir_file(), "w") as f:
        f.write(os.path.dirname(blas))
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    p = build(a.reference, a.force)
    print(p if p else "oracle/_ref could not be built")
    sys.exit(0 if p else 1)
