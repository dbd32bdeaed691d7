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

``--cuda`` additionally builds the same translation units with ``-DTT_WITH_CUDA`` plus
core/cuda_device_context.cpp and layers/kernels/gpu_*.cu (nvcc, sm_100a; cub and thrust come with the
toolkit) against cuBLAS, into ``oracle/_ref/cuda/``: the reference's own fp32 GPU path, used by one GPU
test as a second checker and as a second timed baseline.  Both modules export the same C++ types, so a
process may import only one of them.

Usage:  python oracle/build_ref.py [--reference /path/to/reference] [--force] [--cuda]
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


def default_reference():
    """Where the reference checkout is looked for when no path is given: $TT_REFERENCE_ROOT, else a directory named
    `reference` beside this repository."""
    return os.environ.get("TT_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")


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


def build(reference=None, force=False, verbose=True):
    """Build oracle/_ref/turbo_transformers_cxx*.so. Returns its path, or None when it cannot be built."""
    reference = reference or default_reference()
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


def cuda_module_path():
    suffix = sysconfig.get_config_var("EXT_SUFFIX")
    return os.path.join(OUT_DIR, "cuda", MODULE + suffix)


def build_cuda(reference=None, force=False, verbose=True, cuda_home=None):
    """Build oracle/_ref/cuda/turbo_transformers_cxx*.so (the reference with TT_WITH_CUDA). Returns its path or None."""
    import shutil
    import tempfile
    out = cuda_module_path()
    if os.path.exists(out) and not force:
        return out
    reference = reference or default_reference()
    if cuda_home is None:  # the toolkit that owns the nvcc on PATH, else $CUDA_HOME
        nvcc_on_path = shutil.which("nvcc")
        cuda_home = os.environ.get("CUDA_HOME") or (os.path.dirname(os.path.dirname(os.path.realpath(nvcc_on_path))) if nvcc_on_path else "")
    tt = os.path.join(reference, "turbo_transformers")
    blas, dlpack = find_openblas(), find_dlpack_header()
    nvcc = os.path.join(cuda_home, "bin", "nvcc")
    if not os.path.isdir(tt) or blas is None or dlpack is None or not os.path.exists(nvcc):
        if verbose:
            print(f"[oracle] cuda build skipped: reference={os.path.isdir(tt)} openblas={blas} dlpack={dlpack} nvcc={os.path.exists(nvcc)}")
        return out if os.path.exists(out) else None
    import pybind11
    import torch
    os.makedirs(os.path.dirname(out), exist_ok=True)

    def nontest(pattern):
        return [f for f in sorted(glob.glob(os.path.join(tt, pattern)))
                if "_test." not in os.path.basename(f) and "catch2" not in f and "benchmark" not in f]

    core = [os.path.join(tt, "core", f + ".cpp") for f in
            ("enforce", "memory", "tensor", "config", "profiler", "tensor_copy", "cuda_device_context")]
    core = [c for c in core if os.path.exists(c)]
    srcs = (core + nontest("core/allocator/*.cpp") + nontest("layers/kernels/*.cpp") + nontest("layers/*.cpp")
            + nontest("layers/kernels/*.cu") + [os.path.join(HERE, "blas_shim.cpp"), os.path.join(tt, "python", "pybind.cpp")])
    torch_inc = os.path.join(os.path.dirname(torch.__file__), "include")
    common = ["-O2", "-std=c++17", "-w", "-DTT_BLAS_USE_OPENBLAS", "-DTT_WITH_CUDA", f'-DORACLE_DLPACK_HEADER="{dlpack}"',
              "-include", "functional", "-include", "algorithm", "-include", "numeric", "-include", "sstream",
              "-I", os.path.join(HERE, "shim"), "-I", reference, "-I", torch_inc, "-I", pybind11.get_include(),
              "-I", sysconfig.get_paths()["include"], "-I", os.path.join(cuda_home, "include")]
    if verbose:
        print("[oracle] compiling the reference GPU path:", len(srcs), "translation units")
    objdir = tempfile.mkdtemp(prefix="ref_cuda_obj_")
    try:
        jobs, objs = [], []
        for i, src in enumerate(srcs):
            obj = os.path.join(objdir, f"{i}_{os.path.basename(src)}.o")
            objs.append(obj)
            if src.endswith(".cu"):
                cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC,-fopenmp",
                       "--expt-relaxed-constexpr", *common, "-c", src, "-o", obj]
            else:
                cmd = ["g++", "-fPIC", "-fopenmp", "-march=native", *common, "-c", src, "-o", obj]
            jobs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        failed = False
        for src, job in jobs:
            log, _ = job.communicate()
            if job.returncode != 0:
                failed = True
                if verbose:
                    print(f"[oracle] {src} failed:\n{log[-3000:]}", file=sys.stderr)
        if failed:
            return None
        link = ["g++", "-shared", "-fopenmp", *objs, f"-l:{os.path.basename(blas)}", "-L", os.path.dirname(blas),
                f"-Wl,-rpath,{os.path.dirname(blas)}", "-L", os.path.join(cuda_home, "lib64"),
                f"-Wl,-rpath,{os.path.join(cuda_home, 'lib64')}", "-lcublas", "-lcudart", "-o", out]
        r = subprocess.run(link, capture_output=True, text=True)
        if r.returncode != 0:
            if verbose:
                print(r.stderr[-3000:], file=sys.stderr)
            return None
    finally:
        shutil.rmtree(objdir, ignore_errors=True)
    with open(blas_dir_file(), "w") as f:
        f.write(os.path.dirname(blas))
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=None, help="the reference checkout (default: $TT_REFERENCE_ROOT, else ../reference)")
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--cuda", action="store_true", help="also build the reference's GPU path into oracle/_ref/cuda/")
    a = ap.parse_args()
    p = build(a.reference, a.force)
    print(p if p else "oracle/_ref could not be built")
    ok = bool(p)
    if a.cuda:
        q = build_cuda(a.reference, a.force)
        print(q if q else "oracle/_ref/cuda could not be built")
        ok = ok and bool(q)
    sys.exit(0 if ok else 1)
