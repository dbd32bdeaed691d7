"""In-tree build of the native pieces (nvcc cross-compiles sm_100a without a GPU).

    python -m turbotransformers_b200.build            # libttb.so + the pybind module
    python -m turbotransformers_b200.build --force

Outputs (git-ignored, shipped with the tree to GPU machines):
    turbotransformers_b200/libttb.so                          C ABI + CUDA kernels (include/ttb.h)
    turbotransformers_b200/turbo_transformers_cxx*.so         C++ layer classes + pybind11 surface
    turbotransformers_b200/bert_model_example                 command-line host of the C++ API (npz model, no Python)
"""
import argparse
import glob
import os
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
OBJ = os.path.join(PKG, "build")
LIBTTB = os.path.join(PKG, "libttb.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", "-I", os.path.join(ROOT, "include"), "-I", CSRC]


def _nvcc():
    for c in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if c and (os.path.exists(c) or c == "nvcc"):
            return c
    return "nvcc"


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def cxx_module_path():
    return os.path.join(PKG, "turbo_transformers_cxx" + sysconfig.get_config_var("EXT_SUFFIX"))


def build_libttb(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    cus = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    objs, jobs = [], []
    for cu in cus:
        o = os.path.join(OBJ, os.path.basename(cu)[:-3] + ".o")
        objs.append(o)
        if force or _newer(o, [cu] + hdrs):
            jobs.append((cu, o))

    def compile_one(job):
        cu, o = job
        r = subprocess.run([_nvcc(), *NVCC_FLAGS, "-c", cu, "-o", o], capture_output=True, text=True)
        with open(o + ".log", "w") as f:
            f.write(r.stdout + r.stderr)
        return cu, r

    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for cu, r in ex.map(compile_one, jobs):
                if verbose or r.returncode != 0:
                    print(f"[build] {os.path.basename(cu)}\n{r.stdout}{r.stderr}")
                if r.returncode != 0:
                    raise RuntimeError(f"nvcc failed on {cu}")
    if jobs or not os.path.exists(LIBTTB):
        r = subprocess.run([_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", *objs, "-o", LIBTTB],
                           capture_output=True, text=True)
        if r.returncode != 0:
            print(r.stdout, r.stderr)
            raise RuntimeError("linking libttb.so failed")
    return LIBTTB


def build_cxx_module(force=False, verbose=False):
    """C++ layer classes + pybind11 module; plain g++, links against libttb.so next to it."""
    host = os.path.join(CSRC, "host")
    srcs = sorted(glob.glob(os.path.join(host, "*.cpp")))
    if not srcs:
        return None
    out = cxx_module_path()
    deps = srcs + glob.glob(os.path.join(host, "*.h")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and not _newer(out, deps):
        return out
    import pybind11
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-Wall", "-I", os.path.join(ROOT, "include"),
           "-I", host, "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"], *srcs,
           "-L", PKG, "-l:libttb.so", "-lz", "-Wl,-rpath,$ORIGIN", "-o", out]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout, r.stderr)
    if r.returncode != 0:
        raise RuntimeError("building the pybind module failed")
    return out


EXAMPLE = os.path.join(PKG, "bert_model_example")


def build_example(force=False, verbose=False):
    """The Python-free command-line host: C++ layer classes + npz loader + BertModel, no pybind, no libpython."""
    host = os.path.join(CSRC, "host")
    srcs = [s for s in sorted(glob.glob(os.path.join(host, "*.cpp"))) if os.path.basename(s) != "pybind.cpp"]
    srcs += sorted(glob.glob(os.path.join(CSRC, "example", "*.cpp")))
    deps = srcs + glob.glob(os.path.join(host, "*.h")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    if not force and not _newer(EXAMPLE, deps):
        return EXAMPLE
    cmd = ["g++", "-O2", "-std=c++17", "-Wall", "-pthread", "-I", os.path.join(ROOT, "include"), "-I", host, *srcs,
           "-L", PKG, "-l:libttb.so", "-lz", "-Wl,-rpath,$ORIGIN", "-o", EXAMPLE]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or r.returncode != 0:
        print(r.stdout, r.stderr)
    if r.returncode != 0:
        raise RuntimeError("building bert_model_example failed")
    return EXAMPLE


def build_all(force=False, verbose=False):
    lib = build_libttb(force, verbose)
    mod = build_cxx_module(force, verbose)
    exe = build_example(force, verbose)
    return lib, mod, exe


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    a = ap.parse_args()
    print(build_all(a.force, a.verbose))
