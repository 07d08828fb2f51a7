"""Builds libfeather_b200.so (the C-ABI library declared in include/feather_b200.h) in-tree with nvcc for sm_100a.

Usage: ``python build.py`` from any directory, or ``build_library()`` from Python.  nvcc cross-compiles, so no GPU is
needed to build.  The library links the CUDA runtime statically and resolves the one driver symbol it needs
(cuTensorMapEncodeTiled) at run time, so it also loads on a machine without a driver (every call then reports an error).
"""

import os
import shutil
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC_DIR = os.path.join(PKG_DIR, "csrc")
LIB_PATH = os.path.join(PKG_DIR, "libfeather_b200.so")
SOURCES = ["scaled_mm.cu", "scaled_mm_ext.cu", "quant.cu", "small_m.cu", "exchange.cu"]
HEADERS = ["ptx.cuh", "host_util.h", os.path.join("..", "..", "include", "feather_b200.h")]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--cudart",
    "static",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libfeather_b200.so cannot be built")
    return nvcc


def is_stale():
    if not os.path.exists(LIB_PATH):
        return True
    built = os.path.getmtime(LIB_PATH)
    deps = [os.path.join(CSRC_DIR, s) for s in SOURCES + HEADERS]
    return any(os.path.getmtime(d) > built for d in deps if os.path.exists(d))


def build_library(force=False, verbose=False):
    """Compile every .cu under csrc/ into libfeather_b200.so.  Returns the library path."""
    if not force and not is_stale():
        return LIB_PATH
    nvcc = _nvcc()
    objs = []
    build_dir = os.path.join(PKG_DIR, "build")
    os.makedirs(build_dir, exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = os.path.join(build_dir, src.replace(".cu", ".o"))
        cmd = [nvcc, *NVCC_FLAGS, "-c", os.path.join(CSRC_DIR, src), "-o", obj]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objs.append(obj)
    for src, proc in procs:
        out, _ = proc.communicate()
        if verbose and out:
            print(out)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{out}")
    tmp = LIB_PATH + ".tmp"
    link = [nvcc, "-shared", "--cudart", "static", "-Xcompiler", "-fPIC", "-o", tmp, *objs]
    res = subprocess.run(link, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}")
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


CBENCH_SRC = os.path.join(PKG_DIR, "cbench", "bench_scaled_mm.c")
CBENCH_BIN = os.path.join(PKG_DIR, "cbench", "bench_scaled_mm")


def build_cbench(cc=None):
    """Compile cbench/bench_scaled_mm.c - plain C against include/feather_b200.h, linked with the library and the CUDA runtime."""
    build_library()
    cc = cc or shutil.which("cc") or shutil.which("gcc")
    if cc is None:
        raise RuntimeError("no C compiler found")
    cuda = os.path.dirname(os.path.dirname(_nvcc()))
    cmd = [cc, "-std=c99", "-O2", "-Wall", "-Wextra", "-pedantic", CBENCH_SRC, "-I", os.path.join(PKG_DIR, "..", "include"), "-I", os.path.join(cuda, "include"),
           "-L", PKG_DIR, "-lfeather_b200", "-L", os.path.join(cuda, "lib64"), "-lcudart", "-lm", "-Wl,-rpath," + PKG_DIR,
           "-Wl,-rpath," + os.path.join(cuda, "lib64"), "-o", CBENCH_BIN]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"C harness failed to build:\n{res.stdout}")
    return CBENCH_BIN


if __name__ == "__main__":
    path = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
    if "--cbench" in sys.argv:
        print(build_cbench())
