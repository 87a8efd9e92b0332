"""Compile the CUDA sources of this directory into libsmore_b200.so (sm_100a only).

    python smore_b200/csrc/build.py [--force] [--verbose]

nvcc cross-compiles without a GPU.  The library is built in-tree, next to its sources, so
that it can be loaded with ctypes from a checkout.
"""
import argparse
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
LIB_PATH = os.path.join(HERE, "libsmore_b200.so")

NVCC_FLAGS = ["-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
              "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr"]


TWO_SM_SRC = os.path.join(HERE, "gemm_sm100_2sm.cu")
TWO_SM_LIB = os.path.join(HERE, "libsmore_b200_2sm.so")      # optional companion: two-SM GEMM tiles


def sources():
    """Sources of libsmore_b200.so (the companion library's source is built on its own)."""
    return sorted(f for f in glob.glob(os.path.join(HERE, "*.cu")) if f != TWO_SM_SRC)


def cutlass_include_dirs():
    """Include directories of a CUTLASS 3.x/4.x header tree with sm100 support, or None.  Looked
    for in $CUTLASS_HOME and in the header trees that ship inside installed Python packages."""
    import sysconfig
    roots = []
    if os.environ.get("CUTLASS_HOME"):
        roots.append(os.environ["CUTLASS_HOME"])
    for key in ("purelib", "platlib"):
        site = sysconfig.get_paths().get(key)
        if site:
            roots.append(os.path.join(site, "flashinfer", "data", "cutlass"))
    for r in roots:
        if os.path.isfile(os.path.join(r, "include", "cute", "arch", "mma_sm100_umma.hpp")):
            dirs = [os.path.join(r, "include")]
            util = os.path.join(r, "tools", "util", "include")
            if os.path.isdir(util):
                dirs.append(util)
            return dirs
    return None


def _local_deps(src):
    """The source plus the local headers it includes (one level is enough here)."""
    deps = [src]
    for line in open(src):
        line = line.strip()
        if line.startswith('#include "'):
            name = line.split('"')[1]
            for d in (HERE, os.path.join(ROOT, "include")):
                if os.path.exists(os.path.join(d, name)):
                    deps.append(os.path.join(d, name))
    for h in list(deps[1:]):
        if h.endswith(".cuh"):
            for line in open(h):
                if line.strip().startswith('#include "'):
                    name = line.split('"')[1]
                    for d in (HERE, os.path.join(ROOT, "include")):
                        if os.path.exists(os.path.join(d, name)):
                            deps.append(os.path.join(d, name))
    return deps


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force=False, verbose=False):
    nvcc = os.path.join(CUDA_HOME, "bin", "nvcc")
    obj_dir = os.path.join(HERE, "_obj")
    os.makedirs(obj_dir, exist_ok=True)
    cutlass = cutlass_include_dirs()
    procs, objs = [], []
    for src in sources():
        obj = os.path.join(obj_dir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if not force and not _newer(obj, _local_deps(src) + [os.path.abspath(__file__)]):
            continue
        extra = []
        if os.path.basename(src) == "gemm_sm100.cu" and cutlass:
            extra = ["-DSMORE_HAVE_CUTLASS", "--expt-extended-lambda"]
            for d in cutlass:
                extra += ["-I", d]
        cmd = [nvcc] + NVCC_FLAGS + extra + (["-Xptxas", "-v"] if verbose else []) + \
              ["-I", os.path.join(ROOT, "include"), "-I", HERE, "-c", src, "-o", obj]
        print("+", " ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd)))
    two_sm = None
    if cutlass and os.path.exists(TWO_SM_SRC) and (force or _newer(TWO_SM_LIB, _local_deps(TWO_SM_SRC) +
                                                                    [os.path.abspath(__file__)])):
        cmd = [nvcc] + NVCC_FLAGS + ["-DSMORE_HAVE_CUTLASS", "--expt-extended-lambda"]
        for d in cutlass:
            cmd += ["-I", d]
        cmd += ["-I", os.path.join(ROOT, "include"), "-I", HERE, "-shared", TWO_SM_SRC, "-o", TWO_SM_LIB + ".tmp"]
        print("+", " ".join(cmd), flush=True)
        two_sm = subprocess.Popen(cmd)
    for src, p in procs:
        if p.wait() != 0:
            raise RuntimeError("nvcc failed on " + src)
    if procs or force or _newer(LIB_PATH, objs):
        # link to a temporary name and rename: a reader never sees a half-written library
        cmd = [nvcc, "-shared", "-o", LIB_PATH + ".tmp"] + objs
        print("+", " ".join(cmd), flush=True)
        subprocess.check_call(cmd)
        os.replace(LIB_PATH + ".tmp", LIB_PATH)
    if two_sm is not None:
        if two_sm.wait() != 0:
            raise RuntimeError("nvcc failed on " + TWO_SM_SRC)
        os.replace(TWO_SM_LIB + ".tmp", TWO_SM_LIB)
    return LIB_PATH


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    a = ap.parse_args()
    print(build(a.force, a.verbose))
