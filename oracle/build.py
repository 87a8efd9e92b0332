"""Build the CPU oracle and, when the reference tree is mounted, the reference's own sources.

TEST INFRASTRUCTURE.  Outputs:
  oracle/_build/libsmore_oracle.so     plain-C restatement (smore_oracle.c), OpenMP
  oracle/_ref/libsmore_ref_host.so     the reference's functor header compiled as host C++
                                       behind ref_host_driver.cpp        (needs the reference tree)
  oracle/_ref/libsmore_ref_cuda.so     the reference's CUDA kernels compiled for sm_100a behind
                                       ref_cuda_wrapper.cu               (needs the reference tree)
Reference sources are compiled where they lie; nothing is copied into this repository.

Usage: python oracle/build.py [--reference DIR] [--force]
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEFAULT_REFERENCE = os.environ.get("SMORE_REFERENCE_DIR", "/root/reference")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def _run(cmd):
    print("+", " ".join(cmd), flush=True)
    subprocess.check_call(cmd)


def build_oracle(force=False):
    out_dir = os.path.join(HERE, "_build")
    os.makedirs(out_dir, exist_ok=True)
    src = os.path.join(HERE, "smore_oracle.c")
    out = os.path.join(out_dir, "libsmore_oracle.so")
    if force or _newer(out, [src]):
        _run(["gcc", "-O3", "-march=x86-64-v3", "-fno-fast-math", "-ffp-contract=off", "-fopenmp",
              "-shared", "-fPIC", "-o", out, src, "-lm"])
    return out


def build_reference(reference_dir, force=False):
    ext_dir = os.path.join(reference_dir, "smore", "common", "torchext")
    if not os.path.isfile(os.path.join(ext_dir, "dist_kernel.h")):
        return []
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    built = []
    host_src = os.path.join(HERE, "ref_host_driver.cpp")
    host_out = os.path.join(out_dir, "libsmore_ref_host.so")
    if force or _newer(host_out, [host_src, os.path.join(ext_dir, "dist_kernel.h")]):
        # x86-64-v3, not native: the libraries travel to another machine
        _run(["g++", "-std=c++14", "-O2", "-march=x86-64-v3", "-ffp-contract=off", "-fopenmp", "-w", "-shared", "-fPIC",
              "-I", ext_dir, "-I", os.path.join(CUDA_HOME, "include"),
              "-o", host_out, host_src])
    built.append(host_out)
    cuda_src = os.path.join(HERE, "ref_cuda_wrapper.cu")
    cuda_out = os.path.join(out_dir, "libsmore_ref_cuda.so")
    ref_cu = os.path.join(ext_dir, "ext_cuda_kernel.cu")
    if force or _newer(cuda_out, [cuda_src, ref_cu]):
        _run([os.path.join(CUDA_HOME, "bin", "nvcc"), "-O3", "-std=c++17",
              "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-w",
              "-shared", "-Xcompiler", "-fPIC", "-I", ext_dir,
              "-o", cuda_out, cuda_src, ref_cu])
    built.append(cuda_out)
    return built


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    outs = [build_oracle(a.force)]
    outs += build_reference(a.reference, a.force)
    for o in outs:
        print("built", os.path.relpath(o, HERE))


if __name__ == "__main__":
    sys.exit(main())
