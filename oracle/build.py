"""Build the CPU oracle and, when the reference tree is mounted, the reference's own sources.

TEST INFRASTRUCTURE.  Outputs:
  oracle/_build/libsmore_oracle.so     plain-C restatement (smore_oracle.c), OpenMP
  oracle/_ref/libsmore_ref_host.so     the reference's functor header compiled as host C++
                                       behind ref_host_driver.cpp        (needs the reference tree)
  oracle/_ref/libsmore_ref_cuda.so     the reference's CUDA kernels compiled for sm_100a behind
                                       ref_cuda_wrapper.cu               (needs the reference tree)
  oracle/_ref/libsmore_ref_kg.so       the reference's knowledge-graph container (cpp_sampler's
                                       knowledge_graph.cpp, utils.cpp) behind ref_kg_driver.cpp
  oracle/_ref/pyref/smore/             the reference's Python package (*.py only) placed next to the
                                       two libraries, so that its own op front-ends, models and
                                       training step can be imported where the reference tree is
                                       not mounted (oracle/ref_harness.py)
Reference sources are compiled where they lie; oracle/_ref/ is a build output that version control
ignores, so nothing of the reference enters this repository's history.

Usage: python oracle/build.py [--reference DIR] [--force]
"""
import argparse
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))


def default_reference():
    """$SMORE_REFERENCE_DIR, else a checkout named `reference` beside this repository, else ''."""
    env = os.environ.get("SMORE_REFERENCE_DIR", "")
    if env:
        return env
    beside = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return beside if os.path.isdir(os.path.join(beside, "smore")) else ""


DEFAULT_REFERENCE = default_reference()
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


def build_pyref(reference_dir, force=False):
    """Place the reference's Python package under oracle/_ref/pyref (files are taken as they are)."""
    import shutil
    src_root = os.path.join(reference_dir, "smore")
    if not os.path.isfile(os.path.join(src_root, "common", "torchext", "ext_ops.py")):
        return []
    dst_root = os.path.join(HERE, "_ref", "pyref", "smore")
    n = 0
    for dirpath, dirnames, filenames in os.walk(src_root):
        dirnames[:] = [d for d in dirnames if d not in ("build", "__pycache__")]
        for name in filenames:
            if not name.endswith(".py"):
                continue
            src = os.path.join(dirpath, name)
            dst = os.path.join(dst_root, os.path.relpath(src, src_root))
            if force or _newer(dst, [src]):
                os.makedirs(os.path.dirname(dst), exist_ok=True)
                shutil.copyfile(src, dst)
                n += 1
    if n:
        print("placed %d reference .py files under %s" % (n, os.path.relpath(dst_root, HERE)), flush=True)
    return [dst_root]


def build_reference(reference_dir, force=False):
    if not reference_dir:
        return []
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
    built += build_ref_kg(reference_dir, force)
    built += build_pyref(reference_dir, force)
    return built


def build_ref_kg(reference_dir, force=False):
    """oracle/_ref/libsmore_ref_kg.so: the reference's knowledge-graph container (its own
    knowledge_graph.cpp, alias_method.cpp and utils.cpp, compiled where they lie) behind ref_kg_driver.cpp."""
    import sysconfig
    smp = os.path.join(reference_dir, "smore", "cpp_sampler")
    srcs = [os.path.join(smp, "src", "lib", n) for n in ("knowledge_graph.cpp", "utils.cpp", "alias_method.cpp")]
    if not all(os.path.isfile(s) for s in srcs):
        return []
    try:
        import pybind11
    except ImportError:
        return []
    out = os.path.join(HERE, "_ref", "libsmore_ref_kg.so")
    driver = os.path.join(HERE, "ref_kg_driver.cpp")
    if force or _newer(out, srcs + [driver]):
        # no -DNDEBUG: the reference reads and writes files inside assert()
        _run(["g++", "-std=c++14", "-O2", "-march=x86-64-v3", "-w", "-shared", "-fPIC",
              "-I", os.path.join(smp, "include"), "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
              "-o", out, driver] + srcs)
    return [out]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=DEFAULT_REFERENCE,
                    help="checkout of the reference (default: $SMORE_REFERENCE_DIR, else ../reference); without it only "
                         "the C oracle is built")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    outs = [build_oracle(a.force)]
    outs += build_reference(a.reference, a.force)
    for o in outs:
        print("built", os.path.relpath(o, HERE))


if __name__ == "__main__":
    sys.exit(main())
