"""Builds libqmlp_b200.so (host library + spec-independent kernels) in-tree with nvcc for sm_100a.

Usage: python quick-mlp_b200/build.py [--force]
The per-spec kernel instantiations are built on demand by the library itself (see csrc/jit.cpp) into
quick-mlp_b200/lib/specs/; `prebuild_specs` below instantiates a list of network specs ahead of time so a
machine without a compiler cache hit still finds them.
"""
import hashlib
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
LIB = os.path.join(LIBDIR, "libqmlp_b200.so")
SOURCES = ["host.cpp", "jit.cpp", "capi.cpp", "generic_kernels.cu", "static_scratch.cu"]
NVCC = os.environ.get("QMLP_NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _digest():
    h = hashlib.sha256()
    for root, _, files in sorted(os.walk(CSRC)):
        if os.path.basename(root) == "kernels":
            continue  # template headers only enter the per-spec instantiations
        for f in sorted(files):
            if f.endswith((".cpp", ".cu", ".h", ".hpp")):
                h.update(f.encode())
                h.update(open(os.path.join(root, f), "rb").read())
    h.update(open(os.path.join(CSRC, "kernels", "launch_args.h"), "rb").read())
    h.update(open(os.path.join(HERE, "..", "include", "qmlp_b200.h"), "rb").read())
    return h.hexdigest()


def build_library(force=False, verbose=True):
    os.makedirs(LIBDIR, exist_ok=True)
    stamp = os.path.join(LIBDIR, "libqmlp_b200.stamp")
    digest = _digest()
    if not force and os.path.exists(LIB) and os.path.exists(stamp) and open(stamp).read() == digest:
        return LIB
    cmd = [NVCC, "-std=c++17", "-O3", "-lineinfo", *ARCH, "-shared", "-Xcompiler", "-fPIC,-fvisibility=hidden",
           "-o", LIB] + [os.path.join(CSRC, s) for s in SOURCES] + ["-ldl"]
    if verbose:
        print(" ".join(cmd), flush=True)
    subprocess.check_call(cmd)
    with open(stamp, "w") as f:
        f.write(digest)
    return LIB


if __name__ == "__main__":
    build_library(force="--force" in sys.argv)
    print("built", LIB)
