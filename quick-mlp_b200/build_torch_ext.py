"""Builds quick-mlp_b200/lib/torch_ext/qmlp_cu.so: the TorchScript custom classes torch.classes.qmlp_cu.* (csrc/torch/
qmlp_cu.cpp) over the header-only C++ class layer and libqmlp_b200.so. Host C++ only (no kernels in it); nvcc is not
involved and no GPU is needed to build."""
import os
import shutil

HERE = os.path.dirname(os.path.abspath(__file__))
LIBDIR = os.path.join(HERE, "lib")
OUTDIR = os.path.join(LIBDIR, "torch_ext")
OUT = os.path.join(OUTDIR, "qmlp_cu.so")


def build(verbose=False):
    from torch.utils import cpp_extension
    src = os.path.join(HERE, "csrc", "torch", "qmlp_cu.cpp")
    include = os.path.abspath(os.path.join(HERE, "..", "include"))
    deps = [src, os.path.join(include, "qmlp_b200.h")] + [os.path.join(include, "qmlp", f) for f in os.listdir(os.path.join(include, "qmlp"))]
    if os.path.exists(OUT) and os.path.getmtime(OUT) >= max(os.path.getmtime(p) for p in deps):
        return OUT
    os.makedirs(OUTDIR, exist_ok=True)
    # The extension must share the process's libstdc++.so with libqmlp_b200.so and with PyTorch. A compiler wrapper that
    # links the C++ runtime statically (one is first on PATH in some images) would put a second, uninitialised copy of
    # it into qmlp_cu.so, and every library loaded after it would bind its stream and locale symbols to that copy.
    if os.path.exists("/usr/bin/g++"):
        os.environ["CXX"] = "/usr/bin/g++"
    cpp_extension.load(name="qmlp_cu", sources=[src], extra_include_paths=[include], extra_cflags=["-O2", "-std=c++17"],
                       extra_ldflags=["-L" + LIBDIR, "-lqmlp_b200", "-Wl,-rpath," + LIBDIR, "-lstdc++"],
                       with_cuda=True, is_python_module=False, build_directory=OUTDIR, verbose=verbose)
    for junk in ("build.ninja", ".ninja_deps", ".ninja_log", "qmlp_cu.o"):
        p = os.path.join(OUTDIR, junk)
        if os.path.exists(p):
            os.remove(p)
    return OUT


if __name__ == "__main__":
    print(build(verbose=True))
