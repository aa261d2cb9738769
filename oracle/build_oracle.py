"""Builds the C++ restatement of the reference algorithm (oracle/cpu_ref.cpp) into oracle/_build/liboracle.so.
TEST INFRASTRUCTURE: used by tests/, the smoke check and the benchmark's CPU legs only.

The reference itself cannot be compiled here (its host library needs the cuda-kernel-loader, json, magic_enum and
spdlog submodules, which are empty or absent in the checkout, and its CPU test math needs Eigen, a network download),
so there is no oracle/_ref build.
"""
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_build", "liboracle.so")


def build(force=False):
    src = os.path.join(HERE, "cpu_ref.cpp")
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(src):
        return OUT
    subprocess.check_call(["g++", "-O3", "-march=x86-64-v3", "-fopenmp", "-shared", "-fPIC", "-std=c++17", "-o", OUT, src])
    return OUT


if __name__ == "__main__":
    print(build(force=True))
