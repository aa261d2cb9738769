"""The header-only C++ class layer (include/qmlp/*.h: qmlp::FusedNetwork, IEncoding, Activation, Tensor, TmpMemory,
QuickMLP with the reference's method names, src_cpp/include/qmlp/fused_network.h:16-340) compiles with g++ against
libqmlp_b200.so and behaves: layout queries on the CPU, inference / forward / adjoint against the oracle on a GPU."""
import json
import os
import subprocess

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "quick-mlp_b200", "lib")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build(tmp_path):
    exe = os.path.join(LIBDIR, "shim_check")
    src = os.path.join(ROOT, "tests", "cpp", "shim_check.cpp")
    headers = [os.path.join(ROOT, "include", "qmlp", f) for f in os.listdir(os.path.join(ROOT, "include", "qmlp"))]
    newest = max(os.path.getmtime(p) for p in headers + [src, os.path.join(ROOT, "include", "qmlp_b200.h")])
    if not os.path.exists(exe) or os.path.getmtime(exe) < newest:
        cmd = ["g++", "-std=c++17", "-O1", "-Wall", "-I", os.path.join(ROOT, "include"), "-I", os.path.join(CUDA, "include"), src,
               "-o", exe, "-L", LIBDIR, "-lqmlp_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
               "-Wl,-rpath," + LIBDIR, "-Wl,-rpath," + os.path.join(CUDA, "lib64")]
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-4000:]
    return exe


def _run(exe, *args):
    r = subprocess.run([exe, *args], capture_output=True, text=True, timeout=600)
    lines = dict(l.split(" ", 1) for l in r.stdout.strip().splitlines() if " " in l)
    return r, lines


def test_class_layer_builds_and_reports_the_layout(tmp_path):
    exe = _build(tmp_path)
    cfg = specs.config3(log2_hashmap_size=12)
    spec_file = tmp_path / "spec.json"
    spec_file.write_text(json.dumps(cfg))
    r, out = _run(exe, "layout", str(spec_file))
    assert r.returncode == 0, r.stdout + r.stderr
    spec = oracle.parse_spec(cfg)
    assert out["bad_spec"] == "configuration_error"
    assert out["channels"] == f"{spec.num_inputs} {spec.num_outputs}"
    assert out["layers"] == f"{len(spec.layers)} encodings {len(spec.encodings)}"
    assert out["parameters"] == f"{spec.num_parameters} precision half float"
    e = spec.encodings[0]
    assert out["encoding"] == f"0 HashGrid out {e.num_outputs} max_in 2 params {e.num_parameters} levels {len(e.levels)}"
    text = r.stdout
    for i, l in enumerate(spec.layers):
        assert f"layer {i} w {l.channels_out}x{l.channels_in} at {l.weights_start} bias {l.bias_start if l.use_bias else -1}" in text
    assert out["activation"].startswith("celu code_bytes ")
    assert out["factory"] == "Identity 2 2"


@pytest.mark.gpu
def test_class_layer_runs_the_kernels(tmp_path):
    exe = _build(tmp_path)
    cfg = specs.config2()
    spec = oracle.parse_spec(cfg)
    (tmp_path / "spec.json").write_text(json.dumps(cfg))
    n = 1500
    x = helpers.uniform(61, 1, (n, spec.num_inputs), -1.0, 1.0)
    adj = helpers.uniform(61, 2, (n, spec.num_outputs), -1.0, 1.0)
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.1)
    x.tofile(tmp_path / "x.bin"); adj.tofile(tmp_path / "adj.bin"); params.astype(np.float32).tofile(tmp_path / "params.bin")
    r, out = _run(exe, "gpu", str(tmp_path / "spec.json"), str(tmp_path))
    assert r.returncode == 0 and "gpu ok" in r.stdout, r.stdout + r.stderr
    assert out["grad_view"] == "shared" and float(out["zeroed"]) == 0.0
    expected = oracle.network_forward(spec, params, x, half=True)
    inference = np.fromfile(tmp_path / "inference.bin", dtype=np.float32).reshape(n, -1)
    forward = np.fromfile(tmp_path / "forward.bin", dtype=np.float32).reshape(n, -1)
    helpers.assert_close(inference, expected, "inference through the C++ classes", max_violations=0.01)
    helpers.assert_close(forward, expected, "forward through the C++ classes", max_violations=0.01)
    g = oracle.network_backward(spec, params, x, adj, half=True, want_encodings=False)
    gi = np.fromfile(tmp_path / "adj_input.bin", dtype=np.float32).reshape(n, -1)
    gw = np.fromfile(tmp_path / "grad_params.bin", dtype=np.float32)
    helpers.assert_close(gi, g.adj_input, "input gradient through the C++ classes", rtol=5e-2,
                         atol=2e-2 * float(np.abs(g.adj_input).max()), max_violations=0.05)
    helpers.assert_close(gw, g.grad_params, "weight gradient through the C++ classes", rtol=helpers.RTOL_WGRAD,
                         atol=2e-2 * float(np.abs(g.grad_params).max()), max_violations=0.05)
