"""Generates the golden fixtures in this directory. Run in a checkout where the reference sources are available:

    python tests/golden/make_golden.py /path/to/quick-mlp

1. mlp_reference_simulated.npz - outputs and gradients of the reference's own plain-PyTorch network
   (class SimulatedNetwork, src_py/qmlp/network.py:161-243, imported from the reference checkout and run in fp32 on the
   CPU), the object the reference's tests compare its fused kernels against (tests_py/qmlp_tests/test_network_base.py).
2. dense_grid_torch.npz - dense-grid levels against torch.nn.functional.grid_sample(align_corners=True,
   padding_mode='border'), the reference's check for its grid encoding (tests_py/qmlp_tests/test_encoding.py:108-188),
   extended to resolution 8 and to 3-D.
3. activations_torch.npz - relu / celu / sin and their gradients from torch (tests_py/qmlp_tests/test_activations.py).

Inputs come from a fixed numpy generator; everything is float32. The fixtures are small (< 200 KB).
"""
import json
import os
import sys
import types
import zlib

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def import_reference_simulated_network(ref_root):
    """Imports src_py/qmlp/network.py from the reference without its native library: the modules that load the
    binaries (import_library, encoding) are replaced by stubs; SimulatedNetwork itself is pure PyTorch."""
    pkg_dir = os.path.join(ref_root, "src_py", "qmlp")
    tt = types.ModuleType("torchtyping")

    class _TensorType:
        def __class_getitem__(cls, item):
            return torch.Tensor
    tt.TensorType = _TensorType
    sys.modules["torchtyping"] = tt
    pkg = types.ModuleType("qmlp_reference")
    pkg.__path__ = [pkg_dir]
    sys.modules["qmlp_reference"] = pkg
    il = types.ModuleType("qmlp_reference.import_library")
    il.load_library = lambda: None
    sys.modules["qmlp_reference.import_library"] = il
    enc = types.ModuleType("qmlp_reference.encoding")
    enc.FusedEncoding = object
    sys.modules["qmlp_reference.encoding"] = enc
    import importlib
    net = importlib.import_module("qmlp_reference.network")
    return net.SimulatedNetwork


def identity_cfg(n_in, widths, acts, bias):
    return {"num_inputs": n_in, "num_outputs": widths[-1], "activation_specification": ["qmlp/builtin-activations.json"],
            "encodings": [{"id": "Identity", "start_in": 0, "n_in": n_in}],
            "network": [{"n_out": w, "bias": b, "activation": a} for w, a, b in zip(widths, acts, bias)]}


MLP_CASES = {
    # the reference's own test shapes (test_network_base.py:150-256: widths 16/32/48, celu/identity, no bias) ...
    "ref_16_32_16": identity_cfg(16, [32, 16], ["celu", "celu"], [False, False]),
    "ref_48_16_32_48": identity_cfg(48, [16, 32, 48], ["identity", "celu", "identity"], [False, False, False]),
    # ... uneven widths as tests_cpp/test_against_eigen2.cpp:17-46 (19->16->16, 16->16->23, 20->16->24) ...
    "uneven_19_16_16": identity_cfg(19, [16, 16], ["identity", "identity"], [False, False]),
    "uneven_20_16_24": identity_cfg(20, [16, 24], ["relu", "sine"], [False, False]),
    # ... and what the benchmark configurations add: bias, relu/sine, 64 wide
    "config1": identity_cfg(3, [16, 1], ["relu", "relu"], [False, False]),
    "config2": identity_cfg(3, [64, 64, 64, 64, 1], ["relu", "celu", "sine", "relu", "identity"], [True] * 5),
}


def make_mlp(ref_root):
    Sim = import_reference_simulated_network(ref_root)
    rng = np.random.default_rng(20240601)
    out = {"cases": json.dumps(MLP_CASES)}
    for name, cfg in MLP_CASES.items():
        torch.manual_seed(zlib.crc32(name.encode()))
        net = Sim(json.dumps(cfg), weight_dtype=torch.float32)
        n = 37
        lo = 0.0 if name == "config1" else -1.0
        x = torch.from_numpy(rng.uniform(lo, 1.0, size=(n, cfg["num_inputs"])).astype(np.float32)).requires_grad_(True)
        adj = torch.from_numpy(rng.uniform(-1.0, 1.0, size=(n, cfg["num_outputs"])).astype(np.float32))
        y = net(x)
        y.backward(adj)
        out[f"{name}/x"] = x.detach().numpy()
        out[f"{name}/adj"] = adj.numpy()
        out[f"{name}/y"] = y.detach().numpy()
        out[f"{name}/dx"] = x.grad.numpy()
        for i in range(net.num_layers()):
            out[f"{name}/w{i}"] = net.get_weight(i, False, False).numpy()
            out[f"{name}/dw{i}"] = net.get_weight(i, False, True).numpy()
            if net.has_bias(i):
                out[f"{name}/b{i}"] = net.get_weight(i, True, False).numpy()
                out[f"{name}/db{i}"] = net.get_weight(i, True, True).numpy()
    np.savez_compressed(os.path.join(HERE, "mlp_reference_simulated.npz"), **out)


def make_grid():
    rng = np.random.default_rng(7)
    F = torch.nn.functional
    out = {}
    for name, d, r, c in (("d1_r2", 1, 2, 4), ("d2_r2", 2, 2, 4), ("d2_r8", 2, 8, 3), ("d3_r5", 3, 5, 2)):
        n = 40
        x = torch.from_numpy(rng.uniform(-1.0, 1.0, size=(n, d)).astype(np.float32)).requires_grad_(True)
        p = torch.from_numpy(rng.uniform(-1.0, 1.0, size=(r ** d * c,)).astype(np.float32)).requires_grad_(True)
        adj = torch.from_numpy(rng.uniform(-1.0, 1.0, size=(n, c)).astype(np.float32))
        if d == 1:     # test_encoding.py:124-141
            inp = p.reshape(1, r, 1, c).permute((0, 3, 2, 1))
            grid = torch.cat([x.reshape(1, -1, 1, 1), torch.zeros(1, n, 1, 1)], dim=3)
            y = F.grid_sample(inp, grid, mode="bilinear", align_corners=True, padding_mode="border")[0, :, :, 0].t()
        elif d == 2:   # test_encoding.py:158-186
            inp = p.reshape(1, r, r, c).permute((0, 3, 2, 1))
            y = F.grid_sample(inp, x.reshape(1, -1, 1, 2), mode="bilinear", align_corners=True, padding_mode="border")[0, :, :, 0].t()
        else:          # table index = x2 + r*(x1 + r*x0): (x0, x1, x2, c) -> (N, C, D=x2, H=x1, W=x0)
            inp = p.reshape(1, r, r, r, c).permute((0, 4, 3, 2, 1))
            y = F.grid_sample(inp, x.reshape(1, -1, 1, 1, 3), mode="bilinear", align_corners=True, padding_mode="border")[0, :, :, 0, 0].t()
        y.backward(adj)
        out[f"{name}/meta"] = np.array([d, r, c])
        out[f"{name}/x"], out[f"{name}/p"], out[f"{name}/adj"] = x.detach().numpy(), p.detach().numpy(), adj.numpy()
        out[f"{name}/y"], out[f"{name}/dx"], out[f"{name}/dp"] = y.detach().numpy(), x.grad.numpy(), p.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "dense_grid_torch.npz"), **out)


def make_activations():
    rng = np.random.default_rng(11)
    x = torch.from_numpy(rng.uniform(-4.0, 4.0, size=(64,)).astype(np.float32))
    g = torch.from_numpy(rng.uniform(-1.0, 1.0, size=(64,)).astype(np.float32))
    out = {"x": x.numpy(), "g": g.numpy()}
    for name, fn in (("relu", torch.relu), ("celu", torch.nn.functional.celu), ("sine", torch.sin), ("identity", lambda t: t * 1.0)):
        xx = x.clone().requires_grad_(True)
        y = fn(xx)
        y.backward(g)
        out[f"{name}/y"], out[f"{name}/dx"] = y.detach().numpy(), xx.grad.numpy()
    np.savez_compressed(os.path.join(HERE, "activations_torch.npz"), **out)


if __name__ == "__main__":
    # the reference checkout: first argument, else a directory "reference" beside this repository
    ref = sys.argv[1] if len(sys.argv) > 1 else os.path.normpath(os.path.join(HERE, os.pardir, os.pardir, os.pardir, "reference"))
    make_mlp(ref)
    make_grid()
    make_activations()
    print("fixtures written to", HERE)
