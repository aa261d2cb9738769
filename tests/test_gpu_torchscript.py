"""The stand-alone modules through torch.jit: trace, freeze, save, load, run — the sequence of the reference's
tests_py/qmlp_tests/test_activations.py:13-57 and tests_py/qmlp_tests/test_encoding.py:60-106 — plus their autograd
path against the torch modules the reference compares with."""
import json
import os

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs
from test_gpu_encoding_activation import encoding_cases
from test_gpu_network import LEAKY

pytestmark = pytest.mark.gpu


def _jit_round_trip(module, args, tmp_path):
    import torch
    module.eval()
    traced = torch.jit.trace(module, args)
    frozen = torch.jit.freeze(traced)
    path = os.path.join(str(tmp_path), "module.pt")
    torch.jit.save(frozen, path)
    loaded = torch.jit.load(path)
    return traced, loaded


@pytest.mark.parametrize("name", ["relu", "celu", "sine", "identity"])
def test_activation_module(name, tmp_path):
    import torch
    import qmlp
    act = qmlp.FusedActivation(name)
    baseline = qmlp.FusedActivation.get_activation(name)
    x = torch.from_numpy(helpers.uniform(3, 1, (257, 24), -2.0, 2.0)).cuda().half()
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    out, expected = act(xa), baseline(xb)
    assert out.dtype == torch.float16 and torch.allclose(out, expected, rtol=2e-3, atol=2e-3)
    g = torch.from_numpy(helpers.uniform(3, 2, (257, 24), -1.0, 1.0)).cuda().half()
    out.backward(g)
    expected.backward(g)
    assert torch.allclose(xa.grad, xb.grad, rtol=2e-3, atol=2e-3)
    traced, loaded = _jit_round_trip(act, (x,), tmp_path)
    assert "qmlp_b200::activation_forward" in str(traced.graph)
    assert torch.equal(loaded(x), out.detach())


def test_user_activation_module(tmp_path):
    import torch
    import qmlp
    act = qmlp.FusedActivation(json.dumps(LEAKY))
    x = torch.from_numpy(helpers.uniform(3, 3, (100, 8), -2.0, 2.0)).cuda().half()
    out = act(x)
    assert torch.allclose(out, torch.where(x > 0, x, x * 0.125), rtol=1e-3, atol=1e-3)
    _, loaded = _jit_round_trip(act, (x,), tmp_path)
    assert torch.equal(loaded(x), out)


@pytest.mark.parametrize("name", ["identity", "dense2d", "hash3d_f2", "hash4d_f4"])
def test_encoding_module(name, tmp_path):
    import torch
    import qmlp
    cfg = encoding_cases()[name]
    enc = qmlp.FusedEncoding(json.dumps(cfg))
    e = oracle.parse_encoding(cfg)
    lo = float(e.box_min.min()) if e.box_min is not None else -1.0
    hi = lo + (float((1.0 / e.box_inv_size).max()) if e.box_inv_size is not None else 2.0)
    x_np = helpers.uniform(5, 1, (300, enc.max_input_channel() + 1), lo, hi)
    x = torch.from_numpy(x_np).cuda()
    if enc.has_parameters():
        table_np = helpers.uniform(5, 2, (e.num_parameters,), -1.0, 1.0)
        table = torch.from_numpy(table_np).cuda().requires_grad_(True)
        args = (x, table)
        expected = oracle.grid_forward(e, x_np, table_np)
    else:
        table, args, expected = None, (x,), x_np[:, e.start_in:e.start_in + e.n_in]
    out = enc(*args)
    assert out.shape == (300, enc.num_output_channels()) and out.dtype == torch.float32
    if expected is not None:
        helpers.assert_close(out.detach().cpu().numpy(), expected, f"{name} module output", rtol=1e-4, atol=1e-5)
    if table is not None:     # gradients flow to the table through the registered autograd formula
        out.sum().backward()
        assert table.grad is not None and table.grad.shape == table.shape and float(table.grad.abs().sum()) > 0
    _, loaded = _jit_round_trip(enc, tuple(a.detach() for a in args), tmp_path)
    assert torch.equal(loaded(*[a.detach() for a in args]), out.detach())
