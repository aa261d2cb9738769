"""GPU parity of the stand-alone encoding and activation entry points, through the C ABI.
Follows the reference's tests_py/qmlp_tests/test_encoding.py:10-188 (identity, dense grid 1-D / 2-D against
torch grid_sample, output + input gradient + parameter gradient) and test_activations.py:8-66 (relu, sine against
torch, forward + gradient), and adds what the reference never pins: hashed levels, 3-D / 4-D grids."""
import json

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs

pytestmark = pytest.mark.gpu


def encoding_cases():
    return {
        "identity": {"id": "Identity", "start_in": 1, "n_in": 5},
        "dense1d": specs.hashgrid(1, 1, 4, -1, 2, 16, combination_mode="add", box_min=[-1], box_size=[2]),
        "dense2d": specs.hashgrid(2, 1, 4, -1, 2, 16, combination_mode="add", box_min=[-1, -1], box_size=[2, 2]),
        "dense2d_multires": specs.hashgrid(2, 5, 4, -1, 16, 256, combination_mode="concat"),
        "hash3d_f2": specs.hashgrid(3, 8, 2, 10, 4, 512, per_level_scale=2.0),
        "hash4d_f4": specs.hashgrid(4, 6, 4, 12, 4, 64),
        "hash3d_f3_add": specs.hashgrid(3, 4, 3, 9, 8, 128, combination_mode="add", start_in=2, box_min=[-2, -2, -2], box_size=[4, 4, 4]),
        "hash2d_f8": specs.hashgrid(2, 4, 8, 8, 8, 256),
        "dense6d": specs.hashgrid(6, 2, 1, -1, 2, 3),
        # ray start + direction in, the grid integrated along the ray out (src_cpp/src/encoding_line_integration.cpp)
        "line_average": {"id": "LineIntegration", "start_in": 1, "n_in": 3, "stepsize": 0.05, "blending": "average",
                         "volume": specs.hashgrid(3, 4, 2, 10, 4, 32)},
        "line_additive_add": {"id": "LineIntegration", "start_in": 0, "n_in": 3, "stepsize": 0.11, "blending": "additive",
                              "volume": specs.hashgrid(3, 3, 4, 9, 4, 24, combination_mode="add", box_min=[-1, -1, -1],
                                                       box_size=[2, 2, 2])},
    }


def _enc(name):
    from qmlp import bindings
    cfg = encoding_cases()[name]
    e = bindings.Encoding(json.dumps(cfg))
    oe = oracle.parse_encoding(cfg)
    return cfg, e, oe


@pytest.mark.parametrize("name", ["line_average", "line_additive_add"])
def test_line_integration(name):
    """Rays that start in and around the volume's bounding box, with arbitrary directions (some miss the box): output,
    table gradient and ray gradients against the oracle's restatement of encoding_line_integration.cuh:61-165."""
    import torch
    cfg, e, oe = _enc(name)
    n = 301
    bmin, bsize = float(cfg["volume"]["bounding_box_min"][0]), float(cfg["volume"]["bounding_box_size"][0])
    x = helpers.uniform(7, 1, (n, oe.start_in + 7), bmin - 0.4 * bsize, bmin + 1.4 * bsize)
    x[:, oe.start_in + 3:oe.start_in + 6] = helpers.uniform(7, 2, (n, 3), -1.0, 1.0)
    adj = helpers.uniform(7, 3, (n, oe.num_outputs), -1, 1)
    assert e.num_output_channels() == oe.num_outputs and e.max_input_channel() == oe.start_in + 5
    assert e.parameter_count() == oe.num_parameters and json.loads(e.to_json())["id"] == "LineIntegration"
    table = helpers.uniform(7, 4, (oe.num_parameters,), -1, 1)
    tx = torch.from_numpy(x).cuda().requires_grad_(True)
    tp = torch.from_numpy(table).cuda().requires_grad_(True)
    out = e.forward_with_parameter(tx, tp)
    expect = oracle.grid_forward(oe, x, table)
    assert float(np.abs(expect).sum(axis=1).min()) == 0.0 and float(np.abs(expect).max()) > 0.1   # misses and hits
    scale = float(np.abs(expect).max())
    helpers.assert_close(out.detach().cpu().numpy(), expect, f"{name} forward", rtol=1e-3, atol=1e-4 * scale, max_violations=0.01)
    out.backward(torch.from_numpy(adj).cuda())
    g, ai = oracle.grid_adjoint(oe, x, table, adj, True, True)
    helpers.assert_close(tp.grad.cpu().numpy(), g, f"{name} table gradient", rtol=1e-3, atol=1e-4 * float(np.abs(g).max()),
                         max_violations=0.01)
    helpers.assert_close(tx.grad.cpu().numpy(), ai, f"{name} ray gradient", rtol=2e-3, atol=1e-3 * float(np.abs(ai).max()),
                         max_violations=0.01)


@pytest.mark.parametrize("name", [k for k in encoding_cases() if not k.startswith("line_")])
def test_encoding_forward_and_adjoint(name):
    import torch
    cfg, e, oe = _enc(name)
    n = 257
    n_in = oe.start_in + oe.n_in + 1
    # 1 % beyond the bounding box on both sides: exercises the clamped cells without the ill-conditioned
    # extrapolation weights (|f| >> 1) that far-away points produce
    if oe.id == "Identity":
        lo, hi = -1.0, 1.0
    else:
        bmin, bsize = float(cfg["bounding_box_min"][0]), float(cfg["bounding_box_size"][0])
        lo, hi = bmin - 0.01 * bsize, bmin + 1.01 * bsize
    x = helpers.uniform(3, 1, (n, n_in), lo, hi)
    adj = helpers.uniform(3, 2, (n, oe.num_outputs), -1, 1)
    assert e.num_output_channels() == oe.num_outputs and e.max_input_channel() == oe.start_in + oe.n_in - 1
    tx = torch.from_numpy(x).cuda().requires_grad_(True)
    if oe.id == "Identity":
        out = e.forward(tx)
        assert torch.equal(out.detach().cpu(), torch.from_numpy(x[:, oe.start_in:oe.start_in + oe.n_in]))
        out.backward(torch.from_numpy(adj).cuda())
        expect = np.zeros_like(x); expect[:, oe.start_in:oe.start_in + oe.n_in] = adj
        assert np.array_equal(tx.grad.cpu().numpy(), expect)
        return
    assert e.parameter_count() == oe.num_parameters
    table = helpers.uniform(3, 3, (oe.num_parameters,), -1, 1)
    tp = torch.from_numpy(table).cuda().requires_grad_(True)
    out = e.forward_with_parameter(tx, tp)
    expect = oracle.grid_forward(oe, x, table)
    # fp32 blend on both sides: only summation order and fma contraction differ
    helpers.assert_close(out.detach().cpu().numpy(), expect, f"{name} forward", rtol=1e-4, atol=1e-4)
    out.backward(torch.from_numpy(adj).cuda())
    g, ai = oracle.grid_adjoint(oe, x, table, adj, True, True)
    helpers.assert_close(tp.grad.cpu().numpy(), g, f"{name} parameter gradient", rtol=1e-4, atol=1e-4)
    helpers.assert_close(tx.grad.cpu().numpy(), ai, f"{name} input gradient", rtol=1e-3, atol=1e-3)


def test_grid_indices_bit_exact():
    """One-hot tables turn the gather into an index probe: with table[i] = i (exactly representable) and points on
    cell corners, the output IS the row index, so dense and hashed indices can be compared for equality."""
    import torch
    from qmlp import bindings
    for cfg in (specs.hashgrid(3, 6, 1, 14, 8, 300), specs.hashgrid(4, 4, 1, 16, 8, 64), specs.hashgrid(2, 5, 1, -1, 4, 64)):
        e = bindings.Encoding(json.dumps(cfg))
        oe = oracle.parse_encoding(cfg)
        n = 500
        for li, lv in enumerate(oe.levels):
            # integer cell coordinates in [0, res-2] -> positions exactly on the low corner: weight 1 on one corner
            cells = (helpers.uniform(9, 10 + li, (n, oe.n_in)) * (lv.resolution - 1)).astype(np.int64)
            x = (cells.astype(np.float64) / (lv.resolution - 1)).astype(np.float32)
            iL, iH, f = oracle.grid_cell(oe, lv, x)
            rows = oracle.grid_index(oe, lv, iL)          # element index of the low corner
            level_size = (lv.hash_grid_size if lv.hashed else lv.resolution ** oe.n_in)
            table = np.zeros(oe.num_parameters, dtype=np.float32)
            table[lv.memory_offset:lv.memory_offset + level_size] = np.arange(level_size, dtype=np.float32)
            out = e.inference_with_parameter(torch.from_numpy(x).cuda(), torch.from_numpy(table).cuda()).cpu().numpy()
            exact = f.max(axis=1) == 0                     # points whose fraction is exactly zero
            assert exact.sum() > n // 4
            got = out[exact, li]
            want = (rows[exact] - lv.memory_offset).astype(np.float32)
            assert np.array_equal(got, want), f"level {li}: index mismatch"


def test_dense_grid_matches_grid_sample():
    """The reference's own check (tests_py/qmlp_tests/test_encoding.py:143-188): a dense level equals
    grid_sample(align_corners=True, padding_mode='border')."""
    import torch
    cfg, e, oe = _enc("dense2d")
    r, c, n = 2, 4, 64
    x = torch.from_numpy(helpers.uniform(5, 1, (n, 2), -1, 1)).cuda()
    p = torch.from_numpy(helpers.uniform(5, 2, (r * r * c,), -1, 1)).cuda()
    out = e.inference_with_parameter(x, p)
    inp = p.reshape(1, r, r, c).permute((0, 3, 2, 1))
    ref = torch.nn.functional.grid_sample(inp, x.reshape(1, -1, 1, 2), mode="bilinear", align_corners=True,
                                          padding_mode="border")[0, :, :, 0].t()
    assert torch.allclose(out, ref, atol=1e-6)


@pytest.mark.parametrize("name", ["relu", "celu", "sine", "identity", "leaky"])
def test_activation(name):
    import torch
    from qmlp import bindings
    leaky = {"id": "leaky", "forward": "z = __hgt(x, hZERO()) ? x : __hmul(x, __float2half(0.125f))",
             "adjoint": "adjx = __hgt(x, hZERO()) ? adjz : __hmul(adjz, __float2half(0.125f))"}
    act = bindings.Activation(json.dumps(leaky) if name == "leaky" else name)
    assert act.id() == name
    fn = {"relu": torch.relu, "celu": torch.nn.functional.celu, "sine": torch.sin, "identity": lambda t: t,
          "leaky": lambda t: torch.nn.functional.leaky_relu(t, 0.125)}[name]
    for shape, strided in (((8, 6), False), ((37, 5), False), ((16, 8), True)):
        x = torch.from_numpy(helpers.uniform(1, 1, shape, -3, 3)).cuda().half()
        g = torch.from_numpy(helpers.uniform(1, 2, shape, -1, 1)).cuda().half()
        if strided:
            x = x.t().contiguous().t()
        xa = x.clone().requires_grad_(True)
        out = act.forward(xa)
        out.backward(g)
        xr = x.float().clone().requires_grad_(True)
        ref = fn(xr)
        ref.backward(g.float())
        assert torch.allclose(out.float(), ref, rtol=2e-3, atol=2e-3)
        assert torch.allclose(xa.grad.float(), xr.grad, rtol=2e-3, atol=2e-3)


def test_encoding_errors():
    import torch
    from qmlp import bindings
    from qmlp._capi import QmlpError
    with pytest.raises(QmlpError):
        bindings.Encoding(json.dumps({"id": "Nope", "start_in": 0, "n_in": 1}))
    with pytest.raises(QmlpError):
        bindings.Encoding(json.dumps(specs.hashgrid(7, 1, 1, -1, 2, 2)))      # dimension must be in [1, 6]
    cfg, e, oe = _enc("dense2d")
    with pytest.raises(QmlpError):
        e.inference_with_parameter(torch.zeros((4, 2), device="cuda"), torch.zeros((3,), device="cuda"))  # wrong size
