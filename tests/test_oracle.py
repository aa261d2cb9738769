"""Pins the CPU oracle (oracle/qmlp_oracle.py and its C++ twin oracle/cpu_ref.cpp) against the committed golden
fixtures: the reference's own SimulatedNetwork (fp32), torch grid_sample for dense grids, torch activations.
No GPU needed."""
import json

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs


def _mlp_cases():
    g = helpers.load_golden("mlp_reference_simulated.npz")
    return g, json.loads(str(g["cases"]))


@pytest.mark.parametrize("name", ["ref_16_32_16", "ref_48_16_32_48", "uneven_19_16_16", "uneven_20_16_24", "config1", "config2"])
def test_mlp_matches_reference_simulated_network(name):
    g, cases = _mlp_cases()
    cfg = cases[name]
    spec = oracle.parse_spec(cfg)
    nl = len(spec.layers)
    weights = [g[f"{name}/w{i}"] for i in range(nl)]
    biases = [g[f"{name}/b{i}"] if f"{name}/b{i}" in g else None for i in range(nl)]
    params = helpers.pack_parameters(spec, weights, biases)
    x, adj = g[f"{name}/x"], g[f"{name}/adj"]
    y = oracle.network_forward(spec, params, x)
    np.testing.assert_allclose(y, g[f"{name}/y"], rtol=1e-5, atol=1e-6)
    grads = oracle.network_backward(spec, params, x, adj)
    np.testing.assert_allclose(grads.output, g[f"{name}/y"], rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(grads.adj_input, g[f"{name}/dx"], rtol=1e-4, atol=1e-5)
    for i, l in enumerate(spec.layers):
        gw = oracle.weight_view(spec, grads.grad_params, i)
        n_out, n_in = weights[i].shape
        np.testing.assert_allclose(gw[:n_out, :n_in], g[f"{name}/dw{i}"], rtol=1e-4, atol=1e-5)
        if biases[i] is not None:
            np.testing.assert_allclose(oracle.bias_view(spec, grads.grad_params, i)[:n_out], g[f"{name}/db{i}"], rtol=1e-4, atol=1e-5)
        # padding rows/columns receive exactly zero gradient when the padding weights are zero
        assert np.all(gw[n_out:, :n_in] == 0) or l.activation in ("celu", "sine", "identity")


@pytest.mark.parametrize("name", ["d1_r2", "d2_r2", "d2_r8", "d3_r5"])
def test_dense_grid_matches_grid_sample(name):
    g = helpers.load_golden("dense_grid_torch.npz")
    d, r, c = (int(v) for v in g[f"{name}/meta"])
    enc = oracle.parse_encoding(specs.hashgrid(d, 1, c, -1, r, 16, combination_mode="add", box_min=[-1.0] * d, box_size=[2.0] * d))
    assert enc.num_parameters == r ** d * c and not enc.levels[0].hashed
    x, p, adj = g[f"{name}/x"], g[f"{name}/p"], g[f"{name}/adj"]
    np.testing.assert_allclose(oracle.grid_forward(enc, x, p), g[f"{name}/y"], rtol=1e-5, atol=1e-6)
    gp, gx = oracle.grid_adjoint(enc, x, p, adj, True, True)
    np.testing.assert_allclose(gp, g[f"{name}/dp"], rtol=1e-4, atol=1e-5)
    # grid_sample differentiates with respect to the normalised coordinate in [-1, 1]: d/dx = (r-1)/2 * d/dcell,
    # the factor this oracle carries and the reference kernel omits (exact only for r = 2, its tested case)
    np.testing.assert_allclose(gx, g[f"{name}/dx"], rtol=1e-3, atol=1e-4)
    if r == 2:
        _, gq = oracle.grid_adjoint(enc, x, p, adj, False, True, reference_input_grad_quirk=True)
        np.testing.assert_allclose(gq, g[f"{name}/dx"], rtol=1e-3, atol=1e-4)


def test_activations_match_torch():
    g = helpers.load_golden("activations_torch.npz")
    for name in ("relu", "celu", "sine", "identity"):
        a = oracle.ACTIVATIONS[name]
        np.testing.assert_allclose(a.forward(g["x"]), g[f"{name}/y"], rtol=1e-6, atol=1e-7)
        np.testing.assert_allclose(a.adjoint(g["x"], g["g"]), g[f"{name}/dx"], rtol=1e-6, atol=1e-7)


def test_padding_and_layout_rules():
    """src_cpp/src/fused_network.cpp:146-206 on the reference's uneven test shapes (test_against_eigen2.cpp:17-46)."""
    s = oracle.parse_spec(specs.identity_net(19, [16, 16], ["identity", "identity"], bias=False))
    assert [(l.channels_in, l.channels_out) for l in s.layers] == [(32, 16), (16, 16)]
    s = oracle.parse_spec(specs.identity_net(16, [16, 23], ["identity", "identity"], bias=False))
    assert [(l.channels_in, l.channels_out) for l in s.layers] == [(16, 16), (16, 32)]
    s = oracle.parse_spec(specs.identity_net(20, [17, 24], ["identity", "identity"], bias=[True, True]))
    assert [(l.channels_in, l.channels_out) for l in s.layers] == [(32, 32), (32, 32)]      # hidden 17 -> 32 on both sides
    assert [l.weights_start for l in s.layers] == [0, 1024] and [l.bias_start for l in s.layers] == [2048, 2080]
    assert s.num_parameters == 2112
    # parameter counts of the five benchmark configurations
    counts = [oracle.parse_spec(c).num_parameters for c in (specs.config1(), specs.config2(), specs.config3(), specs.config4(), specs.config5())]
    assert counts == [512, 14608, 7312, 15840, 43408]


def test_level_tables():
    """Level tables of the benchmark grids (double-precision exp/log/pow/floor, src_cpp/src/encoding_hashgrid.cpp:64-96)."""
    lv, n = oracle.grid_levels(4, 16, 4, 22, 16, 2489)
    assert [l.resolution for l in lv] == [16, 22, 31, 43, 61, 86, 120, 168, 236, 330, 462, 647, 907, 1269, 1777, 2489]
    assert [l.hashed for l in lv] == [False] * 4 + [True] * 12 and n == 219895048
    lv, n = oracle.grid_levels(3, 16, 2, 19, 16, 7006, 1.5)
    assert [l.resolution for l in lv] == [16, 24, 36, 54, 81, 121, 182, 273, 410, 615, 922, 1383, 2075, 3113, 4670, 7006]
    assert n == 13026992
    lv, n = oracle.grid_levels(3, 8, 4, 18, 32, 4096)            # reference formula alone: one ulp below 2
    assert [l.resolution for l in lv] == [32, 63, 127, 255, 511, 1023, 2047, 4095]
    lv, n = oracle.grid_levels(3, 8, 4, 18, 32, 4096, 2.0)       # extension key per_level_scale
    assert [l.resolution for l in lv] == [32, 64, 128, 256, 512, 1024, 2048, 4096] and n == 7471104


def test_hash_index_known_values():
    """Hand-computed hashed indices: xor of coordinate*prime in uint32, mod table size
    (src_cpp/include/qmlp/kernels/encoding_hashgrid.cuh:18-24,42-46,76)."""
    enc = oracle.parse_encoding(specs.hashgrid(3, 1, 1, 4, 100, 100))
    lv = enc.levels[0]
    assert lv.hashed and lv.hash_grid_size == 16
    ipos = np.array([[1, 2, 3], [99, 98, 97], [0, 0, 0]], dtype=np.uint32)
    want = []
    for a, b, c in ipos.tolist():
        h = ((a * 1) & 0xffffffff) ^ ((b * 43857811) & 0xffffffff) ^ ((c * 83857661) & 0xffffffff)
        want.append(h % 16)
    assert oracle.grid_index(enc, lv, ipos).tolist() == want
    dense = oracle.parse_encoding(specs.hashgrid(3, 1, 2, -1, 5, 5))
    assert oracle.grid_index(dense, dense.levels[0], np.array([[1, 2, 3]], dtype=np.uint32)).tolist() == [((1 * 5 + 2) * 5 + 3) * 2]


@pytest.mark.parametrize("cfg", [specs.config2(), specs.config3(10), specs.config4(9, 8), specs.config5(10)])
def test_cpp_restatement_matches_numpy_oracle(cfg):
    import cpu_ref
    spec = oracle.parse_spec(cfg)
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.1)
    tables = helpers.grid_tables(spec)
    # inside the bounding box: outside it the fine levels extrapolate with weights |f| >> 1 and amplify fp32 rounding
    x = helpers.uniform(3, 1, (515, spec.num_inputs), 0.0, 1.0)
    a = oracle.network_forward(spec, params, x, tables)
    b = cpu_ref.CpuNetwork(spec, params, tables).forward(x)
    np.testing.assert_allclose(b, a, rtol=1e-4, atol=1e-5)
    c = cpu_ref.CpuNetwork(spec, params, tables).forward(x, threads=1)
    np.testing.assert_array_equal(b, c)


@pytest.mark.parametrize("cfg", [specs.config2(), specs.config3(10), specs.config4(9, 8)])
def test_cpp_training_step_matches_numpy_oracle(cfg):
    """oracle_network_train_step (the CPU leg of the benchmark's training workloads): loss, weight / bias / table
    gradients against network_backward, and two Adam steps against adam_step."""
    import cpu_ref
    spec = oracle.parse_spec(cfg)
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.1).astype(np.float32)
    tables = helpers.grid_tables(spec, scale=0.1)
    x = helpers.uniform(3, 1, (777, spec.num_inputs), 0.0, 1.0)
    target = helpers.uniform(3, 2, (777, spec.num_outputs), -1.0, 1.0)
    net = cpu_ref.CpuNetwork(spec, params, tables)
    loss = net.train_step(x, target, update=False)
    out = oracle.network_forward(spec, params, x, tables)
    g = oracle.network_backward(spec, params, x, oracle.mse_loss_grad(out, target), tables, want_input=False)
    np.testing.assert_allclose(loss, float(((out - target) ** 2).sum()), rtol=1e-5)
    gp, gt = net.gradients()
    np.testing.assert_allclose(gp, g.grad_params, rtol=1e-3, atol=1e-6 * float(np.abs(g.grad_params).max()) + 1e-9)
    for a, b in zip(gt, g.grad_encodings):
        if b is not None:
            np.testing.assert_allclose(a, b, rtol=1e-3, atol=1e-5 * float(np.abs(b).max()))
    # two full steps: the moments carry over, the gradients are cleared in between
    net.zero_gradients()
    p, m, v = params.copy(), np.zeros_like(params), np.zeros_like(params)
    tabs = [t.copy() if t is not None else None for t in tables]
    tm = [np.zeros_like(t) if t is not None else None for t in tables]
    tv = [np.zeros_like(t) if t is not None else None for t in tables]
    for step in (1, 2):
        net.train_step(x, target)
        o = oracle.network_forward(spec, p, x, tabs)
        gg = oracle.network_backward(spec, p, x, oracle.mse_loss_grad(o, target), tabs, want_input=False)
        oracle.adam_step(p, gg.grad_params, m, v, step)
        for i, t in enumerate(tabs):
            if t is not None:
                oracle.adam_step(t, gg.grad_encodings[i], tm[i], tv[i], step)
    # Adam divides by sqrt(v): entries whose gradient is rounding noise move by about the learning rate in either
    # direction, so the comparison allows a small fraction of them
    helpers.assert_close(net.params - params, p - params, "network parameters after two steps", rtol=2e-2, atol=2e-4,
                         max_violations=0.02)
    for a, b, t0 in zip(net.tables, tabs, tables):
        if b is not None:
            helpers.assert_close(a - t0, b - t0, "table after two steps", rtol=2e-2, atol=2e-4, max_violations=0.02)


def test_adam_matches_torch():
    import torch
    rng = np.random.default_rng(0)
    p0 = rng.normal(size=1000).astype(np.float32)
    tp = torch.nn.Parameter(torch.from_numpy(p0.copy()))
    opt = torch.optim.Adam([tp], lr=1e-2)
    p, m, v = p0.copy(), np.zeros_like(p0), np.zeros_like(p0)
    for step in range(1, 6):
        g = rng.normal(size=1000).astype(np.float32) * 10 ** rng.uniform(-6, 0, size=1000).astype(np.float32)
        tp.grad = torch.from_numpy(g.copy())
        opt.step()
        oracle.adam_step(p, g, m, v, step)
    np.testing.assert_allclose(p, tp.detach().numpy(), rtol=1e-5, atol=1e-6)


def test_empty_and_single_point():
    spec = oracle.parse_spec(specs.config1())
    params = helpers.reference_style_parameters(spec)
    assert oracle.network_forward(spec, params, np.zeros((0, 3), np.float32)).shape == (0, 1)
    assert oracle.network_forward(spec, params, np.full((1, 3), 0.5, np.float32)).shape == (1, 1)
