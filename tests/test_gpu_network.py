"""GPU parity of the fused network path (inference, forward-with-stash, adjoint, weight/bias/grid gradients) against
the CPU oracle, called through the C ABI. Mirrors the structure of the reference's
tests_py/qmlp_tests/test_network_base.py:87-147 (fused vs simulated network: inference, forward, input gradients,
parameter gradients at several batch sizes) and tests_cpp/test_against_eigen2.cpp (uneven widths, all-gradient modes).
"""
import json

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs

pytestmark = pytest.mark.gpu

LEAKY = {"id": "leaky", "forward": "z = __hgt(x, hZERO()) ? x : __hmul(x, __float2half(0.125f))",
         "adjoint": "adjx = __hgt(x, hZERO()) ? adjz : __hmul(adjz, __float2half(0.125f))"}


def _leaky_oracle():
    acts = dict(oracle.ACTIVATIONS)
    acts["leaky"] = oracle.OracleActivation(lambda x: np.where(x > 0, x, 0.125 * x).astype(x.dtype),
                                            lambda x, g: np.where(x > 0, g, 0.125 * g).astype(g.dtype))
    return acts


def network_cases():
    """name -> (cfg, input range, parameter style)"""
    return {
        "config1": (specs.config1(), (0.0, 1.0), "reference"),
        "config2": (specs.config2(), (-1.0, 1.0), "xavier"),
        "ref_widths": (specs.identity_net(16, [32, 48, 16], ["celu", "identity", "celu"], bias=False), (-1.0, 1.0), "reference"),
        "uneven": (specs.identity_net(5, [20, 23, 7], ["sine", "relu", "identity"], bias=[True, False, True]), (-1.0, 1.0), "reference"),
        "custom_act": (specs.identity_net(4, [32, 32, 2], ["leaky", "sine", "leaky"], bias=True, extra_activations=[LEAKY]), (-1.0, 1.0), "reference"),
        "config3_small": (specs.config3(log2_hashmap_size=12), (0.0, 1.0), "xavier"),
        "config4_small": (specs.config4(log2_hashmap_size=10, dense_resolution=16), (0.0, 1.0), "xavier"),
        "config5_small": (specs.config5(log2_hashmap_size=12), (0.0, 1.0), "xavier"),
        "grid2d_add_plus_identity": (
            {"num_inputs": 4, "num_outputs": 3, "activation_specification": specs.BUILTIN,
             "encodings": [specs.hashgrid(2, 4, 4, 8, 4, 64, combination_mode="add", start_in=1, box_min=[-1, -1], box_size=[2, 2]),
                           {"id": "Identity", "start_in": 0, "n_in": 4}],
             "network": specs.mlp([32, 3], ["celu", "identity"], True)}, (-1.0, 1.0), "reference"),
    }


def _setup(name):
    import torch
    from qmlp import bindings
    cfg, rng, style = network_cases()[name]
    spec = oracle.parse_spec(cfg)
    net = bindings.Network(json.dumps(cfg))
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.1) if style == "xavier" else helpers.reference_style_parameters(spec)
    tables = helpers.grid_tables(spec, scale=1.0)
    acts = _leaky_oracle()
    dev = torch.device("cuda")
    t_params = torch.from_numpy(params).to(dev)
    t_tables = [torch.from_numpy(t).to(dev) if t is not None else None for t in tables]
    return cfg, rng, spec, net, params, tables, acts, t_params, t_tables


@pytest.mark.parametrize("name", list(network_cases().keys()))
def test_spec_layout_matches_oracle(name):
    cfg, rng, spec, net, *_ = _setup(name)
    assert net.num_network_parameters() == spec.num_parameters
    assert net.num_layers() == len(spec.layers)
    for i, l in enumerate(spec.layers):
        cin, cout, bias, ws, bs = net.layer_info(i)
        assert (cin, cout, bias, ws) == (l.channels_in, l.channels_out, l.use_bias, l.weights_start)
        if l.use_bias:
            assert bs == l.bias_start
    for i, e in enumerate(spec.encodings):
        enc = net.encoding(i)
        assert enc.num_output_channels() == e.num_outputs
        assert enc.parameter_count() == e.num_parameters
        assert enc.grid_levels() == [(lv.memory_offset, lv.resolution, lv.hash_grid_size, lv.hashed) for lv in e.levels]


@pytest.mark.parametrize("name", list(network_cases().keys()))
@pytest.mark.parametrize("n", [1, 33, 1000])
def test_inference(name, n):
    import torch
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup(name)
    x = helpers.uniform(42, 1, (n, spec.num_inputs), *rng)
    out = net.inference(torch.from_numpy(x).cuda(), t_params, t_tables).cpu().numpy()
    emu = oracle.network_forward(spec, params, x, tables, half=True, activations=acts)
    ref = oracle.network_forward(spec, params, x, tables, half=False, activations=acts)
    assert np.isfinite(out).all()
    helpers.assert_close(out, emu, f"{name} inference vs fp16-emulating oracle", max_violations=0.01)
    helpers.assert_close(out, ref, f"{name} inference vs fp32 oracle", max_violations=helpers.MAX_VIOLATIONS)


def test_inference_half_tables_and_strided_io():
    """fp16 gather table (extension) and non-contiguous input/output views."""
    import torch
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup("config3_small")
    n = 777
    x = helpers.uniform(42, 2, (n, spec.num_inputs), *rng)
    wide = torch.zeros((n, 8), device="cuda")
    wide[:, 2:5] = torch.from_numpy(x).cuda()
    half_tables = [t.half() if t is not None else None for t in t_tables]
    out = net.inference(wide[:, 2:5], t_params, half_tables).cpu().numpy()
    tables16 = [t.astype(np.float16).astype(np.float32) if t is not None else None for t in tables]
    emu = oracle.network_forward(spec, params, x, tables16, half=True)
    helpers.assert_close(out, emu, "fp16 table inference", max_violations=0.01)


@pytest.mark.parametrize("name", list(network_cases().keys()))
@pytest.mark.parametrize("n", [32, 513])
def test_forward_and_adjoint(name, n):
    """forward with stash, then the adjoint in every flag combination the reference exercises
    (input only, weights only, everything: tests_cpp/test_against_eigen2.cpp:216-284)."""
    import torch
    from qmlp import _capi
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup(name)
    x = helpers.uniform(42, 3, (n, spec.num_inputs), *rng)
    adj = helpers.uniform(42, 4, (n, spec.num_outputs), -1.0, 1.0)
    g = oracle.network_backward(spec, params, x, adj, tables, half=True, activations=acts)
    g32 = oracle.network_backward(spec, params, x, adj, tables, half=False, activations=acts)

    tx = torch.from_numpy(x).cuda().requires_grad_(True)
    tp = t_params.float().requires_grad_(True)   # fp32 master, cast to half per call like the reference binding
    tt = [t.clone().requires_grad_(True) if t is not None else None for t in t_tables]
    out = net.forward(tx, tp, tt)
    helpers.assert_close(out.detach().cpu().numpy(), g.output, f"{name} forward", max_violations=0.01)
    out.backward(torch.from_numpy(adj).cuda())
    torch.cuda.synchronize()

    # The position gradient of a fine grid level carries the factor (resolution - 1): entries reach 1e3 and an
    # activation-derivative flip caused by one fp16 ulp upstream moves them by O(100). The absolute floor therefore
    # scales with the tensor, and the reference's 5 % allowance for entries outside applies.
    in_scale = max(1.0, float(np.abs(g.adj_input).max()))
    helpers.assert_close(tx.grad.cpu().numpy(), g.adj_input, f"{name} input gradient (emulated)", atol=1e-3 * in_scale,
                         max_violations=helpers.MAX_VIOLATIONS)
    helpers.assert_close(tx.grad.cpu().numpy(), g32.adj_input, f"{name} input gradient (fp32)", atol=1e-3 * in_scale,
                         max_violations=2 * helpers.MAX_VIOLATIONS if in_scale > 10 else helpers.MAX_VIOLATIONS)
    scale = max(1.0, float(np.abs(g.grad_params).max()))
    helpers.assert_close(tp.grad.cpu().numpy() / scale, g.grad_params / scale, f"{name} weight+bias gradient (emulated)",
                         max_violations=0.02)
    helpers.assert_close(tp.grad.cpu().numpy(), g32.grad_params, f"{name} weight+bias gradient (fp32)",
                         rtol=helpers.RTOL_WGRAD, atol=1e-3 * scale, max_violations=helpers.MAX_VIOLATIONS)
    for i, e in enumerate(spec.encodings):
        if e.num_parameters:
            helpers.assert_close(tt[i].grad.cpu().numpy(), g.grad_encodings[i], f"{name} grid gradient (emulated)",
                                 max_violations=0.02)
            helpers.assert_close(tt[i].grad.cpu().numpy(), g32.grad_encodings[i], f"{name} grid gradient (fp32)",
                                 max_violations=helpers.MAX_VIOLATIONS)

    # single-flag variants must reproduce the same numbers
    tx2 = torch.from_numpy(x).cuda().requires_grad_(True)
    out2 = net.forward(tx2, t_params, t_tables)
    out2.backward(torch.from_numpy(adj).cuda())
    helpers.assert_close(tx2.grad.cpu().numpy(), tx.grad.cpu().numpy(), f"{name} input-only variant", rtol=1e-3, atol=1e-4 * in_scale)
    tp3 = t_params.float().requires_grad_(True)
    out3 = net.forward(torch.from_numpy(x).cuda(), tp3, t_tables)
    out3.backward(torch.from_numpy(adj).cuda())
    helpers.assert_close(tp3.grad.cpu().numpy() / scale, tp.grad.cpu().numpy() / scale, f"{name} weights-only variant", atol=1e-4)


def test_gradients_accumulate():
    """adjoint adds to the bound gradient tensors (reference: outAdjWeights[i] += ..., callers zero them)."""
    import ctypes as C
    import torch
    from qmlp import _capi
    from qmlp._capi import check, lib, wrap
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup("config1")
    n = 200
    x = torch.from_numpy(helpers.uniform(1, 5, (n, 3))).cuda()
    adj = torch.from_numpy(helpers.uniform(1, 6, (n, 1), -1, 1)).cuda()
    out = torch.empty((n, 1), device="cuda")
    grads = torch.zeros((spec.num_parameters,), device="cuda")
    adj_in = torch.zeros_like(x)
    fwd = torch.empty((net.forward_memory(n),), dtype=torch.uint8, device="cuda")
    bwd = torch.empty((net.adjoint_memory(n),), dtype=torch.uint8, device="cuda")
    check(lib().qmlp_network_set_parameter(net._h, wrap(t_params), _capi.QMLP_INFERENCE))
    check(lib().qmlp_network_set_parameter(net._h, wrap(grads), _capi.QMLP_GRADIENTS))
    check(lib().qmlp_network_forward(net._h, wrap(x), wrap(out), fwd.data_ptr(), None))
    ai = wrap(adj_in)
    for _ in range(2):
        check(lib().qmlp_network_adjoint(net._h, wrap(x), wrap(adj), 7, C.byref(ai), fwd.data_ptr(), bwd.data_ptr(), None))
    torch.cuda.synchronize()
    once = oracle.network_backward(spec, params, x.cpu().numpy(), adj.cpu().numpy(), half=True)
    scale = max(1.0, float(np.abs(once.grad_params).max()))
    helpers.assert_close(grads.cpu().numpy() / scale, 2 * once.grad_params / scale, "accumulated weight gradient", max_violations=0.02)
    helpers.assert_close(adj_in.cpu().numpy(), 2 * once.adj_input, "accumulated input gradient", max_violations=0.02)
    check(lib().qmlp_network_zero_gradients(net._h, None))
    torch.cuda.synchronize()
    assert float(grads.abs().max()) == 0.0


def test_argument_errors():
    """Same failures as the reference's CHECK_* macros (src_cpp/src/fused_network.cpp:257-278, 509-516)."""
    import torch
    from qmlp._capi import QmlpError, ConfigurationError
    from qmlp import bindings
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup("config1")
    with pytest.raises(QmlpError):
        net.inference(torch.zeros((4, 2), device="cuda"), t_params)            # wrong channel count
    with pytest.raises(QmlpError):
        net.inference(torch.zeros((4, 3), device="cuda"), t_params[:-1].contiguous())   # wrong parameter count
    with pytest.raises(ConfigurationError):
        bindings.Network(json.dumps(dict(specs.config1(), num_outputs=2)))        # last layer != num_outputs
    with pytest.raises(ConfigurationError):
        bad = specs.config1(); bad["encodings"][0]["id"] = "identity"              # factory key is "Identity"
        bindings.Network(json.dumps(bad))
    with pytest.raises(ConfigurationError):
        bad = specs.config1(); bad["network"][0]["activation"] = "nope"
        bindings.Network(json.dumps(bad))
    out = net.inference(torch.zeros((0, 3), device="cuda"), t_params)             # empty batch is a no-op
    assert out.shape == (0, 1)
