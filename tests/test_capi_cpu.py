"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol include/qmlp_b200.h declares;
spec parsing, padding, parameter layout, level tables and error reporting behave like the reference host code
(src_cpp/src/fused_network.cpp:33-223, encoding_hashgrid.cpp:41-112, activation.cpp:152-240); the per-spec source
generator produces what the templates expect. No compute entry point is called."""
import ctypes as C
import json
import os
import re

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from qmlp import _capi
    return _capi.lib()


def test_library_exports_every_declared_symbol():
    from qmlp import _capi
    header = open(os.path.join(ROOT, "include", "qmlp_b200.h")).read()
    declared = set(re.findall(r"QMLP_API\s+[\w\s\*]+?\b(qmlp_\w+)\s*\(", header))
    assert len(declared) >= 55
    lib = C.CDLL(os.path.abspath(_capi.LIB_PATH))
    missing = [name for name in sorted(declared) if not hasattr(lib, name)]
    assert not missing, f"declared but not exported: {missing}"
    assert declared == set(_capi.SIGNATURES), "Python binding table and header differ"


@pytest.mark.parametrize("cfg", [specs.config1(), specs.config2(), specs.config3(), specs.config4(), specs.config5(),
                                 specs.identity_net(19, [16, 16], ["identity", "identity"], bias=False),
                                 specs.identity_net(20, [17, 24], ["identity", "identity"], bias=[True, False])])
def test_layout_equals_oracle(cfg):
    from qmlp import bindings
    bindings.QuickMLP.set_log_level("error")
    net = bindings.Network(json.dumps(cfg))
    spec = oracle.parse_spec(cfg)
    assert (net.channels_in(), net.channels_out(), net.num_layers(), net.num_encodings()) == \
        (spec.num_inputs, spec.num_outputs, len(spec.layers), len(spec.encodings))
    assert net.num_network_parameters() == spec.num_parameters
    for i, l in enumerate(spec.layers):
        cin, cout, bias, ws, bs = net.layer_info(i)
        assert (cin, cout, bias, ws, bs) == (l.channels_in, l.channels_out, l.use_bias, l.weights_start, l.bias_start if l.use_bias else -1)
    for i, e in enumerate(spec.encodings):
        enc = net.encoding(i)
        assert (enc.id(), enc.num_output_channels(), enc.parameter_count(), enc.max_input_channel()) == \
            (e.id, e.num_outputs, e.num_parameters, e.start_in + e.n_in - 1)
        assert enc.grid_levels() == [(lv.memory_offset, lv.resolution, lv.hash_grid_size, lv.hashed) for lv in e.levels]
        assert oracle.parse_encoding(json.loads(enc.to_json())).levels == e.levels       # to_json round trip


def test_parameter_views_and_initialisation():
    import torch
    from qmlp import bindings
    net = bindings.Network(json.dumps(specs.config2()))
    p = torch.zeros((net.num_network_parameters(),), dtype=torch.float16)
    net.initialize_inference_parameters(p, seed=42)
    q = torch.zeros_like(p)
    net.initialize_inference_parameters(q, seed=42)
    assert torch.equal(p, q)                                   # same seed, same stream
    for layer in range(net.num_layers()):
        cin, cout, bias, ws, bs = net.layer_info(layer)
        w = net.parameter_view(layer, False, p)
        assert w.shape == (cout, cin) and w.data_ptr() == p.data_ptr() + 2 * ws        # a view, not a copy
        bound = 1.0 / np.sqrt(cin)                              # U(+-1/sqrt(Cin_padded)), fused_network.cpp:294-305
        assert float(w.abs().max()) <= bound + 1e-3 and float(w.float().std()) > 0.4 * bound
        b = net.parameter_view(layer, True, p)
        assert b.shape == (cout,) and float(b.abs().max()) <= bound + 1e-3


def test_configuration_errors():
    from qmlp import bindings
    from qmlp._capi import ConfigurationError, QmlpError

    def bad(mutate, exc=ConfigurationError):
        cfg = specs.config3(12)
        mutate(cfg)
        with pytest.raises(exc):
            bindings.Network(json.dumps(cfg))
    bad(lambda c: c.update(num_outputs=3))                                     # last layer != num_outputs
    bad(lambda c: c["encodings"][0].update(id="hashgrid"))                     # unknown encoding id
    bad(lambda c: c["encodings"][0].update(start_in=1))                        # reads input channel 3 of 3
    bad(lambda c: c["network"][0].update(activation="gelu"))                   # unknown activation
    bad(lambda c: c.update(network=[]))                                        # empty network
    bad(lambda c: c.pop("activation_specification"))                           # missing key
    bad(lambda c: c["network"][0].update(activation=["relu"] * 3))             # per-channel list of the wrong length
    bad(lambda c: c["encodings"][0].update(n_in=7), QmlpError)                 # grid dimension outside [1, 6]
    bad(lambda c: c.update(activation_specification=["no/such/file.json"]))
    # a per-channel list of the right length is accepted, mixed activations included (the reference stops at code generation)
    mixed = specs.config3(12)
    mixed["network"][0].update(activation=["relu"] * 40 + ["sine"] * 24)
    assert bindings.Network(json.dumps(mixed)).num_layers() == 3
    with pytest.raises(QmlpError):
        bindings.Network("{ not json")
    with pytest.raises(QmlpError):
        bindings.Activation(json.dumps({"id": "not an identifier", "forward": "z = x", "adjoint": "adjx = adjz"}))
    # inline activation objects and the shipped file are both accepted (activation.cpp:166-210)
    cfg = specs.identity_net(3, [16, 1], ["swish", "identity"], extra_activations=[
        {"id": "swish", "forward": "z = x", "adjoint": "adjx = adjz"}])
    assert bindings.Network(json.dumps(cfg)).num_layers() == 2


def test_generated_source_instantiates_templates(tmp_path):
    """The library writes one translation unit per spec into the kernel cache and builds it with nvcc for sm_100a."""
    from qmlp import bindings
    old = bindings.QuickMLP.kernel_cache_dir()
    bindings.QuickMLP.set_kernel_cache_dir(str(tmp_path))
    try:
        custom = {"id": "halfx", "forward": "z = __hmul(x, __float2half(0.5f))", "adjoint": "adjx = __hmul(adjz, __float2half(0.5f))"}
        cfg = specs.identity_net(2, [16, 2], ["halfx", "relu"], bias=[True, False], extra_activations=[custom])
        bindings.Network(json.dumps(cfg)).compile(0)
        files = os.listdir(tmp_path)
        cu = [f for f in files if f.endswith(".cu")]
        assert len(cu) == 1 and any(f.endswith(".so") for f in files)
        src = open(os.path.join(tmp_path, cu[0])).read()
        assert "struct halfx" in src and "ScalarActivation<activations::halfx>" in src and "BuiltinRelu" in src
        assert "CIN[2] = {16, 16}" in src and "BOFF[2] = {512, -1}" in src and "EncIdentity<0, 2, 0>" in src
        bindings.Encoding(json.dumps(specs.hashgrid(2, 2, 2, 6, 4, 32))).compile(False)
        bindings.Activation("sine").compile()
        assert len([f for f in os.listdir(tmp_path) if f.endswith(".so")]) == 3
    finally:
        bindings.QuickMLP.set_kernel_cache_dir(old)


def test_simulated_network_and_weight_copy_are_plain_torch():
    """SimulatedNetwork (the reference's comparison tool, src_py/qmlp/network.py:161-243) runs without the library."""
    import torch
    from qmlp.network import SimulatedNetwork
    cfg = specs.identity_net(4, [8, 2], ["sine", "identity"], bias=True)
    net = SimulatedNetwork(json.dumps(cfg), weight_dtype=torch.float32)
    y = net(torch.zeros((5, 4)))
    assert y.shape == (5, 2) and net.num_layers() == 2 and net.has_bias(0)
    assert net.get_weight(0, False, False).shape == (8, 4)


def test_line_integration_and_per_channel_host_side(tmp_path):
    """Host side of the two spec features the reference declares but cannot instantiate in a fused network: a
    LineIntegration encoding (parse, sizes, JSON round trip, errors of src_cpp/src/encoding_line_integration.cpp:18-49)
    and per-channel activation arrays (generated functor)."""
    from qmlp import bindings
    from qmlp._capi import QmlpError, ConfigurationError
    line = {"id": "LineIntegration", "start_in": 2, "n_in": 3, "stepsize": 0.05, "blending": "average",
            "volume": specs.hashgrid(3, 4, 2, 10, 4, 32)}
    enc = bindings.Encoding(json.dumps(line))
    grid = bindings.Encoding(json.dumps(specs.hashgrid(3, 4, 2, 10, 4, 32)))
    assert enc.max_input_channel() == 2 + 6 - 1 and enc.num_output_channels() == 8 and enc.has_parameters()
    assert enc.parameter_count() == grid.parameter_count() and enc.grid_levels() == grid.grid_levels()
    back = json.loads(enc.to_json())
    assert back["id"] == "LineIntegration" and back["volume"]["id"] == "HashGrid" and back["volume"]["start_in"] == 0
    assert back["blending"] == "average" and abs(back["stepsize"] - 0.05) < 1e-6
    assert json.loads(bindings.Encoding(enc.to_json()).to_json()) == back
    for bad in ({"stepsize": 0.0}, {"n_in": 2}, {"volume": {"id": "Identity", "start_in": 0, "n_in": 3}}):
        with pytest.raises(QmlpError):
            bindings.Encoding(json.dumps(dict(line, **bad)))
    with pytest.raises(QmlpError):
        bindings.Encoding(json.dumps({k: v for k, v in line.items() if k != "blending"}))

    old = bindings.QuickMLP.kernel_cache_dir()
    bindings.QuickMLP.set_kernel_cache_dir(str(tmp_path))
    try:
        cfg = {"num_inputs": 8, "num_outputs": 2, "activation_specification": specs.BUILTIN, "encodings": [line],
               "network": specs.mlp([16, 2], [["relu"] * 6 + ["sine"] * 10, "identity"], True)}
        bindings.Network(json.dumps(cfg)).compile(0)
        src = open(os.path.join(tmp_path, [f for f in os.listdir(tmp_path) if f.endswith(".cu")][0])).read()
        assert "EncLine<2, 3, 4, 2, true, 0, 0, false, true>" in src and "HAS_LINE = true" in src
        assert "struct PerChannelAct0 : PerChannelActivation<PerChannelAct0>" in src
        assert "if (c < 6) return BuiltinRelu::forward(x);" in src and "if (c < 16) return BuiltinSine::forward(x);" in src
    finally:
        bindings.QuickMLP.set_kernel_cache_dir(old)
    with pytest.raises(QmlpError):
        bindings.QuickMLP.set_kernel_path(4)
    bindings.QuickMLP.set_kernel_path(0)


def test_stash_block_layout_helper():
    """helpers.stash_rows undoes the layout the kernels use for pre-activation and delta matrices: element (row, col) of
    an (N32, C) matrix sits at tile * 32 * C + ((col // 8) * 4 + (row % 32) // 8) * 64 + (row % 8) * 8 + col % 8."""
    import numpy as np
    import helpers
    n32, c = 96, 48
    flat = np.zeros(n32 * c, dtype=np.float32)
    for row in range(n32):
        for col in range(c):
            at = (row // 32) * 32 * c + ((col // 8) * 4 + (row % 32) // 8) * 64 + (row % 8) * 8 + col % 8
            flat[at] = row * 1000 + col
    rows = helpers.stash_rows(flat, n32, c)
    want = np.arange(n32)[:, None] * 1000 + np.arange(c)[None, :]
    assert np.array_equal(rows, want.astype(np.float32))
    both = helpers.stash_rows_all(np.concatenate([flat, flat]), n32, [c, c])
    assert np.array_equal(both.reshape(2, n32, c)[1], want.astype(np.float32))
