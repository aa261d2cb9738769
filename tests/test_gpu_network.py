"""GPU parity of the fused network path (inference, forward-with-stash, adjoint, weight/bias/grid gradients) against
the CPU oracle, called through the C ABI. Mirrors the structure of the reference's
tests_py/qmlp_tests/test_network_base.py:87-147 (fused vs simulated network: inference, forward, input gradients,
parameter gradients at several batch sizes) and tests_cpp/test_against_eigen2.cpp (uneven widths, all-gradient modes).
"""
import ctypes as C
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
        # one activation per output channel (the reference parses such arrays and refuses them at code generation,
        # src_cpp/src/fused_network.cpp:106-125, 447): runs of built-ins, a user snippet, and a uniform array
        "per_channel": (specs.identity_net(4, [24, 20, 16, 3],
                                           [["relu"] * 8 + ["sine"] * 10 + ["celu"] * 6, ["identity"] * 5 + ["leaky"] * 15,
                                            ["celu"] * 16, "identity"], bias=True, extra_activations=[LEAKY]),
                        (-1.0, 1.0), "reference"),
        # rays (start, direction) integrated through a hash grid, plus the raw ray as identity features
        "line_net": ({"num_inputs": 6, "num_outputs": 3, "activation_specification": specs.BUILTIN,
                      "encodings": [{"id": "LineIntegration", "start_in": 0, "n_in": 3, "stepsize": 0.07, "blending": "average",
                                     "volume": specs.hashgrid(3, 4, 4, 10, 4, 32)},
                                    {"id": "Identity", "start_in": 0, "n_in": 6}],
                      "network": specs.mlp([32, 3], ["celu", "identity"], True)}, (-0.3, 1.3), "xavier"),
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
@pytest.mark.parametrize("path", [0, 3])
def test_inference(name, n, path):
    """path 0: the kernel the library picks for this batch (the mma.sync kernel at these sizes); path 3: the tcgen05
    kernel regardless of the batch size (falls back to mma.sync for specs wider than 128)."""
    import torch
    from qmlp import bindings
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup(name)
    x = helpers.uniform(42, 1, (n, spec.num_inputs), *rng)
    try:
        bindings.QuickMLP.set_kernel_path(path)
        out = net.inference(torch.from_numpy(x).cuda(), t_params, t_tables).cpu().numpy()
    finally:
        bindings.QuickMLP.set_kernel_path(0)
    assert bindings.QuickMLP.device_status() == 0
    emu = oracle.network_forward(spec, params, x, tables, half=True, activations=acts)
    ref = oracle.network_forward(spec, params, x, tables, half=False, activations=acts)
    assert np.isfinite(out).all()
    helpers.assert_close(out, emu, f"{name} inference vs fp16-emulating oracle", max_violations=0.01)
    helpers.assert_close(out, ref, f"{name} inference vs fp32 oracle", max_violations=helpers.MAX_VIOLATIONS)


@pytest.mark.parametrize("name", ["config2", "uneven", "custom_act", "per_channel", "config4_small", "config5_small"])
@pytest.mark.parametrize("n", [127, 128, 5000, 40001, 200_000])
def test_tensor_core_paths_agree(name, n):
    """The tcgen05 inference kernel and the mma.sync kernel compute the same function (same rounding points: fp32
    accumulate, one rounding to half per layer), and no kernel reports a timed-out on-chip wait."""
    import torch
    from qmlp import bindings
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup(name)
    x = torch.from_numpy(helpers.uniform(42, 7, (n, spec.num_inputs), *rng)).cuda()
    try:
        bindings.QuickMLP.set_kernel_path(3)
        out_best = net.inference(x, t_params, t_tables)
        bindings.QuickMLP.set_kernel_path(1)
        out_mma = net.inference(x, t_params, t_tables)
    finally:
        bindings.QuickMLP.set_kernel_path(0)
    assert bindings.QuickMLP.device_status() == 0
    emu = oracle.network_forward(spec, params, x.cpu().numpy(), tables, half=True, activations=acts)
    helpers.assert_close(out_best.cpu().numpy(), emu, f"{name} best path vs oracle", max_violations=0.01)
    # accumulation order differs (K in steps of 16 inside one instruction vs per-fragment), so allow a few half ulps
    helpers.assert_close(out_best.cpu().numpy(), out_mma.cpu().numpy(), f"{name} tcgen05 vs mma.sync", rtol=5e-3, atol=1e-3,
                         max_violations=0.005)


@pytest.mark.parametrize("name", ["config3_small", "config4_small", "config5_small", "grid2d_add_plus_identity"])
@pytest.mark.parametrize("half_tables", [False, True])
def test_level_major_encoding_pass(name, half_tables):
    """Inference through the level-major encoding pass (encodings of a chunk computed one grid level at a time into
    feature planes, then the layer chain on the planes) equals the fused gather, also across several chunks."""
    import torch
    from qmlp import bindings
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup(name)
    n = (1 << 22) + 4321 if name == "config3_small" else 3000       # more than one chunk (2^22 points) for one case
    x = torch.from_numpy(helpers.uniform(42, 8, (n, spec.num_inputs), *rng)).cuda()
    tabs = [t.half() if (t is not None and half_tables) else t for t in t_tables]
    try:
        bindings.QuickMLP.set_kernel_path(2)
        out_planes = net.inference(x, t_params, tabs)
        bindings.QuickMLP.set_kernel_path(3)     # gather fused into the layer kernel (automatic choice may pick the pass)
        out_fused = net.inference(x, t_params, tabs)
    finally:
        bindings.QuickMLP.set_kernel_path(0)
    assert bindings.QuickMLP.device_status() == 0
    helpers.assert_close(out_planes.cpu().numpy(), out_fused.cpu().numpy(), f"{name} planes vs fused", rtol=5e-3, atol=1e-3,
                         max_violations=0.005)
    m = 2000
    tabs_np = [t.astype(np.float16).astype(np.float32) if (t is not None and half_tables) else t for t in tables]
    emu = oracle.network_forward(spec, params, x[-m:].cpu().numpy(), tabs_np, half=True, activations=acts)
    helpers.assert_close(out_planes[-m:].cpu().numpy(), emu, f"{name} planes vs oracle", max_violations=0.01)


@pytest.mark.parametrize("name,n,chunk", [("config2", 100_003, 0), ("config2", 5000, 1024), ("config3_small", 70_001, 4096),
                                          ("config1", 17, 0), ("config1", 0, 0)])
def test_inference_from_host_memory(name, n, chunk):
    """The chunk-pipelined host-memory entry point returns exactly what the device-tensor call returns, for ragged
    last chunks, batches smaller than a chunk, an empty batch, and when called twice in a row on the same buffers."""
    import torch
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup(name)
    x = torch.from_numpy(helpers.uniform(42, 9, (n, spec.num_inputs), *rng))
    hx = x.pin_memory()
    ref = net.inference(x.cuda(), t_params, t_tables).cpu()
    out = net.inference_host(hx, t_params, t_tables, chunk_points=chunk)
    torch.cuda.current_stream().synchronize()
    assert out.shape == ref.shape
    assert torch.equal(out, ref)
    out.zero_()
    out2 = net.inference_host(hx, t_params, t_tables, output=out, chunk_points=chunk)
    torch.cuda.current_stream().synchronize()
    assert out2 is out and torch.equal(out, ref)
    assert bindings_status() == 0


def bindings_status():
    from qmlp import bindings
    return bindings.QuickMLP.device_status()


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


def _read_stash(spec, fwd_tmp, n):
    """Forward stash layout: [encoded input (N32, Cin0) | pre-activation of layer 0 (N32, Cout0) | layer 1 ...],
    fp16, N32 = N rounded up to 32; the encoded input row-major, the pre-activations in 8 x 8 blocks
    (helpers.stash_rows). Rows >= N are never written."""
    n32 = (n + 31) // 32 * 32
    halfs = fwd_tmp.view(dtype=np.float16)
    out, off = [], 0
    for i, width in enumerate([spec.layers[0].channels_in] + [l.channels_out for l in spec.layers]):
        seg = halfs[off:off + n32 * width]
        rows = seg.reshape(n32, width) if i == 0 else helpers.stash_rows(seg, n32, width)
        out.append(rows[:n].astype(np.float32))
        off += n32 * width
    return out


@pytest.mark.parametrize("name", list(network_cases().keys()))
@pytest.mark.parametrize("n", [32, 513, 4100])
def test_forward_and_adjoint(name, n):
    """forward with stash, then the adjoint with every gradient enabled, through the C ABI.

    The forward stash (encoded input and pre-activations) is compared with the oracle's forward pass. The adjoint is
    then compared with the oracle adjoint evaluated AT THE STASHED STATE, as the reference's backward kernels do:
    with relu/celu a pre-activation within one fp16 ulp of zero flips a derivative and changes that point's whole
    upstream gradient, which says nothing about the adjoint arithmetic under test."""
    import torch
    from qmlp import _capi
    from qmlp._capi import check, lib, wrap
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup(name)
    x = helpers.uniform(42, 3, (n, spec.num_inputs), *rng)
    adj = helpers.uniform(42, 4, (n, spec.num_outputs), -1.0, 1.0)
    tx, tadj = torch.from_numpy(x).cuda(), torch.from_numpy(adj).cuda()
    out = torch.empty((n, spec.num_outputs), device="cuda")
    fwd = torch.full((net.forward_memory(n),), 0x7e, dtype=torch.uint8, device="cuda")     # poison: fp16 NaN pattern
    bwd = torch.full((net.adjoint_memory(n),), 0x7e, dtype=torch.uint8, device="cuda")
    grads = torch.zeros((spec.num_parameters,), device="cuda")
    adj_in = torch.zeros_like(tx)
    grid_grads = [torch.zeros_like(t) if t is not None else None for t in t_tables]
    check(lib().qmlp_network_set_parameter(net._h, wrap(t_params), _capi.QMLP_INFERENCE))
    check(lib().qmlp_network_set_parameter(net._h, wrap(grads), _capi.QMLP_GRADIENTS))
    for i, t in enumerate(t_tables):
        if t is not None:
            net.encoding(i).set_parameter(t, _capi.QMLP_INFERENCE)
            net.encoding(i).set_parameter(grid_grads[i], _capi.QMLP_GRADIENTS)
    check(lib().qmlp_network_forward(net._h, wrap(tx), wrap(out), fwd.data_ptr(), None))
    ai = wrap(adj_in)
    check(lib().qmlp_network_adjoint(net._h, wrap(tx), wrap(tadj), 7, C.byref(ai), fwd.data_ptr(), bwd.data_ptr(), None))
    torch.cuda.synchronize()

    # forward: output and stash against the oracle's own forward pass
    feat = oracle.encode(spec, x, tables)
    o_out, o_pres, _ = oracle.mlp_forward(spec, params, feat, True, acts)
    helpers.assert_close(out.cpu().numpy(), o_out[:, :spec.num_outputs], f"{name} forward output", max_violations=0.01)
    stash = _read_stash(spec, fwd.cpu().numpy(), n)
    helpers.assert_close(stash[0], feat.astype(np.float16).astype(np.float32), f"{name} stashed encoding", rtol=2e-3, atol=1e-3)
    for i, p in enumerate(o_pres):
        helpers.assert_close(stash[1 + i], p, f"{name} stashed pre-activation {i}", max_violations=0.01)

    # adjoint at the stashed state
    g = oracle.network_backward(spec, params, x, adj, tables, half=True, activations=acts, stash=stash)
    in_scale = max(1.0, float(np.abs(g.adj_input).max()))
    helpers.assert_close(adj_in.cpu().numpy(), g.adj_input, f"{name} input gradient", atol=1e-3 * in_scale, max_violations=0.01)
    scale = max(1.0, float(np.abs(g.grad_params).max()))
    helpers.assert_close(grads.cpu().numpy(), g.grad_params, f"{name} weight+bias gradient", atol=1e-3 * scale, max_violations=0.01)
    for i, e in enumerate(spec.encodings):
        if e.num_parameters:
            gs = max(1.0, float(np.abs(g.grad_encodings[i]).max()))
            helpers.assert_close(grid_grads[i].cpu().numpy(), g.grad_encodings[i], f"{name} grid gradient", atol=1e-3 * gs,
                                 max_violations=0.01)

    # fully independent fp32 oracle (its own forward pass): norm-wise agreement
    g32 = oracle.network_backward(spec, params, x, adj, tables, half=False, activations=acts)

    def rel(a, b):
        return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-12))
    assert rel(grads.cpu().numpy(), g32.grad_params) < 0.15, f"{name} weight gradient vs fp32 oracle"
    assert rel(adj_in.cpu().numpy(), g32.adj_input) < 0.15, f"{name} input gradient vs fp32 oracle"


@pytest.mark.parametrize("name", ["config2", "uneven", "config3_small", "grid2d_add_plus_identity"])
def test_autograd_binding(name):
    """The autograd path of the Python binding (role of NetworkBindings::forward, bind_network.cpp:120-321) returns the
    same gradients as direct C-ABI calls, for every flag subset a user can trigger with requires_grad."""
    import torch
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup(name)
    n = 300
    x = helpers.uniform(42, 5, (n, spec.num_inputs), *rng)
    adj = torch.from_numpy(helpers.uniform(42, 6, (n, spec.num_outputs), -1.0, 1.0)).cuda()

    def run(want_x, want_w, want_t):
        tx = torch.from_numpy(x).cuda().requires_grad_(want_x)
        tp = t_params.float().requires_grad_(want_w)      # fp32 master, cast to half per call like the reference binding
        tt = [t.clone().requires_grad_(want_t) if t is not None else None for t in t_tables]
        out = net.forward(tx, tp, tt)
        out.backward(adj)
        torch.cuda.synchronize()
        return out.detach(), tx.grad, tp.grad, [t.grad if t is not None else None for t in tt]

    o_all, gx, gw, gt = run(True, True, True)
    o_inf = net.inference(torch.from_numpy(x).cuda(), t_params, t_tables)
    # forward-with-stash rounds every pre-activation to half before the activation (it is what backward reads);
    # the inference kernel may apply the activation to the fp32 accumulator: same function, a few half ulps apart
    helpers.assert_close(o_all.cpu().numpy(), o_inf.cpu().numpy(), "forward vs inference", rtol=5e-3, atol=1e-3, max_violations=0.005)
    assert gw.dtype == torch.float32 and gw.shape == t_params.shape
    _, gx1, gw1, _ = run(True, False, False)
    assert gw1 is None
    helpers.assert_close(gx1.cpu().numpy(), gx.cpu().numpy(), "input-only flags", rtol=1e-3, atol=1e-4 * max(1.0, float(gx.abs().max())))
    _, gx2, gw2, _ = run(False, True, False)
    assert gx2 is None
    helpers.assert_close(gw2.cpu().numpy(), gw.cpu().numpy(), "weights-only flags", rtol=1e-3, atol=1e-4 * max(1.0, float(gw.abs().max())))
    if any(t is not None for t in t_tables):
        _, _, _, gt3 = run(False, False, True)
        for a, b in zip(gt3, gt):
            if a is not None:
                helpers.assert_close(a.cpu().numpy(), b.cpu().numpy(), "encoding-only flags", rtol=1e-3,
                                     atol=1e-4 * max(1.0, float(b.abs().max())))


@pytest.mark.parametrize("name", ["config3_small", "config4_small", "config5_small", "grid2d_add_plus_identity"])
def test_table_gradient_scatter_paths_agree(name):
    """Weight + table gradients without input gradients: the level-major scatter kernel (adjoint feature planes, merged
    corner pairs) and the scatter inside the backward kernel produce the same sums."""
    import torch
    from qmlp import _capi, bindings
    from qmlp._capi import check, lib, wrap
    cfg, rng, spec, net, params, tables, acts, t_params, t_tables = _setup(name)
    n = 20_011
    tx = torch.from_numpy(helpers.uniform(42, 11, (n, spec.num_inputs), *rng)).cuda()
    tadj = torch.from_numpy(helpers.uniform(42, 12, (n, spec.num_outputs), -1.0, 1.0)).cuda()
    out = torch.empty((n, spec.num_outputs), device="cuda")
    fwd = torch.empty((net.forward_memory(n),), dtype=torch.uint8, device="cuda")
    assert net.adjoint_memory(n, 6) > net.adjoint_memory(n, 2) > 0
    bwd = torch.full((net.adjoint_memory(n, 6),), 0x7e, dtype=torch.uint8, device="cuda")
    results = []
    try:
        for path in (0, 1):
            bindings.QuickMLP.set_kernel_path(path)
            grads = torch.zeros((spec.num_parameters,), device="cuda")
            grid_grads = [torch.zeros_like(t) if t is not None else None for t in t_tables]
            check(lib().qmlp_network_set_parameter(net._h, wrap(t_params), _capi.QMLP_INFERENCE))
            check(lib().qmlp_network_set_parameter(net._h, wrap(grads), _capi.QMLP_GRADIENTS))
            for i, t in enumerate(t_tables):
                if t is not None:
                    net.encoding(i).set_parameter(t, _capi.QMLP_INFERENCE)
                    net.encoding(i).set_parameter(grid_grads[i], _capi.QMLP_GRADIENTS)
            launches = net.launch_count()
            check(lib().qmlp_network_forward(net._h, wrap(tx), wrap(out), fwd.data_ptr(), None))
            check(lib().qmlp_network_adjoint(net._h, wrap(tx), wrap(tadj), 6, None, fwd.data_ptr(), bwd.data_ptr(), None))
            torch.cuda.synchronize()
            results.append((grads, grid_grads, net.launch_count() - launches))
    finally:
        bindings.QuickMLP.set_kernel_path(0)
    assert bindings.QuickMLP.device_status() == 0
    (w0, g0, l0), (w1, g1, l1) = results
    # the separate scatter kernel is used when every grid has two features (only then can corner pairs be merged)
    split = all(e.n_features == 2 for e in spec.encodings if e.num_parameters)
    assert l0 == l1 + (1 if split else 0)
    helpers.assert_close(w0.cpu().numpy(), w1.cpu().numpy(), f"{name} weight gradient, both paths", rtol=1e-4,
                         atol=1e-5 * max(1.0, float(w1.abs().max())))
    for a, b in zip(g0, g1):
        if a is not None:
            assert float(b.abs().max()) > 0
            helpers.assert_close(a.cpu().numpy(), b.cpu().numpy(), f"{name} table gradient, both paths", rtol=1e-3,
                                 atol=1e-5 * max(1.0, float(b.abs().max())))


def test_gradients_accumulate():
    """adjoint adds to the bound gradient tensors (reference: outAdjWeights[i] += ..., callers zero them)."""
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
    stash = _read_stash(spec, fwd.cpu().numpy(), n)
    once = oracle.network_backward(spec, params, x.cpu().numpy(), adj.cpu().numpy(), half=True, stash=stash)
    scale = max(1.0, float(np.abs(once.grad_params).max()))
    helpers.assert_close(grads.cpu().numpy(), 2 * once.grad_params, "accumulated weight gradient", atol=1e-3 * scale, max_violations=0.01)
    helpers.assert_close(adj_in.cpu().numpy(), 2 * once.adj_input, "accumulated input gradient", max_violations=0.01)
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
