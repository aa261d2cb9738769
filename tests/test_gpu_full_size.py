"""The benchmark networks at their full table sizes: 2^19 rows per hashed level (3-D, two features), a dense 64^3 level
plus 2^18 rows per hashed level (four features), and 2^22 rows per hashed level (4-D, four features; 220 M parameters,
element offsets close to 2^28). The kernels take table sizes at run time, so these cases run the same code as the
small-table cases elsewhere; what they add is the index arithmetic, the 32-bit element offsets and the chunked
level-major pass where the numbers are large. The oracle works on the full tables; the batches are a few thousand
points so that it finishes in seconds."""
import json

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs

pytestmark = pytest.mark.gpu

FULL = {"config3": specs.config3, "config4": specs.config4, "config5": specs.config5}


def probe_encodings():
    """Grids with one feature per row for the index probes: the full-size level tables of the 3-D and the 4-D benchmark grid."""
    return [specs.hashgrid(3, 16, 1, 19, 16, 7006, per_level_scale=1.5), specs.hashgrid(4, 16, 1, 22, 16, 2489)]


def bounds_check_jobs():
    """(configuration, fp16-table mask) of the bounds-checking instantiations the tests below use."""
    return [(specs.config5(), 1), (specs.config3(), 1), (specs.config4(), 0), (specs.config3(log2_hashmap_size=12), 1)]


_cache = {}


def _case(name):
    """spec, fp16-rounded parameters and fp32 tables of one full-size network (built once per test session)."""
    if name not in _cache:
        cfg = FULL[name]()
        spec = oracle.parse_spec(cfg)
        params = helpers.xavier_parameters(spec, cfg, bias_scale=0.05)
        tables = helpers.grid_tables(spec, seed=17, scale=0.5)
        _cache[name] = (cfg, spec, params, tables)
    return _cache[name]


@pytest.mark.parametrize("path,half_tables", [(0, False), (2, True), (3, True)], ids=["auto_fp32", "planes_fp16", "tcgen05_fp16"])
@pytest.mark.parametrize("name", list(FULL))
def test_inference_full_size(name, path, half_tables):
    import torch
    from qmlp import bindings
    cfg, spec, params, tables = _case(name)
    n = 4099
    x = helpers.uniform(51, 1, (n, spec.num_inputs))
    used = [t.astype(np.float16).astype(np.float32) if (t is not None and half_tables) else t for t in tables]
    expected = oracle.network_forward(spec, params, x, used, half=True)
    net = bindings.Network(json.dumps(cfg))
    tt = [(torch.from_numpy(t).cuda().half() if half_tables else torch.from_numpy(t).cuda()) if t is not None else None for t in tables]
    try:
        bindings.QuickMLP.set_kernel_path(path)
        out = net.inference(torch.from_numpy(x).cuda(), torch.from_numpy(params).cuda(), tt)
    finally:
        bindings.QuickMLP.set_kernel_path(0)
    helpers.assert_close(out.cpu().numpy(), expected, f"{name} inference at full table size", max_violations=0.01)
    assert bindings.QuickMLP.device_status() == 0


@pytest.mark.parametrize("flags", [6, 7], ids=["weights+tables", "all"])
@pytest.mark.parametrize("name", ["config3", "config4"])
def test_forward_adjoint_full_size(name, flags):
    """qmlp_network_forward + qmlp_network_adjoint on the full tables: output, table gradients (all 13 M / 8.5 M entries),
    weight gradients and, with flags 7, input gradients against the oracle evaluated at the stashed forward state."""
    import ctypes as C
    import torch
    from qmlp import _capi, bindings
    from qmlp._capi import check, lib, wrap
    cfg, spec, params, tables = _case(name)
    n = 4099
    n32 = (n + 31) // 32 * 32
    x = helpers.uniform(52, 1, (n, spec.num_inputs))
    adj = helpers.uniform(52, 2, (n, spec.num_outputs), -1.0, 1.0)
    net = bindings.Network(json.dumps(cfg))
    tx, tadj, tp = torch.from_numpy(x).cuda(), torch.from_numpy(adj).cuda(), torch.from_numpy(params).cuda()
    tt = [torch.from_numpy(t).cuda() for t in tables]
    gw = torch.zeros((spec.num_parameters,), device="cuda")
    gt = [torch.zeros_like(t) for t in tt]
    check(lib().qmlp_network_set_parameter(net._h, wrap(tp), _capi.QMLP_INFERENCE))
    check(lib().qmlp_network_set_parameter(net._h, wrap(gw), _capi.QMLP_GRADIENTS))
    for i, t in enumerate(tt):
        net.encoding(i).set_parameter(t, _capi.QMLP_INFERENCE)
        net.encoding(i).set_parameter(gt[i], _capi.QMLP_GRADIENTS)
    out = torch.empty((n, spec.num_outputs), device="cuda")
    fwd = torch.zeros((net.forward_memory(n) // 2,), dtype=torch.float16, device="cuda")
    bwd = torch.zeros((max(net.adjoint_memory(n, flags), 16),), dtype=torch.uint8, device="cuda")
    gx = torch.zeros_like(tx)
    agx = wrap(gx) if flags & 1 else wrap(None)
    check(lib().qmlp_network_forward(net._h, wrap(tx), wrap(out), fwd.data_ptr(), None))
    check(lib().qmlp_network_adjoint(net._h, wrap(tx), wrap(tadj), flags, C.byref(agx), fwd.data_ptr(), bwd.data_ptr(), None))
    torch.cuda.synchronize()
    assert bindings.QuickMLP.device_status() == 0

    expected = oracle.network_forward(spec, params, x, tables, half=True)
    helpers.assert_close(out.cpu().numpy(), expected, f"{name} forward", max_violations=0.01)
    cin0 = spec.layers[0].channels_in
    stash = [fwd[: n32 * cin0].view(n32, cin0)[:n].float().cpu().numpy()]
    off = n32 * cin0
    for l in spec.layers:
        stash.append(helpers.stash_rows(fwd[off: off + n32 * l.channels_out], n32, l.channels_out)[:n].float().cpu().numpy())
        off += n32 * l.channels_out
    g = oracle.network_backward(spec, params, x, adj, tables, half=True, want_input=bool(flags & 1), stash=stash)
    scale = float(np.abs(g.grad_params).max())
    helpers.assert_close(gw.cpu().numpy(), g.grad_params, f"{name} weight gradients", rtol=helpers.RTOL_WGRAD, atol=1e-2 * scale,
                         max_violations=0.01)
    for i, want in enumerate(g.grad_encodings):
        got = gt[i].cpu().numpy()
        helpers.assert_close(got, want, f"{name} table gradient {i}", rtol=2e-2, atol=1e-2 * float(np.abs(want).max()), max_violations=0.001)
        assert np.count_nonzero(got) > 0 and abs(float(got.sum()) - float(want.sum())) <= 1e-2 * float(np.abs(want).sum())
    if flags & 1:
        helpers.assert_close(gx.cpu().numpy(), g.adj_input, f"{name} input gradient", rtol=5e-2,
                             atol=2e-2 * float(np.abs(g.adj_input).max()), max_violations=0.02)


@pytest.mark.parametrize("sort", [0, 1], ids=["unsorted", "sorted"])
@pytest.mark.parametrize("name", ["config3", "config4"])
def test_trainer_step_full_size(name, sort):
    """Gradients of one fused training step on the full tables (level-major gather, points sorted into bins or not)
    against the oracle."""
    import torch
    from qmlp import bindings
    from qmlp.trainer import FusedTrainer
    cfg, spec, params, tables = _case(name)
    n = 8192
    x = helpers.uniform(53, 1, (n, spec.num_inputs))
    t = helpers.uniform(53, 2, (n, spec.num_outputs), -1.0, 1.0)
    net = bindings.Network(json.dumps(cfg))
    tr = FusedTrainer(net, grid_half_copy=True)
    tr.set_parameters(torch.from_numpy(params.astype(np.float32)).cuda(), [torch.from_numpy(tb).cuda() for tb in tables])
    try:
        bindings.QuickMLP.set_kernel_path(2)
        bindings.QuickMLP.set_tuning("sort_points", sort)
        tr.backend.gradients(torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda(), n, tr.loss_sum)
        torch.cuda.synchronize()
    finally:
        bindings.QuickMLP.set_kernel_path(0)
        bindings.QuickMLP.set_tuning("sort_points", -1)
    assert bindings.QuickMLP.device_status() == 0
    t16 = [tb.astype(np.float16).astype(np.float32) for tb in tables]
    out = oracle.network_forward(spec, params, x, t16, half=True)
    g = oracle.network_backward(spec, params, x, oracle.mse_loss_grad(out, t), t16, half=True, want_input=False)
    np.testing.assert_allclose(float(tr.loss_sum.item()), float(((out - t) ** 2).sum()), rtol=2e-3)
    got_w = tr.segment(tr.gradient, 0).cpu().numpy()
    helpers.assert_close(got_w, g.grad_params, f"{name} weight gradients", rtol=helpers.RTOL_WGRAD,
                         atol=2e-2 * float(np.abs(g.grad_params).max()), max_violations=0.02)
    for i, want in enumerate(g.grad_encodings):
        got = tr.segment(tr.gradient, 1 + i).cpu().numpy()
        helpers.assert_close(got, want, f"{name} table gradient {i}", rtol=5e-2, atol=2e-2 * float(np.abs(want).max()), max_violations=0.002)
        assert abs(float(got.sum()) - float(want.sum())) <= 2e-2 * float(np.abs(want).sum())


def test_sorted_step_large_batch_equals_unsorted():
    """2^18 points of the 3-D hash-grid network at full size: the sorted step with register sums over runs of points in one cell, the sorted step without them and the unsorted
    step leave the same gradient vector, up to the order of the floating-point sums."""
    import torch
    from qmlp import bindings
    from qmlp.trainer import FusedTrainer
    cfg, spec, params, tables = _case("config3")
    n = 1 << 18
    gen = torch.Generator(device="cuda")
    gen.manual_seed(5)
    x = torch.rand((n, 3), device="cuda", generator=gen)
    t = torch.sin(8 * x[:, :1]) * torch.cos(6 * x[:, 1:2]) * torch.sin(4 * x[:, 2:3])
    net = bindings.Network(json.dumps(cfg))
    tr = FusedTrainer(net, grid_half_copy=True)
    tr.set_parameters(torch.from_numpy(params.astype(np.float32)).cuda(), [torch.from_numpy(tb).cuda() for tb in tables])
    results = []
    try:
        for sort, box in ((0, 1), (1, 1), (1, 0)):
            bindings.QuickMLP.set_tuning("sort_points", sort)
            bindings.QuickMLP.set_tuning("scatter_runs", box)
            tr.gradient.zero_()
            tr.loss_sum.zero_()
            tr.backend.gradients(x, t, n, tr.loss_sum)
            torch.cuda.synchronize()
            results.append((tr.gradient.clone(), float(tr.loss_sum.item())))
    finally:
        bindings.QuickMLP.set_tuning("sort_points", -1)
        bindings.QuickMLP.set_tuning("scatter_runs", 1)
    assert bindings.QuickMLP.device_status() == 0
    base, base_loss = results[0]
    scale = float(base.abs().max())
    assert scale > 0
    for (g, loss), what in zip(results[1:], ("sorted", "sorted, no run sums")):
        assert abs(loss - base_loss) <= 1e-4 * abs(base_loss)
        diff = (g - base).abs()
        frac = float((diff > 1e-2 * base.abs() + 2e-3 * scale).float().mean())
        assert frac <= 1e-4, f"{what}: {frac * 100:.4f}% of the gradient entries differ"
        assert abs(float(g.double().sum()) - float(base.double().sum())) <= 1e-3 * float(base.double().abs().sum())


def test_grid_indices_bit_exact_full_size():
    """Index probes (tables that hold their own row number, points on cell corners) through the full-size level tables:
    a 3-D level of 2^19 rows and a 4-D level of 2^22 rows, coarse dense levels and the finest hashed ones, including
    cells at the upper end of every dimension."""
    import torch
    from qmlp import bindings
    for cfg in probe_encodings():
        e = bindings.Encoding(json.dumps(cfg))
        oe = oracle.parse_encoding(cfg)
        assert e.grid_levels() == [(lv.memory_offset, lv.resolution, lv.hash_grid_size, lv.hashed) for lv in oe.levels]
        n = 2000
        table = torch.zeros((oe.num_parameters,), device="cuda")
        for li in (0, 3, 4, len(oe.levels) - 2, len(oe.levels) - 1):
            lv = oe.levels[li]
            cells = (helpers.uniform(9, 40 + li, (n, oe.n_in)) * (lv.resolution - 1)).astype(np.int64)
            cells[: n // 8] = lv.resolution - 2                       # last cell of every dimension ...
            cells[n // 8: n // 4, 0] = lv.resolution - 2              # ... and of one dimension at a time
            x = (cells.astype(np.float64) / (lv.resolution - 1)).astype(np.float32)
            iL, iH, f = oracle.grid_cell(oe, lv, x)
            rows = oracle.grid_index(oe, lv, iL)
            level_size = lv.hash_grid_size if lv.hashed else lv.resolution ** oe.n_in
            assert level_size <= (1 << 24)                            # row numbers stay exact in fp32
            table.zero_()
            table[lv.memory_offset:lv.memory_offset + level_size] = torch.arange(level_size, device="cuda", dtype=torch.float32)
            out = e.inference_with_parameter(torch.from_numpy(x).cuda(), table).cpu().numpy()
            exact = f.max(axis=1) == 0
            assert exact.sum() > n // 8
            assert np.array_equal(out[exact, li], (rows[exact] - lv.memory_offset).astype(np.float32)), f"level {li}: index mismatch"


@pytest.fixture
def bounds_check():
    """Kernels instantiated with QMLP_BOUNDS_CHECK for one test: every table row, stash offset and plane offset is tested
    against the declared size, an access outside is skipped and reported through the status word."""
    from qmlp import bindings
    bindings.QuickMLP.set_tuning("bounds_check", 1)
    yield
    bindings.QuickMLP.set_tuning("bounds_check", 0)
    bindings.QuickMLP.set_tuning("bounds_shrink", 0)


def test_full_size_cases_under_bounds_check(bounds_check):
    """The full-size networks once more through bounds-checking kernels: 4-D tables of 2^22 rows (element offsets close to
    2^28) through the chunked level-major pass, a training step on the 2^19-row tables, forward and adjoint of the
    two-grid network. No access leaves its buffer (status word 0) and the results are those of the regular kernels."""
    import ctypes as C
    import torch
    from qmlp import _capi, bindings
    from qmlp._capi import check, lib, wrap
    from qmlp.trainer import FusedTrainer
    # inference, 4-D grid, fp16 tables, level-major pass
    cfg, spec, params, tables = _case("config5")
    x = torch.from_numpy(helpers.uniform(81, 1, (70_001, 4))).cuda()         # more than one 2^16-point chunk of planes
    tp = torch.from_numpy(params).cuda()
    tt = [torch.from_numpy(tables[0]).cuda().half()]
    checked = bindings.Network(json.dumps(cfg)).inference(x, tp, tt)
    assert bindings.QuickMLP.device_status() == 0
    bindings.QuickMLP.set_tuning("bounds_check", 0)
    regular = bindings.Network(json.dumps(cfg)).inference(x, tp, tt)
    bindings.QuickMLP.set_tuning("bounds_check", 1)
    assert torch.equal(checked, regular)
    del tt, checked, regular
    # training step, 3-D grid
    cfg, spec, params, tables = _case("config3")
    n = 1 << 18
    gen = torch.Generator(device="cuda"); gen.manual_seed(9)
    x = torch.rand((n, 3), device="cuda", generator=gen)
    t = torch.sin(8 * x[:, :1]) * torch.cos(6 * x[:, 1:2]) * torch.sin(4 * x[:, 2:3])
    grads = []
    for flag in (1, 0):
        bindings.QuickMLP.set_tuning("bounds_check", flag)
        tr = FusedTrainer(bindings.Network(json.dumps(cfg)), grid_half_copy=True)
        tr.set_parameters(torch.from_numpy(params.astype(np.float32)).cuda(), [torch.from_numpy(tables[0]).cuda()])
        tr.backend.gradients(x, t, n, tr.loss_sum)
        torch.cuda.synchronize()
        assert bindings.QuickMLP.device_status() == 0
        grads.append(tr.gradient.clone())
        del tr
    bindings.QuickMLP.set_tuning("bounds_check", 1)
    scale = float(grads[1].abs().max())
    assert float(((grads[0] - grads[1]).abs() > 1e-2 * grads[1].abs() + 2e-3 * scale).float().mean()) <= 1e-4
    # forward + adjoint, dense + hash grid with four features, fp32 tables
    cfg, spec, params, tables = _case("config4")
    n = 4099
    net = bindings.Network(json.dumps(cfg))
    tx = torch.from_numpy(helpers.uniform(82, 1, (n, 3))).cuda()
    tadj = torch.from_numpy(helpers.uniform(82, 2, (n, 4), -1.0, 1.0)).cuda()
    tp = torch.from_numpy(params).cuda()
    tt = [torch.from_numpy(tb).cuda() for tb in tables]
    gw = torch.zeros((spec.num_parameters,), device="cuda")
    gt = [torch.zeros_like(tb) for tb in tt]
    check(lib().qmlp_network_set_parameter(net._h, wrap(tp), _capi.QMLP_INFERENCE))
    check(lib().qmlp_network_set_parameter(net._h, wrap(gw), _capi.QMLP_GRADIENTS))
    for i, tb in enumerate(tt):
        net.encoding(i).set_parameter(tb, _capi.QMLP_INFERENCE)
        net.encoding(i).set_parameter(gt[i], _capi.QMLP_GRADIENTS)
    out = torch.empty((n, 4), device="cuda")
    fwd = torch.zeros((net.forward_memory(n),), dtype=torch.uint8, device="cuda")
    bwd = torch.zeros((max(net.adjoint_memory(n, 7), 16),), dtype=torch.uint8, device="cuda")
    gx = torch.zeros_like(tx)
    agx = wrap(gx)
    check(lib().qmlp_network_forward(net._h, wrap(tx), wrap(out), fwd.data_ptr(), None))
    check(lib().qmlp_network_adjoint(net._h, wrap(tx), wrap(tadj), 7, C.byref(agx), fwd.data_ptr(), bwd.data_ptr(), None))
    assert bindings.QuickMLP.device_status() == 0
    assert float(gw.abs().max()) > 0 and all(float(g.abs().max()) > 0 for g in gt) and float(gx.abs().max()) > 0


def test_bounds_check_reports_instead_of_faulting(bounds_check):
    """With every size declared 3000 elements smaller than it is (test hook), the checks must fire: table rows beyond
    the declared end, stash and plane offsets beyond theirs. The accesses are skipped, the kernels finish, the status
    word carries the three bits, and nothing faults (the real buffers are larger than declared)."""
    import torch
    from qmlp import bindings
    from qmlp.trainer import FusedTrainer
    cfg = specs.config3(log2_hashmap_size=12)
    spec = oracle.parse_spec(cfg)
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.05).astype(np.float32)
    table = helpers.grid_tables(spec, scale=0.5)[0]
    n = 8192
    x = torch.from_numpy(helpers.uniform(83, 1, (n, 3))).cuda()
    t = torch.from_numpy(helpers.uniform(83, 2, (n, 1), -1.0, 1.0)).cuda()
    tr = FusedTrainer(bindings.Network(json.dumps(cfg)), grid_half_copy=True)
    tr.set_parameters(torch.from_numpy(params).cuda(), [torch.from_numpy(table).cuda()])
    bindings.QuickMLP.set_kernel_path(2)        # level-major gather: the planes are in use
    try:
        tr.backend.gradients(x, t, n, tr.loss_sum)
        assert bindings.QuickMLP.device_status() == 0                      # honest sizes: silent
        bindings.QuickMLP.set_tuning("bounds_shrink", 3000)
        tr.gradient.zero_()
        tr.backend.gradients(x, t, n, tr.loss_sum)
        status = bindings.QuickMLP.device_status()
    finally:
        bindings.QuickMLP.set_kernel_path(0)
        bindings.QuickMLP.set_tuning("bounds_shrink", 0)
    assert status & 2, "rows beyond the declared end of the table were not reported"
    assert status & 4, "stash offsets beyond the declared size were not reported"
    assert status & 8, "plane offsets beyond the declared size were not reported"
    assert not (status & 1)
    assert bool(torch.isfinite(tr.gradient).all())
    assert bindings.QuickMLP.device_status() == 0                          # reading the word cleared it
