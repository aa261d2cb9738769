"""GPU parity of the fused training step (forward + L2 loss + backward + weight/bias/grid gradients + Adam) against the
CPU oracle. The reference has no fused step; its training loop is mse_loss + torch.optim.Adam in user code
(tests_py/qmlp_tests/test_network_image.py:41-55), so the oracle applies torch's Adam rule to oracle gradients."""
import json

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs

pytestmark = pytest.mark.gpu


def _target(x):   # smooth analytic target for the 3-D hash-grid training cases
    return (np.sin(8 * x[:, 0]) * np.cos(6 * x[:, 1]) * np.sin(4 * x[:, 2])).astype(np.float32)[:, None]


def smooth_config3(log2_hashmap_size=11):
    """Configuration 3 with celu in place of relu: celu has a continuous derivative, so last-bit differences in the
    forward pass cannot flip an activation derivative and the update can be compared entry by entry."""
    cfg = specs.config3(log2_hashmap_size=log2_hashmap_size)
    for layer in cfg["network"][:-1]:
        layer["activation"] = "celu"
    return cfg


def two_grid_config():
    """The mixed-encoding benchmark network (dense grid + hash grid, four features per row, 36 -> 128 -> 64 -> 16 -> 4) with
    small tables and celu in place of relu (continuous derivative: entry-by-entry comparison of gradients)."""
    cfg = specs.config4(log2_hashmap_size=12, dense_resolution=16)
    for layer in cfg["network"]:
        if layer["activation"] == "relu":
            layer["activation"] = "celu"
    return cfg


def dims_config(dims):
    return specs.grid_net(dims, [specs.hashgrid(dims, 6, 2, 11, 4, 96)], [32, 2], ["celu", "identity"])


@pytest.fixture
def kernel_path(request):
    """Library-wide kernel path for one test (2: level-major encoding pass for every grid network, which the automatic
    choice takes only for large gather-dominated batches), restored afterwards."""
    from qmlp import bindings
    bindings.QuickMLP.set_kernel_path(request.param)
    yield request.param
    bindings.QuickMLP.set_kernel_path(0)


@pytest.fixture
def tuning(request):
    """Library-wide tuning switches of the training step for one test, restored to automatic afterwards."""
    from qmlp import bindings
    for key, value in request.param.items():
        bindings.QuickMLP.set_tuning(key, value)
    yield request.param
    for key in ("sort_points", "split_scatter"):
        bindings.QuickMLP.set_tuning(key, -1)
    bindings.QuickMLP.set_tuning("scatter_runs", 1)


SORT_MODES = [{"sort_points": 0}, {"sort_points": 1}, {"sort_points": 1, "scatter_runs": 0}]
SORT_IDS = ["unsorted", "sorted", "sorted_noruns"]


@pytest.mark.parametrize("tuning", SORT_MODES, indirect=True, ids=SORT_IDS)
@pytest.mark.parametrize("kernel_path", [0, 2], indirect=True)
@pytest.mark.parametrize("half_tables", [True, False])
def test_training_steps_match_oracle(half_tables, kernel_path, tuning):
    import torch
    from qmlp import bindings
    from qmlp.trainer import FusedTrainer
    cfg = smooth_config3()
    spec = oracle.parse_spec(cfg)
    net = bindings.Network(json.dumps(cfg))
    n, steps, lr = 2048, 3, 1e-2
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.05).astype(np.float32)
    table = helpers.grid_tables(spec, scale=0.1)[0]
    tr = FusedTrainer(net, lr=lr, grid_half_copy=half_tables)
    tr.set_parameters(torch.from_numpy(params).cuda(), [torch.from_numpy(table).cuda()])

    p_w, p_t = params.copy(), table.copy()
    m_w, v_w, m_t, v_t = (np.zeros_like(a) for a in (p_w, p_w, p_t, p_t))
    for step in range(1, steps + 1):
        x = helpers.uniform(100 + step, 1, (n, 3))
        t = _target(x)
        tr.step(torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda())
        # oracle: half working copies of the master parameters, gradients of mean squared error, Adam
        w16 = p_w.astype(np.float16)
        t16 = p_t.astype(np.float16).astype(np.float32) if half_tables else p_t
        out = oracle.network_forward(spec, w16, x, [t16], half=True)
        adj = oracle.mse_loss_grad(out, t)
        g = oracle.network_backward(spec, w16, x, adj, [t16], half=True, want_input=False)
        oracle.adam_step(p_w, g.grad_params, m_w, v_w, step, lr=lr)
        oracle.adam_step(p_t, g.grad_encodings[0], m_t, v_t, step, lr=lr)
    torch.cuda.synchronize()
    got_w = tr.segment(tr.master, 0).cpu().numpy()
    got_t = tr.segment(tr.master, 1).cpu().numpy()
    # Adam's first steps move every touched parameter by ~lr regardless of gradient size, so compare the update
    helpers.assert_close(got_w - params, p_w - params, "network update", rtol=5e-2, atol=2e-3, max_violations=0.02)
    helpers.assert_close(got_t - table, p_t - table, "grid update", rtol=5e-2, atol=2e-3, max_violations=0.02)
    assert float(tr.gradient.abs().max()) == 0.0            # the update zeroes the gradient buffer
    assert torch.equal(tr.half[: spec.num_parameters], tr.master[: spec.num_parameters].half())
    loss = tr.mean_loss(n * steps)
    assert np.isfinite(loss) and loss > 0


def _step_gradients(cfg, x, t, half_tables, table_scale=0.1):
    """Fused gradient vector of one step (before Adam) from the CUDA kernels, with the trainer and the oracle inputs."""
    import torch
    from qmlp import bindings
    from qmlp.trainer import FusedTrainer
    spec = oracle.parse_spec(cfg)
    net = bindings.Network(json.dumps(cfg))
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.05).astype(np.float32)
    tables = helpers.grid_tables(spec, scale=table_scale)
    tr = FusedTrainer(net, grid_half_copy=half_tables)
    tr.set_parameters(torch.from_numpy(params).cuda(), [torch.from_numpy(tb).cuda() if tb is not None else None for tb in tables])
    tr.backend.gradients(torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda(), x.shape[0], tr.loss_sum)
    torch.cuda.synchronize()
    return tr, spec, params, tables


def _targets4(x):
    return np.stack([np.sin(8 * x[:, 0]) * np.cos(6 * x[:, 1]), np.cos(5 * x[:, 2]), np.sin(3 * x[:, 0] + 2 * x[:, 1]),
                     np.cos(4 * x[:, 1]) * np.sin(7 * x[:, 2])], 1).astype(np.float32)


@pytest.mark.parametrize("tuning", SORT_MODES + [{"sort_points": 1, "split_scatter": 0}], indirect=True,
                         ids=SORT_IDS + ["sorted_inline_scatter"])
@pytest.mark.parametrize("kernel_path", [0, 2], indirect=True)
def test_step_gradients_two_grids_four_features(kernel_path, tuning):
    """Dense grid + hash grid with four features per row on the same inputs (the shape of the mixed-encoding benchmark
    network, small tables): weight, bias and both table gradients of one step against the oracle, on every path of the
    step (points sorted into bins or not, runs of points in one cell summed in registers or not, scatter inside the backward
    kernel or separate)."""
    cfg = two_grid_config()
    n = 6000
    x = helpers.uniform(21, 1, (n, 3))
    t = _targets4(x)
    tr, spec, params, tables = _step_gradients(cfg, x, t, half_tables=True)
    w16 = params.astype(np.float16)
    t16 = [tb.astype(np.float16).astype(np.float32) for tb in tables]
    out = oracle.network_forward(spec, w16, x, t16, half=True)
    g = oracle.network_backward(spec, w16, x, oracle.mse_loss_grad(out, t), t16, half=True, want_input=False)
    got_w = tr.segment(tr.gradient, 0).cpu().numpy()
    scale = float(np.abs(g.grad_params).max())
    helpers.assert_close(got_w, g.grad_params, "weight and bias gradients", rtol=5e-2, atol=2e-2 * scale, max_violations=0.02)
    for i in range(2):
        got = tr.segment(tr.gradient, 1 + i).cpu().numpy()
        want = g.grad_encodings[i]
        helpers.assert_close(got, want, f"table gradient of encoding {i}", rtol=5e-2, atol=2e-2 * float(np.abs(want).max()),
                             max_violations=0.02)
        # every contribution arrives exactly once: the totals agree far more closely than single rows
        assert abs(float(got.sum()) - float(want.sum())) <= 2e-2 * float(np.abs(want).sum())


@pytest.mark.parametrize("dims", [2, 4])
def test_sorted_step_other_dimensions(dims):
    """Bins of the point sort in two and four dimensions (512 x 512 and 16^4 bins): sorted and unsorted steps give the same
    gradients, and both match the oracle."""
    import torch
    from qmlp import bindings
    cfg = dims_config(dims)
    n = 5000
    x = helpers.uniform(31, dims, (n, dims), -0.05, 1.05)          # some points outside the bounding box: border bins
    t = helpers.uniform(31, 9, (n, 2), -1.0, 1.0)
    grads = []
    try:
        for sort in (0, 1):
            bindings.QuickMLP.set_tuning("sort_points", sort)
            tr, spec, params, tables = _step_gradients(cfg, x, t, half_tables=False)
            grads.append(tr.gradient.cpu().numpy().copy())
    finally:
        bindings.QuickMLP.set_tuning("sort_points", -1)
    scale = float(np.abs(grads[0]).max())
    helpers.assert_close(grads[1], grads[0], "sorted against unsorted step", rtol=1e-2, atol=2e-3 * scale, max_violations=0.002)
    w16 = params.astype(np.float16)
    out = oracle.network_forward(spec, w16, x, tables, half=True)
    g = oracle.network_backward(spec, w16, x, oracle.mse_loss_grad(out, t), tables, half=True, want_input=False)
    want = g.grad_encodings[0]
    got = grads[1][tr.backend.segments[1]:tr.backend.segments[1] + want.size]
    helpers.assert_close(got, want, "table gradient", rtol=5e-2, atol=2e-2 * float(np.abs(want).max()), max_violations=0.02)


def test_loss_decreases_on_config3_small():
    import torch
    from qmlp import bindings
    from qmlp.trainer import FusedTrainer
    cfg = specs.config3(log2_hashmap_size=14)
    spec = oracle.parse_spec(cfg)
    net = bindings.Network(json.dumps(cfg))
    tr = FusedTrainer(net, lr=1e-2)
    params = helpers.xavier_parameters(spec, cfg).astype(np.float32)
    table = helpers.grid_tables(spec, scale=1e-4)[0]
    tr.set_parameters(torch.from_numpy(params).cuda(), [torch.from_numpy(table).cuda()])
    n = 1 << 14
    losses = []
    for step in range(60):
        x = helpers.uniform(7, step, (n, 3))
        tr.step(torch.from_numpy(x).cuda(), torch.from_numpy(_target(x)).cuda())
        if step % 20 == 19:
            losses.append(tr.mean_loss(n * 20))
    assert losses[-1] < 0.5 * losses[0], losses


def test_step_from_host_memory_with_prefetch():
    """step_host (batch in page-locked host memory, the following batch uploaded on a copy stream while the step runs)
    leaves exactly the parameters that step() leaves on the same batches; gradients come from atomic sums, so "exactly"
    is up to their summation order."""
    import torch
    from qmlp import bindings
    from qmlp.trainer import FusedTrainer
    cfg = smooth_config3()
    spec = oracle.parse_spec(cfg)
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.05).astype(np.float32)
    table = helpers.grid_tables(spec, scale=0.1)[0]
    batches = []
    for i in range(4):
        x = helpers.uniform(11, 10 + i, (3000, 3))
        batches.append((torch.from_numpy(x).pin_memory(), torch.from_numpy(_target(x)).pin_memory()))

    def run(host):
        tr = FusedTrainer(bindings.Network(json.dumps(cfg)), lr=1e-2)
        tr.set_parameters(torch.from_numpy(params).cuda(), [torch.from_numpy(table).cuda()])
        for i, (x, t) in enumerate(batches):
            if host:
                nxt = batches[i + 1] if i + 1 < len(batches) and i != 1 else None    # one step without a prefetch in between
                tr.step_host(x, t, next_batch=nxt)
            else:
                tr.step(x.cuda(), t.cuda())
        torch.cuda.synchronize()
        return tr.master.cpu().numpy(), float(tr.loss_sum.item())

    m_dev, l_dev = run(False)
    m_host, l_host = run(True)
    assert abs(l_dev - l_host) <= 1e-4 * max(1.0, abs(l_dev))
    # Adam turns a gradient entry into a step of about lr whatever its size, so entries whose gradient is rounding noise
    # (atomic sums in a different order) may move differently: nearly all entries agree closely, none by more than the
    # four steps of lr = 1e-2 that were taken
    diff = np.abs(m_host - m_dev)
    assert float((diff > 2e-4 + 1e-3 * np.abs(m_dev)).mean()) < 0.01 and float(diff.max()) <= 4.1e-2
    assert bindings.QuickMLP.device_status() == 0
