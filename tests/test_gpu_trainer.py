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


def _target(x):   # smooth analytic target of BASELINE config 3
    return (np.sin(8 * x[:, 0]) * np.cos(6 * x[:, 1]) * np.sin(4 * x[:, 2])).astype(np.float32)[:, None]


def smooth_config3(log2_hashmap_size=11):
    """Configuration 3 with celu in place of relu: celu has a continuous derivative, so last-bit differences in the
    forward pass cannot flip an activation derivative and the update can be compared entry by entry."""
    cfg = specs.config3(log2_hashmap_size=log2_hashmap_size)
    for layer in cfg["network"][:-1]:
        layer["activation"] = "celu"
    return cfg


@pytest.fixture
def kernel_path(request):
    """Library-wide kernel path for one test (2: level-major encoding pass for every grid network, which the automatic
    choice takes only for large gather-dominated batches), restored afterwards."""
    from qmlp import bindings
    bindings.QuickMLP.set_kernel_path(request.param)
    yield request.param
    bindings.QuickMLP.set_kernel_path(0)


@pytest.mark.parametrize("kernel_path", [0, 2], indirect=True)
@pytest.mark.parametrize("half_tables", [True, False])
def test_training_steps_match_oracle(half_tables, kernel_path):
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
