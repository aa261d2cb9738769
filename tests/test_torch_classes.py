"""The TorchScript custom classes torch.classes.qmlp_cu.{QuickMLP, Network, Encoding, Activation} (the reference's
src_cpp/pytorch-bindings/src/bindings.cpp:102-122, bind_network.cpp:348-411): registration, method set, scripting of a
module that holds a Network, save / load and pickling need no GPU; numerics and autograd run on one."""
import io
import json
import pickle

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs


def _classes():
    import qmlp
    return qmlp.load_torch_classes()


def _holder_module():
    """A scriptable module that owns a Network custom class, its weights and one grid table."""
    import torch

    class Holder(torch.nn.Module):
        def __init__(self, net, weights, table):
            super().__init__()
            self.net = net
            self.weights = torch.nn.Parameter(weights)
            self.table = torch.nn.Parameter(table)

        def forward(self, x: torch.Tensor) -> torch.Tensor:
            return self.net.forward(x, self.weights, [self.table])

    return Holder


def test_method_set_and_layout():
    cu = _classes()
    cfg = specs.config3(log2_hashmap_size=12)
    spec = oracle.parse_spec(cfg)
    net = cu.Network(json.dumps(cfg), ".")
    assert (net.channels_in(), net.channels_out(), net.num_layers(), net.num_encodings()) == (3, 1, len(spec.layers), 1)
    assert net.num_network_parameters() == spec.num_parameters
    assert cu.Network.MatrixSize() == 16 and cu.Network.WarpSize() == 32 and cu.Network.MaxSharedMemoryBytes() > 48 * 1024
    assert json.loads(net.cfg()) == cfg and net.parent() == "."
    enc = net.encoding(0)
    assert enc.has_parameters() and enc.num_output_channels() == 32 and enc.max_input_channel() == 2
    assert json.loads(enc.to_json())["id"] == "HashGrid"
    for name in ("create_inference_parameters", "initialize_inference_parameters", "parameter_view", "inference", "forward"):
        assert hasattr(net, name)
    for name in ("create_inference_parameters", "create_gradient_parameters", "inference", "adjoint", "inference_with_parameter",
                 "adjoint_with_parameter", "forward", "forward_with_parameter"):
        assert hasattr(enc, name)
    act = cu.Activation("celu")
    assert all(hasattr(act, n) for n in ("inference", "adjoint", "forward"))
    assert isinstance(cu.QuickMLP.is_cuda_available(), bool)
    cu.QuickMLP.set_log_level("warn")
    with pytest.raises(RuntimeError, match="configuration error"):
        cu.Network(json.dumps({"num_inputs": 3, "num_outputs": 1, "encodings": [{"id": "NoSuchEncoding"}], "network": []}), ".")
    # pickling = configuration strings (bind_network.cpp:403-410)
    assert pickle.loads(pickle.dumps(net)).num_network_parameters() == spec.num_parameters
    assert pickle.loads(pickle.dumps(enc)).num_output_channels() == 32
    # the weight view shares memory with the flat vector
    import torch
    flat = torch.zeros(spec.num_parameters, dtype=torch.float16)
    w1 = net.parameter_view(1, False, flat)
    l1 = spec.layers[1]
    assert tuple(w1.shape) == (l1.channels_out, l1.channels_in)
    w1.fill_(1.0)
    assert float(flat[l1.weights_start:l1.weights_start + l1.channels_in * l1.channels_out].sum()) == l1.channels_in * l1.channels_out
    assert float(flat.sum()) == l1.channels_in * l1.channels_out


def test_module_with_a_network_scripts_saves_and_loads():
    import torch
    cu = _classes()
    cfg = specs.config3(log2_hashmap_size=12)
    spec = oracle.parse_spec(cfg)
    net = cu.Network(json.dumps(cfg), ".")
    module = _holder_module()(net, torch.zeros(spec.num_parameters, dtype=torch.float16), torch.zeros(spec.encodings[0].num_parameters))
    scripted = torch.jit.script(module)
    buf = io.BytesIO()
    torch.jit.save(scripted, buf)
    buf.seek(0)
    loaded = torch.jit.load(buf)
    assert json.loads(loaded.net.cfg()) == cfg and loaded.net.num_network_parameters() == spec.num_parameters


@pytest.mark.gpu
def test_scripted_network_matches_the_oracle_and_differentiates():
    import torch
    cu = _classes()
    cfg = specs.config3(log2_hashmap_size=12)
    spec = oracle.parse_spec(cfg)
    params = helpers.xavier_parameters(spec, cfg, bias_scale=0.05)
    table = helpers.grid_tables(spec, scale=0.5)[0]
    n = 3001
    x = helpers.uniform(71, 1, (n, 3))
    adj = helpers.uniform(71, 2, (n, 1), -1.0, 1.0)
    net = cu.Network(json.dumps(cfg), ".")
    module = _holder_module()(net, torch.from_numpy(params), torch.from_numpy(table)).cuda()
    scripted = torch.jit.script(module)
    tx = torch.from_numpy(x).cuda().requires_grad_(True)
    out = scripted(tx)
    expected = oracle.network_forward(spec, params, x, [table], half=True)
    helpers.assert_close(out.detach().cpu().numpy(), expected, "scripted forward", max_violations=0.01)
    out.backward(torch.from_numpy(adj).cuda())
    g = oracle.network_backward(spec, params, x, adj, [table], half=True)
    helpers.assert_close(scripted.weights.grad.float().cpu().numpy(), g.grad_params, "weight gradient", rtol=helpers.RTOL_WGRAD,
                         atol=2e-2 * float(np.abs(g.grad_params).max()), max_violations=0.05)
    helpers.assert_close(scripted.table.grad.cpu().numpy(), g.grad_encodings[0], "table gradient", rtol=5e-2,
                         atol=2e-2 * float(np.abs(g.grad_encodings[0]).max()), max_violations=0.02)
    helpers.assert_close(tx.grad.cpu().numpy(), g.adj_input, "input gradient", rtol=5e-2, atol=2e-2 * float(np.abs(g.adj_input).max()),
                         max_violations=0.05)
    # without gradients the call is the inference kernel, same values
    with torch.no_grad():
        again = scripted(torch.from_numpy(x).cuda())
    helpers.assert_close(again.cpu().numpy(), expected, "scripted inference", max_violations=0.01)
    # the same classes agree with the ctypes-based Python classes of the package
    from qmlp import bindings
    ref = bindings.Network(json.dumps(cfg)).inference(torch.from_numpy(x).cuda(), torch.from_numpy(params).cuda(), [torch.from_numpy(table).cuda()])
    assert torch.allclose(again, ref, rtol=1e-3, atol=1e-3)


@pytest.mark.gpu
def test_encoding_and_activation_classes():
    import torch
    cu = _classes()
    cfg = specs.hashgrid(3, 4, 2, 10, 4, 32)
    oe = oracle.parse_encoding(cfg)
    enc = cu.Encoding(json.dumps(cfg))
    x = helpers.uniform(72, 1, (500, 3))
    table = helpers.uniform(72, 2, (oe.num_parameters,), -1, 1)
    tx = torch.from_numpy(x).cuda().requires_grad_(True)
    tp = torch.from_numpy(table).cuda().requires_grad_(True)
    out = enc.forward_with_parameter(tx, tp)
    helpers.assert_close(out.detach().cpu().numpy(), oracle.grid_forward(oe, x, table), "encoding forward", rtol=1e-4, atol=1e-4)
    adj = helpers.uniform(72, 3, (500, oe.num_outputs), -1, 1)
    out.backward(torch.from_numpy(adj).cuda())
    gp, gx = oracle.grid_adjoint(oe, x, table, adj, True, True)
    helpers.assert_close(tp.grad.cpu().numpy(), gp, "encoding parameter gradient", rtol=1e-4, atol=1e-4)
    helpers.assert_close(tx.grad.cpu().numpy(), gx, "encoding input gradient", rtol=1e-3, atol=1e-3)
    act = cu.Activation("sine")
    h = torch.from_numpy(helpers.uniform(72, 4, (64, 16), -2, 2)).cuda().half().requires_grad_(True)
    z = act.forward(h)
    assert torch.allclose(z.float(), torch.sin(h.float()), atol=2e-3)
    z.backward(torch.ones_like(z))
    assert torch.allclose(h.grad.float(), torch.cos(h.detach().float()), atol=5e-3)
