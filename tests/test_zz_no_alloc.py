"""The allocation-free forward entry point (qmlp_network_forward_static_scratch), through the C ABI.

It exists for callers that cannot allocate device memory at call time (a plug-in on a fixed memory budget, a
latency-critical loop): the forward stash lives in a fixed device array inside the library. The test runs it twice in
a row, on batches of different size, and compares each result with the regular entry point (qmlp_network_forward with
a caller-allocated stash), which runs the same kernel. This file is named so that pytest collects it last.
"""
import ctypes as C
import json

import numpy as np
import pytest

import helpers
import qmlp_oracle as oracle
import specs

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 32 << 20   # QMLP_STATIC_SCRATCH_BYTES in include/qmlp_b200.h


def _network(cfg):
    import torch
    from qmlp import _capi, bindings
    from qmlp._capi import check, lib, wrap
    spec = oracle.parse_spec(cfg)
    net = bindings.Network(json.dumps(cfg))
    params = torch.from_numpy(helpers.xavier_parameters(spec, cfg, bias_scale=0.1)).cuda()
    tables = [torch.from_numpy(t).cuda() if t is not None else None for t in helpers.grid_tables(spec)]
    check(lib().qmlp_network_set_parameter(net._h, wrap(params), _capi.QMLP_INFERENCE))
    for i, t in enumerate(tables):
        if t is not None:
            net.encoding(i).set_parameter(t, _capi.QMLP_INFERENCE)
    return spec, net, (params, tables)   # keep the parameter tensors alive


@pytest.mark.parametrize("cfg", [specs.config3(log2_hashmap_size=12), specs.config2()], ids=["hashgrid", "identity"])
def test_static_scratch_forward_matches_regular_forward(cfg):
    import torch
    from qmlp._capi import check, lib, wrap
    spec, net, keep = _network(cfg)
    for call, n in enumerate((4099, 777)):          # two calls in a row; the second leaves stale rows in the array
        x = torch.from_numpy(helpers.uniform(11, call, (n, spec.num_inputs))).cuda()
        expected = torch.empty((n, spec.num_outputs), device="cuda")
        stash = torch.empty((net.forward_memory(n),), dtype=torch.uint8, device="cuda")
        check(lib().qmlp_network_forward(net._h, wrap(x), wrap(expected), stash.data_ptr(), None))
        got = torch.full((n, spec.num_outputs), float("nan"), device="cuda")
        check(lib().qmlp_network_forward_static_scratch(net._h, wrap(x), wrap(got), None))
        torch.cuda.synchronize()
        helpers.assert_close(got.cpu().numpy(), expected.cpu().numpy(), f"static-scratch forward, call {call}")
        ref = oracle.network_forward(spec, keep[0].cpu().numpy(), x.cpu().numpy(),
                                     [t.cpu().numpy() if t is not None else None for t in keep[1]], half=True)
        helpers.assert_close(got.cpu().numpy(), ref, f"static-scratch forward vs oracle, call {call}", max_violations=0.01)


def test_static_scratch_rejects_oversized_batches():
    import torch
    from qmlp._capi import QmlpError, check, lib, wrap
    spec, net, keep = _network(specs.config2())
    per_point = net.forward_memory(32) // 32
    too_many = STATIC_SCRATCH_BYTES // per_point + 64
    assert net.forward_memory(too_many) > STATIC_SCRATCH_BYTES
    x = torch.zeros((too_many, spec.num_inputs), device="cuda")
    out = torch.empty((too_many, spec.num_outputs), device="cuda")
    with pytest.raises(QmlpError, match="static scratch"):
        check(lib().qmlp_network_forward_static_scratch(net._h, wrap(x), wrap(out), None))
    largest = STATIC_SCRATCH_BYTES // per_point // 32 * 32          # the largest batch that fits still runs
    check(lib().qmlp_network_forward_static_scratch(net._h, wrap(x[:largest]), wrap(out[:largest]), None))
    torch.cuda.synchronize()
