"""The allocation-free forward entry point (qmlp_network_forward_static_scratch), through the C ABI.

It exists for callers that cannot allocate device memory at call time (a plug-in on a fixed memory budget, a
latency-critical loop): the forward stash lives in a fixed device array inside the library. The test runs it twice in
a row, on batches of different size, and compares each result with the regular entry point (qmlp_network_forward with
a caller-allocated stash), which runs the same kernel; it also compares the stash the call leaves in the fixed array,
byte for byte, with the caller-allocated one, feeds it to the backward pass, and checks that the call leaves the amount
of free device memory unchanged. This file is named so that pytest collects it last.
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


def _static_scratch_view(num_bytes):
    """The first `num_bytes` of the library's fixed array on the current device as a torch uint8 tensor (no copy)."""
    import torch
    from qmlp._capi import check, lib
    address, size = C.c_void_p(), C.c_size_t()
    check(lib().qmlp_static_scratch(C.byref(address), C.byref(size)))
    assert size.value == STATIC_SCRATCH_BYTES and address.value % 256 == 0 and num_bytes <= size.value

    class _Array:   # __cuda_array_interface__ of a foreign device pointer
        __cuda_array_interface__ = {"shape": (num_bytes,), "typestr": "|u1", "data": (address.value, False), "version": 3}
    return torch.as_tensor(_Array(), device="cuda"), address.value


@pytest.mark.parametrize("cfg", [specs.config3(log2_hashmap_size=12), specs.config2()], ids=["hashgrid", "identity"])
def test_static_scratch_stash_feeds_the_backward_pass(cfg):
    """The stash in the fixed array equals the one qmlp_network_forward writes into caller memory, and
    qmlp_network_adjoint accepts the array as its forward scratch: same input, weight and table gradients."""
    import torch
    from qmlp import _capi
    from qmlp._capi import check, lib, wrap
    spec, net, keep = _network(cfg)
    n = 2051                                                       # not a multiple of 32: the last tile is ragged
    x = torch.from_numpy(helpers.uniform(12, 0, (n, spec.num_inputs))).cuda()
    adj = torch.from_numpy(helpers.uniform(12, 1, (n, spec.num_outputs), -1.0, 1.0)).cuda()
    out_a = torch.empty((n, spec.num_outputs), device="cuda")
    out_b = torch.empty((n, spec.num_outputs), device="cuda")
    nbytes = net.forward_memory(n)
    stash = torch.zeros((nbytes,), dtype=torch.uint8, device="cuda")
    view, address = _static_scratch_view(nbytes)
    view.zero_()                                                   # rows of the ragged tail are never written by either call
    check(lib().qmlp_network_forward(net._h, wrap(x), wrap(out_a), stash.data_ptr(), None))
    check(lib().qmlp_network_forward_static_scratch(net._h, wrap(x), wrap(out_b), None))
    torch.cuda.synchronize()
    assert torch.equal(view, stash), "the stash in the fixed array differs from the caller-allocated one"

    flags = _capi.GRADIENTS_INPUT | _capi.GRADIENTS_NETWORK_WEIGHTS | _capi.GRADIENTS_INPUT_ENCODINGS
    results = []
    for forward_scratch in (stash.data_ptr(), address):
        gw = torch.zeros((net.num_network_parameters(),), device="cuda")
        check(lib().qmlp_network_set_parameter(net._h, wrap(gw), _capi.QMLP_GRADIENTS))
        gts = []
        for i, t in enumerate(keep[1]):
            g = torch.zeros(t.shape, device="cuda") if t is not None else None
            if g is not None:
                net.encoding(i).set_parameter(g, _capi.QMLP_GRADIENTS)
            gts.append(g)
        gx = torch.zeros_like(x)
        tmp = torch.empty((max(net.adjoint_memory(n, flags), 16),), dtype=torch.uint8, device="cuda")
        agx = wrap(gx)
        check(lib().qmlp_network_adjoint(net._h, wrap(x), wrap(adj), flags, C.byref(agx), forward_scratch, tmp.data_ptr(), None))
        torch.cuda.synchronize()
        results.append((gx, gw, gts))
    (gx_a, gw_a, gt_a), (gx_b, gw_b, gt_b) = results
    helpers.assert_close(gx_b.cpu().numpy(), gx_a.cpu().numpy(), "input gradient from the fixed-array stash")
    # the sums are accumulated with atomics in an order that differs from run to run
    helpers.assert_close(gw_b.cpu().numpy(), gw_a.cpu().numpy(), "weight gradient from the fixed-array stash", atol=1e-3 * float(gw_a.abs().max()))
    for a, b in zip(gt_a, gt_b):
        if a is not None:
            helpers.assert_close(b.cpu().numpy(), a.cpu().numpy(), "table gradient from the fixed-array stash", atol=1e-3 * float(a.abs().max()))


def test_static_scratch_call_allocates_no_device_memory():
    """The property the entry point exists for: once the network's kernels are loaded, a call changes neither the free
    device memory the driver reports nor what torch's allocator holds."""
    import torch
    from qmlp._capi import check, lib, wrap
    spec, net, keep = _network(specs.config2())
    x = torch.from_numpy(helpers.uniform(13, 0, (4096, spec.num_inputs))).cuda()
    out = torch.empty((4096, spec.num_outputs), device="cuda")
    vx, vo = wrap(x), wrap(out)
    check(lib().qmlp_network_forward_static_scratch(net._h, vx, vo, None))   # first call: kernels loaded, address resolved
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    reserved_before = torch.cuda.memory_reserved()
    for _ in range(3):
        check(lib().qmlp_network_forward_static_scratch(net._h, vx, vo, None))
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)
    assert torch.cuda.memory_reserved() == reserved_before


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
