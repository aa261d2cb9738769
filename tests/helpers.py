"""Shared helpers of the parity tests: deterministic inputs, parameter initialisation, tolerance checks."""
import json
import math

import numpy as np

import qmlp_oracle as oracle

# tolerance for fp16 results: the stated target of 1e-2 relative, plus the absolute floor the reference's own
# comparison uses (tests_py/qmlp_tests/test_network_base.py:95-96)
RTOL, ATOL = 1e-2, 1e-3
RTOL_WGRAD = 1e-1          # the reference's bound for weight gradients (test_network_base.py:97)
MAX_VIOLATIONS = 0.05      # the reference accepts up to 5 % of entries outside (test_network_base.py:54-67)


def violation_fraction(actual, expected, rtol=RTOL, atol=ATOL):
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    assert actual.shape == expected.shape, (actual.shape, expected.shape)
    bad = ~(np.abs(actual - expected) <= rtol * np.abs(expected) + atol)
    return float(np.mean(bad)) if bad.size else 0.0


def assert_close(actual, expected, name, rtol=RTOL, atol=ATOL, max_violations=0.0):
    frac = violation_fraction(actual, expected, rtol, atol)
    if frac > max_violations:
        a = np.asarray(actual, dtype=np.float64); e = np.asarray(expected, dtype=np.float64)
        err = np.abs(a - e)
        i = np.unravel_index(np.argmax(err), err.shape)
        raise AssertionError(f"{name}: {frac * 100:.3f}% of entries outside rtol={rtol} atol={atol} "
                             f"(allowed {max_violations * 100:.2f}%); worst at {i}: actual={a[i]} expected={e[i]}")


def uniform(seed, tensor_id, shape, lo=0.0, hi=1.0):
    n = int(np.prod(shape))
    return oracle.splitmix_uniform(seed, tensor_id, n, lo, hi).reshape(shape)


def xavier_parameters(spec: "oracle.NetSpec", cfg: dict, seed=7, bias_scale=0.0):
    """fp16 parameter vector: Xavier-uniform on the unpadded block, padding zero, biases U(+-bias_scale)."""
    p = np.zeros(spec.num_parameters, dtype=np.float32)
    n_in = spec.encoded_channels
    for i, (l, lc) in enumerate(zip(spec.layers, cfg["network"])):
        n_out = lc["n_out"]
        bound = math.sqrt(6.0 / (n_in + n_out))
        w = np.zeros((l.channels_out, l.channels_in), dtype=np.float32)
        w[:n_out, :n_in] = uniform(seed, 100 + i, (n_out, n_in), -bound, bound)
        p[l.weights_start:l.weights_start + w.size] = w.ravel()
        if l.use_bias and bias_scale > 0:
            b = np.zeros(l.channels_out, dtype=np.float32)
            b[:n_out] = uniform(seed, 200 + i, (n_out,), -bias_scale, bias_scale)
            p[l.bias_start:l.bias_start + l.channels_out] = b
        n_in = n_out
    return p.astype(np.float16)


def reference_style_parameters(spec: "oracle.NetSpec", seed=11):
    """U(+-1/sqrt(Cin_padded)) over every padded entry, the distribution of
    FusedNetwork::initializeInferenceParameters (src_cpp/src/fused_network.cpp:280-307)."""
    p = np.zeros(spec.num_parameters, dtype=np.float32)
    for i, l in enumerate(spec.layers):
        bound = 1.0 / math.sqrt(l.channels_in)
        n = l.channels_in * l.channels_out
        p[l.weights_start:l.weights_start + n] = uniform(seed, 300 + i, (n,), -bound, bound)
        if l.use_bias:
            p[l.bias_start:l.bias_start + l.channels_out] = uniform(seed, 400 + i, (l.channels_out,), -bound, bound)
    return p.astype(np.float16)


def grid_tables(spec: "oracle.NetSpec", seed=13, scale=1.0):
    """One fp32 table per encoding (None for encodings without parameters), U(+-scale)."""
    out = []
    for i, e in enumerate(spec.encodings):
        if not e.num_parameters:
            out.append(None)
        elif e.num_parameters > (1 << 22):
            # full-size benchmark tables (up to 220 M entries): numpy's generator is an order of magnitude quicker than
            # the portable counter-based one and nothing outside this process has to reproduce these values
            rng = np.random.default_rng(seed * 1000 + i)
            out.append(((rng.random(e.num_parameters, dtype=np.float32) * 2 - 1) * np.float32(scale)).astype(np.float32))
        else:
            out.append(uniform(seed, 500 + i, (e.num_parameters,), -scale, scale))
    return out


def pack_parameters(spec: "oracle.NetSpec", weights, biases):
    """Unpadded per-layer (n_out, n_in) weights / (n_out,) biases -> the padded flat fp32 vector (padding zero)."""
    p = np.zeros(spec.num_parameters, dtype=np.float32)
    for i, l in enumerate(spec.layers):
        w = np.zeros((l.channels_out, l.channels_in), dtype=np.float32)
        w[:weights[i].shape[0], :weights[i].shape[1]] = weights[i]
        p[l.weights_start:l.weights_start + w.size] = w.ravel()
        if l.use_bias and biases[i] is not None:
            p[l.bias_start:l.bias_start + biases[i].shape[0]] = biases[i]
    return p


def load_golden(name):
    import os
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", name))


def stash_rows(flat, n32, width):
    """Row-major (N32, width) copy of one pre-activation or delta matrix of the stash. The kernels store such a matrix
    as tiles of 32 points, each tile in blocks of 8 points x 8 channels, block (cb, rb) of a tile at (cb * 4 + rb) * 64
    halfs and point-major inside (one mma fragment register of a warp = one 128-byte block). numpy array or torch tensor."""
    blocks = flat.reshape(n32 // 32, width // 8, 4, 8, 8)            # tile, cb, rb, point, channel
    if isinstance(blocks, np.ndarray):
        return np.ascontiguousarray(blocks.transpose(0, 2, 3, 1, 4)).reshape(n32, width)
    return blocks.permute(0, 2, 3, 1, 4).contiguous().reshape(n32, width)


def stash_rows_all(flat, n32, widths):
    """Row-major copies of consecutive stash matrices of the given widths, concatenated into one flat array again
    (the layout the reference's kernels use for the same buffers)."""
    out, off = [], 0
    for w in widths:
        out.append(stash_rows(flat[off:off + n32 * w], n32, w).reshape(-1))
        off += n32 * w
    if isinstance(out[0], np.ndarray):
        return np.concatenate(out)
    import torch
    return torch.cat(out)
