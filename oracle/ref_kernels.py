"""ctypes front end of the reference inference kernels that build_ref_kernels.py builds.  TEST INFRASTRUCTURE: loaded by
tests/ and by bench.py's reference leg only, never by the product."""
import ctypes as C

import numpy as np

import build_ref_kernels
import qmlp_oracle as oracle


class _RefGrid(C.Structure):
    _fields_ = [("table", C.c_void_p), ("grad", C.c_void_p), ("levels", C.POINTER(C.c_int)), ("boxMin", C.POINTER(C.c_float)),
                ("boxInvSize", C.POINTER(C.c_float))]


def _grid_array(spec, tables, grads=None):
    """Host array of RefGrid entries (one per encoding with parameters) and the numpy arrays it points into."""
    import torch
    keep, grids = [], []
    for i, (e, t) in enumerate(zip(spec.encodings, tables)):
        if not e.num_parameters:
            continue
        assert t is not None and t.dtype == torch.float32 and t.is_contiguous() and t.numel() == e.num_parameters
        g = grads[i] if grads is not None else None
        assert g is None or (g.dtype == torch.float32 and g.is_contiguous() and g.numel() == e.num_parameters)
        lv = np.array([[l.memory_offset, l.resolution, l.hash_grid_size, int(l.hashed)] for l in e.levels], dtype=np.int32)
        bmin = np.ascontiguousarray(e.box_min, dtype=np.float32)
        binv = np.ascontiguousarray(e.box_inv_size, dtype=np.float32)
        keep += [lv, bmin, binv]
        grids.append(_RefGrid(t.data_ptr(), g.data_ptr() if g is not None else None, lv.ctypes.data_as(C.POINTER(C.c_int)),
                              bmin.ctypes.data_as(C.POINTER(C.c_float)), binv.ctypes.data_as(C.POINTER(C.c_float))))
    return (_RefGrid * max(1, len(grids)))(*grids), keep


class ReferenceInference:
    """The reference's NetworkKernelInferenceAndForward for one configuration (src_cpp/include/qmlp/kernels/
    network_forward.cuh), launched as FusedNetwork::inference launches it."""

    def __init__(self, cfg):
        path = build_ref_kernels.build(cfg)
        if path is None:
            raise FileNotFoundError("the reference kernel for this configuration has not been built")
        self.lib = C.CDLL(path)
        self.lib.ref_inference.restype = C.c_int
        self.lib.ref_inference.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(_RefGrid), C.c_int,
                                           C.POINTER(C.c_float), C.POINTER(C.c_int)]
        self.spec = oracle.parse_spec(cfg)
        assert self.lib.ref_num_parameters() == self.spec.num_parameters, "parameter layout differs from the oracle's"
        self.launch_info = None

    def __call__(self, x, params_half, tables, iterations=0):
        """x: (N, Cin) fp32 CUDA tensor; params_half: fp16 CUDA vector; tables: fp32 CUDA tensors (None for encodings
        without parameters). Returns (output tensor, mean milliseconds per launch)."""
        import torch
        assert x.is_cuda and x.dtype == torch.float32 and x.is_contiguous()
        assert params_half.dtype == torch.float16 and params_half.is_contiguous()
        n = x.shape[0]
        out = torch.empty((n, self.spec.num_outputs), dtype=torch.float32, device=x.device)
        arr, keep = _grid_array(self.spec, tables)
        ms = C.c_float(0)
        info = (C.c_int * 3)()
        torch.cuda.synchronize()
        err = self.lib.ref_inference(n, x.data_ptr(), out.data_ptr(), params_half.data_ptr(), arr, iterations, C.byref(ms), info)
        if err != 0:
            raise RuntimeError("reference kernel launch failed with CUDA error %d" % err)
        self.launch_info = tuple(info)
        return out, float(ms.value)


class ReferenceBackward:
    """The reference's NetworkKernelBackward for one configuration (src_cpp/include/qmlp/kernels/network_backward.cuh,
    Layer::adjoint of kernels/layer.cuh:194-265, the encodings' adjoint), with input, weight (delta stash) and encoding
    gradients all enabled, launched as FusedNetwork::adjoint launches it (src_cpp/src/fused_network.cpp:1012-1079)."""

    def __init__(self, cfg):
        path = build_ref_kernels.build(cfg, kind="backward")
        if path is None:
            raise FileNotFoundError("the reference backward kernel for this configuration has not been built")
        self.lib = C.CDLL(path)
        self.lib.ref_backward.restype = C.c_int
        self.lib.ref_backward.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                          C.POINTER(_RefGrid), C.POINTER(C.c_int), C.POINTER(C.c_float)]
        self.last_ms = 0.0
        self.spec = oracle.parse_spec(cfg)
        assert self.lib.ref_num_parameters() == self.spec.num_parameters
        self.stash_halfs = self.lib.ref_stash_halfs_per_point()
        assert self.stash_halfs == sum(l.channels_out for l in self.spec.layers)
        self.launch_info = None

    def __call__(self, x, adj_output, params_half, pre_activations, tables, table_grads):
        """x (N, Cin) fp32; adj_output (N, Cout) fp32; pre_activations: CUDA fp16 tensor of N32 * stash_halfs elements
        ((N32, Cout_l) row-major per layer, layers in order). table_grads are accumulated into.
        Returns (adj_input (N, Cin) fp32, deltas: fp16 tensor laid out like pre_activations)."""
        import torch
        n = x.shape[0]
        n32 = (n + 31) // 32 * 32
        assert pre_activations.dtype == torch.float16 and pre_activations.numel() == n32 * self.stash_halfs
        cout_padded = self.spec.layers[-1].channels_out
        adj_padded = torch.zeros((n, cout_padded), dtype=torch.float32, device=x.device)
        adj_padded[:, :adj_output.shape[1]] = adj_output
        adj_input = torch.zeros_like(x)
        deltas = torch.zeros((n32 * self.stash_halfs,), dtype=torch.float16, device=x.device)
        arr, keep = _grid_array(self.spec, tables, table_grads)
        info = (C.c_int * 3)()
        torch.cuda.synchronize()
        ms = C.c_float(0)
        err = self.lib.ref_backward(n, x.data_ptr(), adj_padded.data_ptr(), adj_input.data_ptr(), params_half.data_ptr(),
                                    pre_activations.data_ptr(), deltas.data_ptr(), arr, info, C.byref(ms))
        self.last_ms = float(ms.value)
        if err != 0:
            raise RuntimeError("reference backward kernel failed with CUDA error %d" % err)
        self.launch_info = tuple(info)
        return adj_input, deltas


class ReferenceWeightUpdate:
    """The reference's WeightUpdateSingleBlockKernel, one launch per layer in a single thread block each
    (src_cpp/include/qmlp/kernels/network_weight_update_block.cuh:356-494, launched as FusedNetwork::adjoint does,
    src_cpp/src/fused_network.cpp:1081-1144). Weight matrices only: the reference has no bias gradient."""

    def __init__(self, cfg):
        path = build_ref_kernels.build(cfg, kind="wgrad")
        if path is None:
            raise FileNotFoundError("the reference weight-update kernel for this configuration has not been built")
        self.lib = C.CDLL(path)
        self.lib.ref_weight_update.restype = C.c_int
        self.lib.ref_weight_update.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(_RefGrid),
                                               C.POINTER(C.c_int), C.POINTER(C.c_float)]
        self.last_ms = 0.0
        self.spec = oracle.parse_spec(cfg)
        assert self.lib.ref_num_parameters() == self.spec.num_parameters
        assert self.lib.ref_num_layers() == len(self.spec.layers)
        self.launch_info = None

    def __call__(self, x, pre_activations, deltas, tables):
        """x (N, Cin) fp32; pre_activations / deltas: fp16 CUDA tensors, (N32, Cout_l) row-major per layer in layer
        order. Returns the fp32 gradient vector in the flat parameter layout (bias entries zero)."""
        import torch
        n = x.shape[0]
        grads = torch.zeros((self.spec.num_parameters,), dtype=torch.float32, device=x.device)
        arr, keep = _grid_array(self.spec, tables)
        info = (C.c_int * (2 * len(self.spec.layers)))()
        torch.cuda.synchronize()
        ms = C.c_float(0)
        err = self.lib.ref_weight_update(n, x.data_ptr(), grads.data_ptr(), pre_activations.data_ptr(), deltas.data_ptr(), arr, info,
                                         C.byref(ms))
        self.last_ms = float(ms.value)
        if err != 0:
            raise RuntimeError("reference weight-update kernel failed with error %d" % err)
        self.launch_info = tuple(info)
        return grads
