"""Python objects with the method set of the reference's ``torch.classes.qmlp_cu`` custom classes
(QuickMLP, Network, Encoding, Activation: src_cpp/pytorch-bindings/src/bindings.cpp:102-122,
bind_network.cpp:348-411, bind_encoding.cpp:167-197, bind_activation.cpp:82-98), implemented over the C ABI.
Autograd support mirrors NetworkBindings::forward (bind_network.cpp:120-321),
EncodingBindings (bind_encoding.cpp:134-163) and ActivationBindings (bind_activation.cpp:52-79).
"""
import ctypes as C
import json
import threading
from typing import List, Optional, Sequence

import torch

from . import _capi
from ._capi import check, current_stream, lib, wrap


class QuickMLP:
    """qmlp::QuickMLP singleton (src_cpp/include/qmlp/qmlp.h:14-94) as static methods."""

    @staticmethod
    def is_cuda_available() -> bool:
        return bool(lib().qmlp_is_cuda_available())

    @staticmethod
    def set_log_level(level: str):
        check(lib().qmlp_set_log_level(level.encode()))

    @staticmethod
    def set_compile_debug_mode(enabled: bool):
        check(lib().qmlp_set_compile_debug_mode(int(bool(enabled))))

    @staticmethod
    def is_compile_debug_mode() -> bool:
        return bool(lib().qmlp_is_compile_debug_mode())

    @staticmethod
    def set_kernel_cache_dir(path: str):
        check(lib().qmlp_set_kernel_cache_dir(path.encode()))

    @staticmethod
    def kernel_cache_dir() -> str:
        return lib().qmlp_get_kernel_cache_dir().decode()

    @staticmethod
    def set_kernel_path(path: int):
        """0: best kernels instantiated for a spec (tcgen05 inference when the widths allow), 1: mma.sync only."""
        check(lib().qmlp_set_kernel_path(int(path)))

    @staticmethod
    def set_tuning(key: str, value: int):
        """Tuning switches of the fused training step ("sort_points", "split_scatter", "scatter_runs"; -1 = automatic) and
        of the kernel instantiation ("bounds_check": 1 = kernels that test every table row, stash and plane offset and
        report through device_status() instead of faulting; "bounds_shrink": test hook, declares all sizes that many
        elements smaller)."""
        check(lib().qmlp_set_tuning(key.encode(), int(value)))

    @staticmethod
    def device_status() -> int:
        """Synchronises and returns (then clears) the device status word: non-zero means a kernel gave up on a
        bounded wait and its outputs are invalid."""
        s = C.c_int(0)
        check(lib().qmlp_device_status(C.byref(s)))
        return s.value


# ---------------------------------------------------------------------------------------------------------------------
class Activation:
    def __init__(self, cfg: str):
        self._cfg = cfg
        h = C.c_void_p()
        check(lib().qmlp_activation_create(cfg.encode(), C.byref(h)))
        self._h = h

    def __del__(self):
        try:
            if getattr(self, "_h", None) and _capi._lib is not None:
                _capi._lib.qmlp_activation_destroy(self._h)
                self._h = None
        except Exception:   # interpreter shutdown: module globals may already be gone
            pass

    def cfg(self) -> str:
        return self._cfg

    def id(self) -> str:
        return lib().qmlp_activation_id(self._h).decode()

    def to_json(self) -> str:
        return lib().qmlp_activation_to_json(self._h).decode()

    def compile(self):
        check(lib().qmlp_activation_compile(self._h))

    def inference(self, input: torch.Tensor) -> torch.Tensor:
        output = torch.empty_like(input, memory_format=torch.contiguous_format)
        check(lib().qmlp_activation_forward(self._h, wrap(input), wrap(output), current_stream()))
        return output

    def adjoint(self, input: torch.Tensor, adj_output: torch.Tensor) -> torch.Tensor:
        adj_input = torch.empty_like(input, memory_format=torch.contiguous_format)
        check(lib().qmlp_activation_adjoint(self._h, wrap(input), wrap(adj_output), wrap(adj_input), current_stream()))
        return adj_input

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return _ActivationFunction.apply(input, self)

    def __getstate__(self):   # pickle = cfg string, bind_activation.cpp:91-97
        return self._cfg

    def __setstate__(self, cfg):
        self.__init__(cfg)


class _ActivationFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, act):
        ctx.act = act
        ctx.save_for_backward(input)
        return act.inference(input)

    @staticmethod
    def backward(ctx, grad_output):
        (input,) = ctx.saved_tensors
        return ctx.act.adjoint(input, grad_output.contiguous()), None


# ---------------------------------------------------------------------------------------------------------------------
class Encoding:
    def __init__(self, cfg: Optional[str] = None, _handle=None, _owner=None):
        self._owner = _owner   # keeps the owning network alive for borrowed handles
        if _handle is not None:
            self._h, self._owned = _handle, False
        else:
            h = C.c_void_p()
            check(lib().qmlp_encoding_create(cfg.encode(), C.byref(h)))
            self._h, self._owned = h, True
        self._cfg = self.to_json()

    def __del__(self):
        try:
            if getattr(self, "_owned", False) and getattr(self, "_h", None) and _capi._lib is not None:
                _capi._lib.qmlp_encoding_destroy(self._h)
                self._h = None
        except Exception:   # interpreter shutdown: module globals may already be gone
            pass

    def cfg(self) -> str:
        return self._cfg

    def to_json(self) -> str:
        return lib().qmlp_encoding_to_json(self._h).decode()

    def id(self) -> str:
        return lib().qmlp_encoding_id(self._h).decode()

    def max_input_channel(self) -> int:
        return lib().qmlp_encoding_max_input_channel(self._h)

    def num_output_channels(self) -> int:
        return lib().qmlp_encoding_num_output_channels(self._h)

    def has_parameters(self) -> bool:
        return bool(lib().qmlp_encoding_has_parameters(self._h))

    def parameter_count(self) -> int:
        return lib().qmlp_encoding_parameter_count(self._h)

    def grid_levels(self):
        """[(memory_offset, resolution, hash_grid_size, hashed)] of a grid encoding; [] otherwise."""
        n = lib().qmlp_encoding_grid_levels(self._h, 0, None, None, None, None)
        if n <= 0:
            return []
        off = (C.c_int64 * n)(); res = (C.c_int32 * n)(); hs = (C.c_int32 * n)(); hd = (C.c_int32 * n)()
        lib().qmlp_encoding_grid_levels(self._h, n, off, res, hs, hd)
        return [(off[i], res[i], hs[i], bool(hd[i])) for i in range(n)]

    def create_inference_parameters(self, device="cuda") -> torch.Tensor:
        # bind_encoding.cpp:40-48: uninitialised fp32 vector
        assert self.has_parameters()
        return torch.empty((self.parameter_count(),), dtype=torch.float32, device=device)

    def create_gradient_parameters(self, device="cuda") -> torch.Tensor:
        assert self.has_parameters()
        return torch.zeros((self.parameter_count(),), dtype=torch.float32, device=device)

    def set_parameter(self, tensor: Optional[torch.Tensor], usage: int):
        check(lib().qmlp_encoding_set_parameter(self._h, wrap(tensor), usage))

    def compile(self, half_table: bool = False):
        check(lib().qmlp_encoding_compile(self._h, int(half_table)))

    def _out(self, input):
        return torch.empty((input.shape[0], self.num_output_channels()), dtype=torch.float32, device=input.device)

    def inference(self, input: torch.Tensor) -> torch.Tensor:
        output = self._out(input)
        check(lib().qmlp_encoding_forward(self._h, wrap(input), wrap(output), current_stream(), None))
        return output

    def inference_with_parameter(self, input: torch.Tensor, parameters: torch.Tensor) -> torch.Tensor:
        output = self._out(input)
        p = wrap(parameters)
        check(lib().qmlp_encoding_forward(self._h, wrap(input), wrap(output), current_stream(), C.byref(p)))
        return output

    def adjoint_with_parameter(self, input, parameters, adj_output, want_input=True, want_param=True):
        adj_input = torch.zeros_like(input) if want_input else None
        adj_param = torch.zeros_like(parameters, dtype=torch.float32) if (want_param and parameters is not None) else None
        mode = (1 if want_input else 0) | (2 if adj_param is not None else 0)
        p = wrap(parameters) if parameters is not None else None
        g = wrap(adj_param) if adj_param is not None else None
        check(lib().qmlp_encoding_adjoint(self._h, wrap(input), wrap(adj_output.contiguous()), wrap(adj_input), current_stream(),
                                          C.byref(p) if p is not None else None, C.byref(g) if g is not None else None, mode))
        return adj_input, adj_param

    def adjoint(self, input, adj_output):
        return self.adjoint_with_parameter(input, None, adj_output, True, False)[0]

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return _EncodingFunction.apply(input, None, self)

    def forward_with_parameter(self, input: torch.Tensor, parameters: torch.Tensor) -> torch.Tensor:
        return _EncodingFunction.apply(input, parameters, self)

    def __getstate__(self):   # pickle = cfg string, bind_encoding.cpp:190-196
        return self._cfg

    def __setstate__(self, cfg):
        self.__init__(cfg)


class _EncodingFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, parameters, enc):
        ctx.enc = enc
        ctx.has_param = parameters is not None
        ctx.save_for_backward(input, parameters) if parameters is not None else ctx.save_for_backward(input)
        if parameters is not None:
            return enc.inference_with_parameter(input, parameters)
        return enc.inference(input)

    @staticmethod
    def backward(ctx, grad_output):
        saved = ctx.saved_tensors
        input = saved[0]
        parameters = saved[1] if ctx.has_param else None
        gi, gp = ctx.enc.adjoint_with_parameter(input, parameters, grad_output, ctx.needs_input_grad[0],
                                                ctx.has_param and ctx.needs_input_grad[1])
        return gi, gp, None


# ---------------------------------------------------------------------------------------------------------------------
class Network:
    """torch.classes.qmlp_cu.Network(cfg: str, parent: str = '.'), bind_network.cpp:348-411."""

    def __init__(self, cfg: str, parent: str = "."):
        self._cfg, self._parent = cfg, parent
        h = C.c_void_p()
        check(lib().qmlp_network_create(cfg.encode(), parent.encode(), C.byref(h)))
        self._h = h
        self._mutex = threading.Lock()   # parameter pointers are instance state, bind_network.h:20

    def __del__(self):
        try:
            if getattr(self, "_h", None) and _capi._lib is not None:
                _capi._lib.qmlp_network_destroy(self._h)
                self._h = None
        except Exception:   # interpreter shutdown: module globals may already be gone
            pass

    def cfg(self) -> str:
        return self._cfg

    def parent(self) -> str:
        return self._parent

    @staticmethod
    def MatrixSize() -> int:
        return 16

    @staticmethod
    def WarpSize() -> int:
        return 32

    @staticmethod
    def MaxSharedMemoryBytes() -> int:
        return 227 * 1024

    def is_parallel_streams(self) -> bool:
        return False   # weight gradients of all layers run in one kernel here

    def set_parallel_streams(self, v: bool):
        pass

    def num_encodings(self) -> int:
        return lib().qmlp_network_num_encodings(self._h)

    def encoding(self, idx: int) -> Encoding:
        h = C.c_void_p()
        check(lib().qmlp_network_encoding(self._h, idx, C.byref(h)))
        return Encoding(_handle=h, _owner=self)

    def channels_in(self) -> int:
        return lib().qmlp_network_channels_in(self._h)

    def channels_out(self) -> int:
        return lib().qmlp_network_channels_out(self._h)

    def num_layers(self) -> int:
        return lib().qmlp_network_num_layers(self._h)

    def num_network_parameters(self) -> int:
        return lib().qmlp_network_parameter_count(self._h)

    def layer_info(self, layer: int):
        cin, cout, bias = C.c_int(), C.c_int(), C.c_int()
        ws, bs = C.c_int64(), C.c_int64()
        check(lib().qmlp_network_layer_info(self._h, layer, C.byref(cin), C.byref(cout), C.byref(bias), C.byref(ws), C.byref(bs)))
        return cin.value, cout.value, bool(bias.value), ws.value, bs.value

    def create_inference_parameters(self, device="cuda") -> torch.Tensor:
        return torch.zeros((self.num_network_parameters(),), dtype=torch.float16, device=device)

    def initialize_inference_parameters(self, dst: torch.Tensor, seed: Optional[int] = None):
        # bind_network.cpp:63-74: seed drawn from torch's CPU generator
        if seed is None:
            seed = int(torch.randint(2 ** 62, (1,)).item())
        assert dst.dtype == torch.float16 and dst.dim() == 1 and dst.shape[0] == self.num_network_parameters()
        host = torch.empty((self.num_network_parameters(),), dtype=torch.float16)
        check(lib().qmlp_network_initialize_parameters_host(self._h, seed, host.data_ptr()))
        dst.copy_(host)

    def parameter_view(self, layer: int, bias: bool, parameters: torch.Tensor) -> torch.Tensor:
        # NetworkBindings::view, bind_network.cpp:323-345 (shares memory with `parameters`)
        assert parameters.dtype in (torch.float32, torch.float16)
        assert parameters.dim() == 1 and parameters.shape[0] == self.num_network_parameters()
        cin, cout, has_bias, ws, bs = self.layer_info(layer)
        if bias:
            if not has_bias:
                return torch.empty((0,), dtype=parameters.dtype, device=parameters.device)
            return parameters[bs:bs + cout]
        return parameters[ws:ws + cin * cout].view(cout, cin)

    # -- launches ----------------------------------------------------------------------------------------------------
    def _bind(self, network_parameters, encoding_parameters: Sequence[Optional[torch.Tensor]]):
        if network_parameters is not None:
            check(lib().qmlp_network_set_parameter(self._h, wrap(network_parameters), _capi.QMLP_INFERENCE))
        for i in range(min(len(encoding_parameters), self.num_encodings())):
            p = encoding_parameters[i]
            if p is not None:
                self.encoding(i).set_parameter(p, _capi.QMLP_INFERENCE)

    @staticmethod
    def _half(p: torch.Tensor) -> torch.Tensor:
        return p if p.dtype == torch.float16 else p.to(torch.float16)

    def inference(self, input: torch.Tensor, network_parameters: torch.Tensor,
                  encoding_parameters: Sequence[Optional[torch.Tensor]] = ()) -> torch.Tensor:
        with self._mutex:
            output = torch.empty((input.shape[0], self.channels_out()), dtype=torch.float32, device=input.device)
            np_half = self._half(network_parameters)
            self._bind(np_half, encoding_parameters)
            check(lib().qmlp_network_inference(self._h, wrap(input), wrap(output), current_stream()))
            return output

    def inference_host(self, input: torch.Tensor, network_parameters: torch.Tensor,
                       encoding_parameters: Sequence[Optional[torch.Tensor]] = (),
                       output: Optional[torch.Tensor] = None, chunk_points: int = 0) -> torch.Tensor:
        """Inference of a batch that lives in host memory: `input` is a contiguous fp32 CPU tensor (page-locked for the
        copies to overlap), the result is a CPU tensor (`output` if given, else a new page-locked one). Parameters are
        device tensors as in `inference`. Uploads, kernels and downloads of successive chunks overlap
        (qmlp_network_inference_host); the result is complete once the current CUDA stream is."""
        assert input.device.type == "cpu" and input.dtype == torch.float32 and input.is_contiguous()
        with self._mutex:
            n = input.shape[0]
            if output is None:
                output = torch.empty((n, self.channels_out()), dtype=torch.float32, pin_memory=True)
            assert output.device.type == "cpu" and output.dtype == torch.float32 and output.is_contiguous()
            assert tuple(output.shape) == (n, self.channels_out()) and input.shape[1] == self.channels_in()
            self._bind(self._half(network_parameters), encoding_parameters)
            check(lib().qmlp_network_inference_host(self._h, input.data_ptr(), output.data_ptr(), n, int(chunk_points),
                                                    current_stream()))
            return output

    def forward(self, input: torch.Tensor, network_parameters: torch.Tensor,
                encoding_parameters: Sequence[Optional[torch.Tensor]] = ()) -> torch.Tensor:
        flags = 0
        if input.requires_grad:
            flags |= _capi.GRADIENTS_INPUT
        if network_parameters is not None and network_parameters.requires_grad:
            flags |= _capi.GRADIENTS_NETWORK_WEIGHTS
        if any(p is not None and p.requires_grad for p in encoding_parameters):
            flags |= _capi.GRADIENTS_INPUT_ENCODINGS
        if flags == 0 or not torch.is_grad_enabled():
            return self.inference(input, network_parameters, encoding_parameters)
        return _NetworkFunction.apply(self, flags, input, network_parameters, *encoding_parameters)

    def forward_memory(self, n: int, flags: int = 7) -> int:
        b = C.c_size_t()
        check(lib().qmlp_network_forward_memory(self._h, n, flags, C.byref(b)))
        return b.value

    def adjoint_memory(self, n: int, flags: int = 7) -> int:
        b = C.c_size_t()
        check(lib().qmlp_network_adjoint_memory(self._h, n, flags, C.byref(b)))
        return b.value

    def compile(self, grid_half_mask: int = 0):
        check(lib().qmlp_network_compile(self._h, grid_half_mask))

    def launch_count(self) -> int:
        return lib().qmlp_network_launch_count(self._h)

    def __getstate__(self):   # pickle = [cfg, parent], bind_network.cpp:403-410
        return (self._cfg, self._parent)

    def __setstate__(self, state):
        self.__init__(*state)


class _NetworkFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, net: Network, flags: int, input, network_parameters, *encoding_parameters):
        np_half = Network._half(network_parameters.detach())
        tmp = torch.empty((max(net.forward_memory(input.shape[0], flags), 16),), dtype=torch.uint8, device=input.device)
        output = torch.empty((input.shape[0], net.channels_out()), dtype=torch.float32, device=input.device)
        with net._mutex:
            net._bind(np_half, [p.detach() if p is not None else None for p in encoding_parameters])
            check(lib().qmlp_network_forward(net._h, wrap(input.detach()), wrap(output), tmp.data_ptr(), current_stream()))
        ctx.net, ctx.flags = net, flags
        ctx.param_dtype = network_parameters.dtype
        ctx.num_enc = len(encoding_parameters)
        ctx.enc_defined = [p is not None for p in encoding_parameters]
        ctx.save_for_backward(input, np_half, tmp, *[p for p in encoding_parameters if p is not None])
        return output

    @staticmethod
    def backward(ctx, grad_output):
        net, flags = ctx.net, ctx.flags
        saved = ctx.saved_tensors
        input, np_half, tmp = saved[0], saved[1], saved[2]
        enc_saved = list(saved[3:])
        enc_params: List[Optional[torch.Tensor]] = [enc_saved.pop(0) if d else None for d in ctx.enc_defined]
        grad_output = grad_output.contiguous()
        adj_input = torch.zeros_like(input) if flags & _capi.GRADIENTS_INPUT else None
        adj_params = None
        adj_enc: List[Optional[torch.Tensor]] = [None] * ctx.num_enc
        with net._mutex:
            net._bind(np_half, enc_params)
            if flags & _capi.GRADIENTS_NETWORK_WEIGHTS:
                adj_params = torch.zeros(np_half.shape, dtype=torch.float32, device=np_half.device)
                check(lib().qmlp_network_set_parameter(net._h, wrap(adj_params), _capi.QMLP_GRADIENTS))
            if flags & _capi.GRADIENTS_INPUT_ENCODINGS:
                for i, p in enumerate(enc_params):
                    if p is not None and p.requires_grad:
                        adj_enc[i] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                        net.encoding(i).set_parameter(adj_enc[i], _capi.QMLP_GRADIENTS)
                    elif i < net.num_encodings():
                        net.encoding(i).set_parameter(None, _capi.QMLP_GRADIENTS)
            adj_tmp = torch.empty((max(net.adjoint_memory(input.shape[0], flags), 16),), dtype=torch.uint8, device=input.device)
            ai = wrap(adj_input)
            check(lib().qmlp_network_adjoint(net._h, wrap(input), wrap(grad_output), flags, C.byref(ai), tmp.data_ptr(),
                                             adj_tmp.data_ptr(), current_stream()))
        if adj_params is not None:
            adj_params = adj_params.to(ctx.param_dtype)
        return (None, None, adj_input, adj_params, *adj_enc)
