"""ctypes binding of libqmlp_b200.so (declared in include/qmlp_b200.h).

This is the layer the reference fills with its TorchScript custom classes
(src_cpp/pytorch-bindings/src/bindings.cpp:102-122); PyTorch is only used for device memory and streams.
The library must be present: there is no fallback path.
"""
import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "..", "lib", "libqmlp_b200.so")

QMLP_FLOAT, QMLP_HALF, QMLP_DOUBLE = 0, 1, 2
QMLP_INFERENCE, QMLP_GRADIENTS = 0, 1
GRADIENTS_INPUT, GRADIENTS_NETWORK_WEIGHTS, GRADIENTS_INPUT_ENCODINGS = 1, 2, 4
ENCODING_INPUT_GRADIENTS, ENCODING_PARAM_GRADIENTS = 1, 2


class Tensor(C.Structure):
    """qmlp_tensor_t"""
    _fields_ = [("data", C.c_void_p), ("precision", C.c_int32), ("ndim", C.c_int32),
                ("sizes", C.c_int64 * 2), ("strides", C.c_int64 * 2)]


class TrainerConfig(C.Structure):
    """qmlp_trainer_config_t"""
    _fields_ = [("learning_rate", C.c_float), ("beta1", C.c_float), ("beta2", C.c_float), ("epsilon", C.c_float),
                ("grid_half_copy", C.c_int32), ("reserved", C.c_int32)]


class QmlpError(RuntimeError):
    pass


class ConfigurationError(QmlpError):
    pass


_lib = None

# name -> (restype, argtypes); every symbol include/qmlp_b200.h declares
_P = C.c_void_p
_TP = C.POINTER(Tensor)
SIGNATURES = {
    "qmlp_last_error": (C.c_char_p, []),
    "qmlp_is_cuda_available": (C.c_int, []),
    "qmlp_set_log_level": (C.c_int, [C.c_char_p]),
    "qmlp_set_compile_debug_mode": (C.c_int, [C.c_int]),
    "qmlp_is_compile_debug_mode": (C.c_int, []),
    "qmlp_set_kernel_cache_dir": (C.c_int, [C.c_char_p]),
    "qmlp_get_kernel_cache_dir": (C.c_char_p, []),
    "qmlp_set_kernel_include_dir": (C.c_int, [C.c_char_p]),
    "qmlp_set_kernel_path": (C.c_int, [C.c_int]),
    "qmlp_device_status": (C.c_int, [C.POINTER(C.c_int)]),
    "qmlp_set_tuning": (C.c_int, [C.c_char_p, C.c_int]),
    "qmlp_set_kernel_timing": (C.c_int, [C.c_int]),
    "qmlp_read_kernel_timing": (C.c_int, [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "qmlp_network_create": (C.c_int, [C.c_char_p, C.c_char_p, C.POINTER(_P)]),
    "qmlp_network_destroy": (None, [_P]),
    "qmlp_network_channels_in": (C.c_int, [_P]),
    "qmlp_network_channels_out": (C.c_int, [_P]),
    "qmlp_network_num_layers": (C.c_int, [_P]),
    "qmlp_network_num_encodings": (C.c_int, [_P]),
    "qmlp_network_parameter_count": (C.c_int64, [_P]),
    "qmlp_network_parameter_precision": (C.c_int, [_P, C.c_int]),
    "qmlp_network_layer_info": (C.c_int, [_P, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                          C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "qmlp_network_encoding": (C.c_int, [_P, C.c_int, C.POINTER(_P)]),
    "qmlp_network_set_parameter": (C.c_int, [_P, _TP, C.c_int]),
    "qmlp_network_initialize_parameters": (C.c_int, [_P, C.c_uint64]),
    "qmlp_network_initialize_parameters_host": (C.c_int, [_P, C.c_uint64, _P]),
    "qmlp_network_inference": (C.c_int, [_P, _TP, _TP, _P]),
    "qmlp_network_inference_host": (C.c_int, [_P, _P, _P, C.c_int64, C.c_int64, _P]),
    "qmlp_network_forward_memory": (C.c_int, [_P, C.c_int64, C.c_int, C.POINTER(C.c_size_t)]),
    "qmlp_network_forward": (C.c_int, [_P, _TP, _TP, _P, _P]),
    "qmlp_network_forward_static_scratch": (C.c_int, [_P, _TP, _TP, _P]),
    "qmlp_static_scratch": (C.c_int, [C.POINTER(_P), C.POINTER(C.c_size_t)]),
    "qmlp_network_zero_gradients": (C.c_int, [_P, _P]),
    "qmlp_network_adjoint_memory": (C.c_int, [_P, C.c_int64, C.c_int, C.POINTER(C.c_size_t)]),
    "qmlp_network_adjoint": (C.c_int, [_P, _TP, _TP, C.c_int, _TP, _P, _P, _P]),
    "qmlp_network_clear_cached_kernels": (C.c_int, [_P]),
    "qmlp_network_compile": (C.c_int, [_P, C.c_int]),
    "qmlp_network_launch_count": (C.c_int64, [_P]),
    "qmlp_encoding_create": (C.c_int, [C.c_char_p, C.POINTER(_P)]),
    "qmlp_encoding_destroy": (None, [_P]),
    "qmlp_encoding_to_json": (C.c_char_p, [_P]),
    "qmlp_encoding_id": (C.c_char_p, [_P]),
    "qmlp_encoding_max_input_channel": (C.c_int, [_P]),
    "qmlp_encoding_num_output_channels": (C.c_int, [_P]),
    "qmlp_encoding_has_parameters": (C.c_int, [_P]),
    "qmlp_encoding_parameter_count": (C.c_int64, [_P]),
    "qmlp_encoding_parameter_precision": (C.c_int, [_P, C.c_int]),
    "qmlp_encoding_grid_levels": (C.c_int, [_P, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int32),
                                            C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    "qmlp_encoding_set_parameter": (C.c_int, [_P, _TP, C.c_int]),
    "qmlp_encoding_zero_gradients": (C.c_int, [_P, _P]),
    "qmlp_encoding_forward": (C.c_int, [_P, _TP, _TP, _P, _TP]),
    "qmlp_encoding_adjoint": (C.c_int, [_P, _TP, _TP, _TP, _P, _TP, _TP, C.c_int]),
    "qmlp_encoding_compile": (C.c_int, [_P, C.c_int]),
    "qmlp_activation_compile": (C.c_int, [_P]),
    "qmlp_activation_create": (C.c_int, [C.c_char_p, C.POINTER(_P)]),
    "qmlp_activation_destroy": (None, [_P]),
    "qmlp_activation_id": (C.c_char_p, [_P]),
    "qmlp_activation_to_json": (C.c_char_p, [_P]),
    "qmlp_activation_forward": (C.c_int, [_P, _TP, _TP, _P]),
    "qmlp_activation_adjoint": (C.c_int, [_P, _TP, _TP, _TP, _P]),
    "qmlp_trainer_create": (C.c_int, [_P, C.POINTER(TrainerConfig), C.POINTER(_P)]),
    "qmlp_trainer_destroy": (None, [_P]),
    "qmlp_trainer_fused_count": (C.c_int64, [_P]),
    "qmlp_trainer_segment_start": (C.c_int64, [_P, C.c_int]),
    "qmlp_trainer_workspace_bytes": (C.c_int, [_P, C.c_int64, C.POINTER(C.c_size_t)]),
    "qmlp_trainer_bind": (C.c_int, [_P, _P, _P, _P, _P, _P]),
    "qmlp_trainer_refresh_half": (C.c_int, [_P, _P]),
    "qmlp_trainer_gradients": (C.c_int, [_P, _TP, _TP, C.c_int64, _P, C.c_size_t, _P, _P]),
    "qmlp_trainer_gradients_part": (C.c_int, [_P, _TP, _TP, C.c_int64, _P, C.c_size_t, _P, C.c_int, _P]),
    "qmlp_trainer_scatter_levels": (C.c_int, [_P, C.c_int, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
    "qmlp_trainer_update": (C.c_int, [_P, C.c_int64, C.c_float, _P]),
}


def lib():
    """Loads the shared library once; raises if it has not been built (python quick-mlp_b200/build.py)."""
    global _lib
    if _lib is None:
        path = os.path.abspath(os.environ.get("QMLP_B200_LIBRARY", LIB_PATH))
        if not os.path.exists(path):
            raise ImportError(f"{path} not found: build it with `python quick-mlp_b200/build.py`. "
                              "There is no CPU or PyTorch fallback for the fused kernels.")
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int):
    if status != 0:
        msg = lib().qmlp_last_error().decode("utf-8", "replace")
        if status == 2:
            raise ConfigurationError(msg)
        raise QmlpError(msg)


_PRECISION = {torch.float32: QMLP_FLOAT, torch.float16: QMLP_HALF, torch.float64: QMLP_DOUBLE}


def wrap(t, require_cuda=True) -> Tensor:
    """torch.Tensor -> qmlp_tensor_t (non-owning). None -> undefined tensor.
    Same role as qmlp::wrap in the reference bindings (src_cpp/pytorch-bindings/src/bindings.cpp:25-60)."""
    out = Tensor()
    if t is None:
        return out
    if require_cuda and not t.is_cuda:
        raise QmlpError("tensor must live on a CUDA device")
    if t.dtype not in _PRECISION:
        raise QmlpError(f"unsupported dtype {t.dtype}")
    if t.dim() < 1 or t.dim() > 2:
        raise QmlpError("only 1-D and 2-D tensors are supported")
    out.data = t.data_ptr()
    out.precision = _PRECISION[t.dtype]
    out.ndim = t.dim()
    for i in range(t.dim()):
        out.sizes[i] = t.shape[i]
        out.strides[i] = t.stride(i)
    return out


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream
