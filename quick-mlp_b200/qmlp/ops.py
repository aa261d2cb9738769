"""Stand-alone activation and encoding as registered torch operators (``torch.ops.qmlp_b200.*``).

The reference registers TorchScript custom classes (``torch.classes.qmlp_cu.Activation / Encoding``,
src_cpp/pytorch-bindings/src/bind_activation.cpp:82-98, bind_encoding.cpp:167-197) so that its ``FusedActivation`` and
``FusedEncoding`` modules survive ``torch.jit.trace`` / ``freeze`` / ``save`` / ``load``
(tests_py/qmlp_tests/test_activations.py:42-57, test_encoding.py:84-106). Here the modules call operators whose only
non-tensor argument is the configuration string: a traced graph holds the string as a constant and the operator name,
and loading it needs nothing but this package imported. The operator looks the compiled object up by that string.
"""
from typing import Optional, Tuple

import torch

from . import bindings

_activations = {}
_encodings = {}


def _activation(cfg: str) -> "bindings.Activation":
    a = _activations.get(cfg)
    if a is None:
        a = _activations[cfg] = bindings.Activation(cfg)
    return a


def _encoding(cfg: str) -> "bindings.Encoding":
    e = _encodings.get(cfg)
    if e is None:
        e = _encodings[cfg] = bindings.Encoding(cfg)
    return e


# ---- activation (half tensors of any shape with a last channel dimension) ---------------------------------------------
@torch.library.custom_op("qmlp_b200::activation_forward", mutates_args=())
def activation_forward(input: torch.Tensor, cfg: str) -> torch.Tensor:
    return _activation(cfg).inference(input)


@activation_forward.register_fake
def _(input, cfg):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


@torch.library.custom_op("qmlp_b200::activation_adjoint", mutates_args=())
def activation_adjoint(input: torch.Tensor, adj_output: torch.Tensor, cfg: str) -> torch.Tensor:
    return _activation(cfg).adjoint(input, adj_output)


@activation_adjoint.register_fake
def _(input, adj_output, cfg):
    return torch.empty_like(input, memory_format=torch.contiguous_format)


def _activation_setup(ctx, inputs, output):
    input, cfg = inputs
    ctx.cfg = cfg
    ctx.save_for_backward(input)


def _activation_backward(ctx, grad_output):
    (input,) = ctx.saved_tensors
    return activation_adjoint(input, grad_output.contiguous(), ctx.cfg), None


activation_forward.register_autograd(_activation_backward, setup_context=_activation_setup)


# ---- encoding (float32 (N, C) tensors; optional float32 or float16 table) ------------------------------------------------
@torch.library.custom_op("qmlp_b200::encoding_forward", mutates_args=())
def encoding_forward(input: torch.Tensor, parameters: Optional[torch.Tensor], cfg: str) -> torch.Tensor:
    enc = _encoding(cfg)
    if parameters is None:
        return enc.inference(input)
    return enc.inference_with_parameter(input, parameters)


@encoding_forward.register_fake
def _(input, parameters, cfg):
    return input.new_empty((input.shape[0], _encoding(cfg).num_output_channels()))


@torch.library.custom_op("qmlp_b200::encoding_adjoint", mutates_args=())
def encoding_adjoint(input: torch.Tensor, parameters: Optional[torch.Tensor], adj_output: torch.Tensor, want_input: bool,
                     want_parameters: bool, cfg: str) -> Tuple[torch.Tensor, torch.Tensor]:
    adj_input, adj_param = _encoding(cfg).adjoint_with_parameter(input, parameters, adj_output, want_input, want_parameters)
    if adj_input is None:
        adj_input = input.new_zeros((0,))
    if adj_param is None:
        adj_param = input.new_zeros((0,))
    return adj_input, adj_param


@encoding_adjoint.register_fake
def _(input, parameters, adj_output, want_input, want_parameters, cfg):
    adj_input = torch.empty_like(input) if want_input else input.new_empty((0,))
    adj_param = (torch.empty_like(parameters, dtype=torch.float32) if (want_parameters and parameters is not None)
                 else input.new_empty((0,)))
    return adj_input, adj_param


def _encoding_setup(ctx, inputs, output):
    input, parameters, cfg = inputs
    ctx.cfg = cfg
    ctx.has_parameters = parameters is not None
    ctx.param_dtype = parameters.dtype if parameters is not None else None
    if parameters is not None:
        ctx.save_for_backward(input, parameters)
    else:
        ctx.save_for_backward(input)


def _encoding_backward(ctx, grad_output):
    saved = ctx.saved_tensors
    input = saved[0]
    parameters = saved[1] if ctx.has_parameters else None
    want_input = ctx.needs_input_grad[0]
    want_param = ctx.has_parameters and ctx.needs_input_grad[1]
    adj_input, adj_param = encoding_adjoint(input, parameters, grad_output.contiguous(), want_input, want_param, ctx.cfg)
    return (adj_input if want_input else None,
            adj_param.to(ctx.param_dtype) if want_param else None,
            None)


encoding_forward.register_autograd(_encoding_backward, setup_context=_encoding_setup)
