"""qmlp.FusedActivation, API of src_py/qmlp/activation.py:8-79."""
import torch

from . import ops  # noqa: F401  (registers torch.ops.qmlp_b200.*)
from .bindings import Activation


class FusedActivation(torch.nn.Module):
    """Fused activation in a custom CUDA kernel (half precision only)."""

    @staticmethod
    def get_activation(name: str) -> torch.nn.Module:
        """PyTorch module equal to a built-in activation (src_py/qmlp/activation.py:13-37)."""
        if name == "relu":
            return torch.nn.ReLU()
        if name == "celu":
            return torch.nn.CELU()
        if name == "sine":
            class Sine(torch.nn.Module):
                def forward(self, x):
                    return torch.sin(x)
            return Sine()
        if name == "identity":
            return torch.nn.Identity()
        raise ValueError("Unknown or user-specified activation")

    def __init__(self, cfg: str):
        """``cfg`` is a built-in id (relu, celu, sine, identity) or an inline JSON object
        {"id": ..., "forward": "z = ...", "adjoint": "adjx = ..."} with CUDA statements over half."""
        super().__init__()
        self._cfg = cfg
        self._activation = Activation(cfg)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        # a registered operator keyed by the configuration string: traceable, freezable, saveable (qmlp/ops.py)
        return torch.ops.qmlp_b200.activation_forward(input, self._cfg)

    def __repr__(self):
        return f"FusedActivation(\"{self._cfg}\")"

    __str__ = __repr__
