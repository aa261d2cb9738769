"""qmlp.FusedEncoding, API of src_py/qmlp/encoding.py:9-122."""
import torch

from . import ops  # noqa: F401  (registers torch.ops.qmlp_b200.*)
from .bindings import Encoding


class FusedEncoding(torch.nn.Module):
    """Stand-alone encoding (Identity or HashGrid) with autograd support. Inputs and outputs are float32."""

    def __init__(self, cfg_or_impl):
        super().__init__()
        if isinstance(cfg_or_impl, str):
            self._encoding = Encoding(cfg_or_impl)
        elif isinstance(cfg_or_impl, Encoding):
            self._encoding = cfg_or_impl
        else:
            raise TypeError("expected a json string or an Encoding")
        self._cfg = self._encoding.to_json()
        self._max_input_channel = self._encoding.max_input_channel()
        self._num_output_channels = self._encoding.num_output_channels()
        self._has_parameters = self._encoding.has_parameters()

    def max_input_channel(self) -> int:
        return self._max_input_channel

    def num_output_channels(self) -> int:
        return self._num_output_channels

    def has_parameters(self) -> bool:
        return self._has_parameters

    def create_parameter_tensor(self) -> torch.Tensor:
        assert self.has_parameters()
        t = self._encoding.create_inference_parameters()
        torch.nn.init.normal_(t)
        return t

    def forward(self, input: torch.Tensor, parameters: torch.Tensor = None) -> torch.Tensor:
        # a registered operator keyed by the configuration string: traceable, freezable, saveable (qmlp/ops.py)
        return torch.ops.qmlp_b200.encoding_forward(input, parameters, self._cfg)

    def __repr__(self):
        return f'FusedEncoding("""{self._cfg}""")'

    __str__ = __repr__
