"""qmlp.FusedNetwork / SimulatedNetwork / copy_torch_to_fused, API of src_py/qmlp/network.py:12-258."""
import json
import warnings

import torch

from .activation import FusedActivation
from .bindings import Network
from .encoding import FusedEncoding


class FusedNetwork(torch.nn.Module):
    """A fully fused coordinate-MLP: input encodings, linear layers and activations in one kernel."""

    def __init__(self, cfg: str, parent: str = ".", weight_dtype=torch.float16, device="cuda", verbose=False):
        super().__init__()
        self._cfg, self._parent = cfg, parent
        self._network = Network(cfg, parent)
        self._num_output_channels = self._network.channels_out()
        self._num_layers = self._network.num_layers()

        weights = self._network.create_inference_parameters(device)
        self._network.initialize_inference_parameters(weights)
        self.weights = torch.nn.Parameter(weights.to(weight_dtype), requires_grad=True)

        # Encoding parameters are real parameters here and are passed to every forward call, so a stock
        # optimiser can train a hash grid (the reference creates them but passes an empty list,
        # src_py/qmlp/network.py:44-62,152).
        self._num_encodings = self._network.num_encodings()
        assert self._num_encodings > 0
        self._encodings = [self._network.encoding(i) for i in range(self._num_encodings)]
        params = []
        for e in self._encodings:
            if e.has_parameters():
                params.append(torch.nn.Parameter(torch.zeros((e.parameter_count(),), dtype=torch.float32, device=device)))
            else:
                params.append(torch.nn.Parameter(torch.zeros((1,), device=device), requires_grad=False))
        self.encoding_parameters = torch.nn.ParameterList(params)
        if verbose:
            print("Number of trainable network parameters:", weights.shape)

    @staticmethod
    def MatrixSize() -> int:
        return Network.MatrixSize()

    @staticmethod
    def WarpSize() -> int:
        return Network.WarpSize()

    @staticmethod
    def MaxSharedMemoryBytes() -> int:
        return Network.MaxSharedMemoryBytes()

    def is_parallel_streams(self) -> bool:
        return self._network.is_parallel_streams()

    def set_parallel_streams(self, v: bool):
        self._network.set_parallel_streams(v)

    def num_encodings(self) -> int:
        return self._network.num_encodings()

    def encoding(self, index: int) -> FusedEncoding:
        return FusedEncoding(self._encodings[index])

    def channels_in(self) -> int:
        return self._network.channels_in()

    def channels_out(self) -> int:
        return self._network.channels_out()

    def num_layers(self) -> int:
        return self._num_layers

    def num_output_channels(self) -> int:
        return self._num_output_channels

    def get_weight(self, layer: int, bias: bool, grad: bool) -> torch.Tensor:
        p = self.weights.grad if grad else self.weights.data
        return torch.clone(self._network.parameter_view(layer, bias, p).detach())

    def set_weight(self, layer: int, bias: bool, grad: bool, value: torch.Tensor):
        p = self.weights.grad if grad else self.weights.data
        t = self._network.parameter_view(layer, bias, p)
        assert value.shape == t.shape
        assert value.dtype == t.dtype
        t.copy_(value)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        assert len(x.shape) == 2
        assert x.shape[1] == self.channels_in()
        if self.weights.requires_grad and self.weights.dtype == torch.float16 and torch.is_grad_enabled():
            warnings.warn("Attempt to train network with 16-bit weights: the gradient tensor will also have 16-bit "
                          "precision. Consider weight_dtype=torch.float32.")
        enc = [p if e.has_parameters() else None for p, e in zip(self.encoding_parameters, self._encodings)]
        return self._network.forward(x, self.weights, enc)

    def __repr__(self):
        return f"FusedNetwork(\"{self._cfg}\")"

    __str__ = __repr__


class SimulatedNetwork(torch.nn.Module):
    """The same network in stock PyTorch layers, for identity encodings only (src_py/qmlp/network.py:161-243).
    It is a comparison tool for users, never a fallback for FusedNetwork."""

    def __init__(self, cfg: str, weight_dtype=torch.float16):
        super().__init__()
        cfg = json.loads(cfg)
        self._channels_in = cfg["num_inputs"]
        self._channels_out = cfg["num_outputs"]
        self._weight_dtype = weight_dtype
        if len(cfg["encodings"]) == 1:
            e = cfg["encodings"][0]
            if e["id"] != "Identity" or e["start_in"] != 0 or e["n_in"] != self._channels_in:
                raise ValueError("Only identity encoding supported and it must consume all inputs")
        elif len(cfg["encodings"]) > 1:
            raise ValueError("Only a single encoding supported")
        layers, self._has_bias = [], []
        n_in, n_out = self._channels_in, None
        for layer in cfg["network"]:
            n_out = layer["n_out"]
            layers.append(torch.nn.Linear(n_in, n_out, bias=layer["bias"], dtype=weight_dtype))
            layers.append(FusedActivation.get_activation(layer["activation"]))
            self._has_bias.append(layer["bias"])
            n_in = n_out
        if n_out != self._channels_out:
            raise ValueError("Last layer does not match the number of outputs")
        self.layers = torch.nn.Sequential(*layers)
        self._num_layers = len(cfg["network"])

    def channels_in(self):
        return self._channels_in

    def channels_out(self):
        return self._channels_out

    def num_layers(self) -> int:
        return self._num_layers

    def has_bias(self, layer: int):
        return self._has_bias[layer]

    def get_weight(self, layer: int, bias: bool, grad: bool) -> torch.Tensor:
        lin = self.layers[2 * layer]
        t = lin.bias if bias else lin.weight
        return torch.clone(t.grad.detach()) if grad else torch.clone(t.detach())

    def set_weight(self, layer: int, bias: bool, grad: bool, value: torch.Tensor):
        lin = self.layers[2 * layer]
        t = lin.bias if bias else lin.weight
        if grad:
            t.grad = torch.clone(value.detach())
        else:
            with torch.no_grad():
                t.copy_(value.detach())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.layers(x.to(self._weight_dtype)).to(torch.float32)


def copy_torch_to_fused(dst: FusedNetwork, src: SimulatedNetwork, grad: bool = False):
    """Copies weights (or gradients) of ``src`` into the padded matrices of ``dst`` (padding set to zero)."""
    assert dst.num_layers() == src.num_layers()
    with torch.no_grad():
        for layer in range(src.num_layers()):
            for bias in ([False, True] if src.has_bias(layer) else [False]):
                w = src.get_weight(layer, bias, grad)
                p = dst.weights.grad if grad else dst.weights.data
                t = dst._network.parameter_view(layer, bias, p)
                t.zero_()
                if bias:
                    t[:w.shape[0]].copy_(w.to(t.dtype))
                else:
                    t[:w.shape[0], :w.shape[1]].copy_(w.to(t.dtype))
