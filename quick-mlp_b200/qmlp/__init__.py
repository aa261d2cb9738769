"""Python face of the sm_100a fused-network library: the module layout and class names of the reference's
``qmlp`` package (src_py/qmlp/__init__.py:1-14), implemented over libqmlp_b200.so."""
from ._version import __version__
from .import_library import load_library, load_torch_classes
from .activation import FusedActivation
from .encoding import FusedEncoding
from .network import SimulatedNetwork, FusedNetwork, copy_torch_to_fused
from .trainer import FusedTrainer, shard_points

__all__ = [
    "__version__",
    "load_library",
    "load_torch_classes",
    "FusedActivation",
    "FusedEncoding",
    "FusedNetwork",
    "SimulatedNetwork",
    "copy_torch_to_fused",
    "FusedTrainer",
    "shard_points",
]
