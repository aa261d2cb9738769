"""Network specifications used by the parity tests: the five benchmark configurations and the builders for
scaled-down relatives of them that the CPU oracle finishes in seconds (all defined in the package, qmlp/configs.py)."""
from qmlp.configs import (BUILTIN, config1, config2, config3, config4, config5, dumps, grid_net, hashgrid,  # noqa: F401
                          identity_net, mlp)
