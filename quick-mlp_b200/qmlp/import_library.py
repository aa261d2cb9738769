"""Loads the native library once (role of src_py/qmlp/import_library.py:5-39)."""
from . import _capi


def load_library():
    if load_library.library_loaded:
        return
    lib = _capi.lib()
    if not lib.qmlp_is_cuda_available():
        # Same policy as the reference (import_library.py:23-29): objects could be built, but no kernel can launch.
        raise ImportError("CUDA not found, QuickMLP can't be imported")
    _capi.check(lib.qmlp_set_compile_debug_mode(0))
    _capi.check(lib.qmlp_set_log_level(b"warn"))
    load_library.library_loaded = True


load_library.library_loaded = False


def load_torch_classes():
    """Registers the TorchScript custom classes ``torch.classes.qmlp_cu.{QuickMLP, Network, Encoding, Activation}``
    (what ``torch.classes.load_library`` does for the reference's qmlp_cu.so, src_py/qmlp/import_library.py:19-21).
    Returns the ``torch.classes.qmlp_cu`` namespace. The extension is built by ``quick-mlp_b200/build_torch_ext.py``."""
    import os
    import torch
    if not load_torch_classes.loaded:
        path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "lib", "torch_ext", "qmlp_cu.so")
        if not os.path.exists(path):
            raise ImportError(f"{os.path.abspath(path)} not found: build it with `python quick-mlp_b200/build_torch_ext.py`")
        torch.classes.load_library(os.path.abspath(path))
        load_torch_classes.loaded = True
    return torch.classes.qmlp_cu


load_torch_classes.loaded = False
