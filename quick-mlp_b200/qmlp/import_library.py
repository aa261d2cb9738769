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
