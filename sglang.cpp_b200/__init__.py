"""B200-native (sm_100a) per-step token loop behind sglang.cpp's operator interface.

The directory is named ``sglang.cpp_b200``; import it through
``__graft_entry__.load_package()`` (module name ``sglang_cpp_b200``).  All
arithmetic runs in the CUDA kernels of ``lib/libb200_token_loop.so`` (C ABI:
``include/b200_token_loop.h``); importing this package without that library
raises — there is no CPU or eager fallback.
"""
from . import _lib
from ._lib import B200Error, EPILOGUE_GEGLU, EPILOGUE_NONE, EPILOGUE_SWIGLU


def load_library():
    """Load the C-ABI shared library (raises ImportError if it has not been built)."""
    return _lib.load()


def __getattr__(name):
    # torch-dependent host mirrors are imported lazily so that the symbol-export
    # checks can load the library without importing torch.
    if name == "layers":
        import importlib
        return importlib.import_module(".layers", __name__)
    if name == "engine":
        import importlib
        return importlib.import_module(".engine", __name__)
    raise AttributeError(name)
