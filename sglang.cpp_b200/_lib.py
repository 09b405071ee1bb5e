"""ctypes binding of ``libb200_token_loop.so`` (the C ABI in ``include/b200_token_loop.h``).

The binding is deliberately thin: every Python-visible operator in this package
ends in exactly one of the calls declared here, and there is no fallback of any
kind — if the shared library is missing the import fails with instructions to
build it.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p, POINTER
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
LIB_PATH = PKG_DIR / "lib" / "libb200_token_loop.so"

B200_OK = 0
ERROR_NAMES = {
    1: "B200_ERR_INVALID_ARGUMENT",
    2: "B200_ERR_CUDA",
    3: "B200_ERR_TIMEOUT",
    4: "B200_ERR_UNSUPPORTED",
    5: "B200_ERR_STATE",
}

EPILOGUE_NONE = 0
EPILOGUE_SWIGLU = 1
EPILOGUE_GEGLU = 2


class B200Error(RuntimeError):
    """Raised when a C-ABI call returns a non-zero status (the reference raises c10::Error)."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{ERROR_NAMES.get(code, code)}: {message}")
        self.code = code


_P = c_void_p
_I = c_int
_L = c_int64
_F = c_float

# name -> (restype, argtypes).  Every symbol include/b200_token_loop.h declares is listed.
PROTOTYPES: dict[str, tuple] = {
    "b200_last_error": (c_char_p, []),
    "b200_abi_version": (_I, []),
    "b200_read_device_status": (_I, [POINTER(c_int32), _P]),
    "b200_rmsnorm": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "b200_fused_add_rmsnorm": (_I, [_P, _P, _P, _I, _I, _F, _P]),
    "b200_qk_rmsnorm_strided": (_I, [_P, _P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _L, _F, _P]),
    "b200_rope_neox_inplace": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _L, _L, _L, _L, _P]),
    "b200_store_kv": (_I, [_P, _P, _P, _P, _P, _I, _I, _I, _L, _L, _L, _P]),
    "b200_qknorm_rope_store": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _L, _F, _I, _P]),
    "b200_silu_and_mul": (_I, [_P, _P, _I, _I, _P]),
    "b200_gelu_and_mul": (_I, [_P, _P, _I, _I, _P]),
    "b200_embedding": (_I, [_P, _P, _P, _I, _I, _I, _P]),
    "b200_gather_int32_2d": (_I, [_P, _P, _L, _L, _L, _P, _P, _L, _P]),
    "b200_write_token_pool": (_I, [_P, _L, _L, _L, _P, _P, _P, _L, _P]),
    "b200_linear": (_I, [_P, _P, _P, _P, _I, _I, _I, _L, _I, _P]),
    "b200_attention_decode_workspace_bytes": (_L, [_I, _I, _I, _I]),
    "b200_attention_decode": (_I, [_P, _P, _L, _L, _P, _P, _L, _P, _L, _P, _P, _I, _I, _I, _I, _I, _F, _P, _L, _P]),
    "b200_attention_prefill": (_I, [_P, _P, _L, _L, _P, _P, _L, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _P]),
    "b200_argmax": (_I, [_P, _P, _I, _I, _L, _P]),
}

_lib = None


def load() -> ctypes.CDLL:
    """Load the shared library (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
            "(nvcc, sm_100a).  There is no fallback path."
        )
    lib = ctypes.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(code: int) -> None:
    if code != B200_OK:
        msg = load().b200_last_error()
        raise B200Error(code, msg.decode() if msg else "")


def call(name: str, *args) -> None:
    """Call an int-returning entry point and raise B200Error on a non-zero status."""
    check(getattr(load(), name)(*args))
