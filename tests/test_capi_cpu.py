"""The C-ABI library loads without a GPU and exports every symbol the public header declares."""
import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200_token_loop.h"


def declared_symbols():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = declared_symbols()
    assert "b200_linear" in syms and "b200_attention_decode" in syms
    assert len(syms) >= 15


def test_library_exports_every_declared_symbol(pkg):
    lib = pkg.load_library()
    missing = [s for s in declared_symbols() if not hasattr(lib, s)]
    assert not missing, f"declared in the header but not exported: {missing}"


def test_binding_covers_every_declared_symbol(pkg):
    from sglang_cpp_b200 import _lib

    unbound = [s for s in declared_symbols() if s not in _lib.PROTOTYPES]
    assert not unbound, f"no ctypes prototype for: {unbound}"
    stale = [s for s in _lib.PROTOTYPES if s not in declared_symbols()]
    assert not stale, f"prototype without a declaration: {stale}"


def test_abi_version_and_error_text(pkg):
    lib = pkg.load_library()
    assert lib.b200_abi_version() == 1
    # Argument checks run before any CUDA call, so they work without a GPU.
    rc = lib.b200_rmsnorm(None, None, None, 1, 8, ctypes.c_float(1e-6), None)
    assert rc == 1
    assert b"NULL" in lib.b200_last_error()
    rc = lib.b200_linear(ctypes.c_void_p(16), ctypes.c_void_p(16), ctypes.c_void_p(16), None, 4, 64, 100, 100, 0, None)
    assert rc == 1 and b"multiple of 64" in lib.b200_last_error()


def test_missing_library_fails_loudly(pkg, monkeypatch, tmp_path):
    from sglang_cpp_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()
