"""CPU-side checks of the C ABI: the shared library loads and exports every symbol that
include/b200sparse.h declares (no kernel is launched), and the package refuses to run without it."""

import ctypes
import re
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "b200sparse.h"


def _declared_symbols():
    text = HEADER.read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b2s_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_symbols()
    for must in ("b2s_version", "b2s_status_string", "b2s_csr_inspect", "b2s_tile_count",
                 "b2s_tile_plan", "b2s_spmv_csr", "b2s_spmm_csr", "b2s_csr2csc_bytes",
                 "b2s_csr2csc"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from flagsparse_b200 import _lib
    assert _lib.LIB_PATH.exists(), "libb200sparse.so not built (python -m flagsparse_b200._build)"
    lib = ctypes.CDLL(str(_lib.LIB_PATH))
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} declared in b200sparse.h but not exported"
    # the ctypes table binds exactly the declared set
    assert sorted(_lib.SIGNATURES) == _declared_symbols()


def test_host_only_entry_points():
    from flagsparse_b200 import _lib
    lib = _lib.load()
    assert lib.b2s_version() == 100
    assert lib.b2s_status_string(0) == b"ok"
    assert b"dtype" in lib.b2s_status_string(1)
    assert lib.b2s_tile_count(10, 90, 32) == 4
    assert lib.b2s_tile_count(0, 0, 32) == 0
    assert lib.b2s_spmv_tile_items(0, 0) > 0 and lib.b2s_spmm_tile_items(0, 0) > 0
    assert lib.b2s_csr2csc_bytes(10, 10, 0) > 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from flagsparse_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libb200sparse.so")
    with pytest.raises(RuntimeError, match="no CPU or Triton fallback"):
        _lib.load()
