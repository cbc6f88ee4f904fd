"""The C-ABI library loads and exports every symbol the header declares (no GPU compute)."""
import ctypes
import os
import re

import pytest

from pfhe_b200 import _native

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "pfhe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pfhe_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    L = _native.lib()
    names = _declared()
    assert set(names) == set(_native.EXPORTED_SYMBOLS)
    for n in names:
        assert getattr(L, n) is not None


def test_version_and_nbytes():
    L = _native.lib()
    assert L.pfhe_version() >= 100
    assert L.pfhe_tensor_nbytes(2, 32) == 18 and L.pfhe_tensor_nbytes(2, 33) == 36
    assert L.pfhe_tensor_nbytes(3, 64) == 40 and L.pfhe_tensor_nbytes(8, 1) == 34
    assert L.pfhe_tensor_nbytes(0, 5) == 20 and L.pfhe_tensor_nbytes(1, 5) == 10 and L.pfhe_tensor_nbytes(30, 5) == 10
    assert L.pfhe_tensor_nbytes(6, 32) == 22 and L.pfhe_tensor_nbytes(7, 33) == 48          # Q5_0, Q5_1
    assert [L.pfhe_tensor_nbytes(t, 257) for t in (10, 11, 12, 13, 14)] == [168, 220, 288, 352, 420]   # K-quants
    assert L.pfhe_tensor_nbytes(9, 32) == _native.ERR_BAD_TYPE
    assert "not one of" in _native.last_error()


def test_argument_errors_map_to_reference_exceptions():
    L = _native.lib()
    # all of these are rejected before any CUDA call
    rc = L.pfhe_dequant_launch(15, 0, None, 0, None, 0, 32, None)
    with pytest.raises(NotImplementedError):
        _native.check(rc)
    rc = L.pfhe_dequant_launch(2, 7, None, 18, None, 128, 32, None)
    with pytest.raises(ValueError):
        _native.check(rc)
    rc = L.pfhe_dequant_launch(2, 0, None, 17, None, 128, 32, None)
    assert rc == _native.ERR_SHORT_SOURCE
    with pytest.raises(ValueError, match="Data too short: 17 < 18"):
        _native.check(rc)
    assert L.pfhe_dequant_launch(2, 1, None, 18, None, 63, 32, None) == _native.ERR_SHORT_DEST
    assert L.pfhe_dequant_launch(2, 1, None, 0, None, 0, 0, None) == _native.OK      # nothing to do
    assert L.pfhe_loader_submit(None, None, 0, 2, 1, 1, None, 0, 0, None) == _native.ERR_BAD_ARG
    handle = ctypes.c_void_p()
    assert L.pfhe_loader_create(0, 0, 1 << 20, 1, ctypes.byref(handle)) == _native.ERR_BAD_ARG
    assert L.pfhe_loader_destroy(None) == _native.OK


def test_missing_library_is_loud(monkeypatch):
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", "/nonexistent/libpfhe_b200.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _native.lib()
