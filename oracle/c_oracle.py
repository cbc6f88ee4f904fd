"""ctypes wrapper over ``dequant_oracle.c`` (test infrastructure only)."""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_OUT = {"f32": 0, "f16": 1, "bf16": 2}
GGML_ORDER = 0x100
_NP_OUT = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16}
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile beside it."""
    src = os.path.join(_HERE, "dequant_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        L.oracle_nbytes.restype = ctypes.c_int64
        L.oracle_nbytes.argtypes = [ctypes.c_int, ctypes.c_int64]
        L.oracle_read_tensor.restype = ctypes.c_int
        L.oracle_read_tensor.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,
                                         ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        L.oracle_cast.restype = ctypes.c_int
        L.oracle_cast.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p, ctypes.c_int]
        L.oracle_widen.restype = ctypes.c_int
        L.oracle_widen.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
        L.oracle_max_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def read_tensor(ggml_type: int, data, numel: int, out_dtype: str = "f32", via_dtype: str | None = None,
                n_threads: int = 1, out: np.ndarray | None = None, scratch: np.ndarray | None = None) -> np.ndarray:
    """Decode + cast; bf16 is returned as raw uint16 bit patterns."""
    raw = np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1)
    L = lib()
    first = via_dtype if (via_dtype is not None and via_dtype != out_dtype) else out_dtype
    res = out if (out is not None and first == out_dtype) else np.empty(numel, dtype=_NP_OUT[first])
    if first != "f32" and scratch is None:
        scratch = np.empty(numel, dtype=np.float32)
    rc = L.oracle_read_tensor(ggml_type, raw.ctypes.data, raw.size, numel, _OUT[first], res.ctypes.data,
                              scratch.ctypes.data if scratch is not None else None, n_threads)
    if rc == -1:
        raise NotImplementedError(f"Dequantization not implemented for type {ggml_type}")
    if rc == -2:
        raise ValueError(f"Data too short: {raw.size} < {L.oracle_nbytes(ggml_type, numel)}")
    if first == out_dtype:
        return res
    wide = np.empty(numel, dtype=np.float32)
    L.oracle_widen(res.ctypes.data, numel, _OUT[first], wide.ctypes.data)
    final = out if out is not None else np.empty(numel, dtype=_NP_OUT[out_dtype])
    L.oracle_cast(wide.ctypes.data, numel, _OUT[out_dtype], final.ctypes.data, n_threads)
    return final
