"""Vectorised NumPy restatement of the reference's GGUF decode arithmetic.

Test infrastructure only (see the package docstring).  Each function names the
reference lines it restates; paths are relative to the reference project.
"""
from __future__ import annotations

import numpy as np

# ggml type ids and (elements per block, bytes per block):
# src/phfe/inference/gguf_loader.py:33-65
F32, F16, Q4_0, Q4_1, Q8_0, BF16 = 0, 1, 2, 3, 8, 30
# OR-ed into Q4_0 / Q4_1: ggml's own element order (low nibbles -> elements 0..15, high nibbles ->
# 16..31, as in ggml's published dequantize_row_q4_0/q4_1) instead of the reference's interleaving.
GGML_ORDER = 0x100
BLOCK_GEOMETRY = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), Q8_0: (32, 34)}
TYPE_NAMES = {F32: "F32", F16: "F16", BF16: "BF16", Q4_0: "Q4_0", Q4_1: "Q4_1", Q8_0: "Q8_0"}


def nbytes(ggml_type: int, numel: int) -> int:
    """``GGUFTensorInfo.nbytes`` (gguf_loader.py:131-139)."""
    ggml_type &= ~GGML_ORDER
    if ggml_type not in BLOCK_GEOMETRY:
        raise ValueError(f"Unknown dtype {ggml_type} for size calculation")
    be, bb = BLOCK_GEOMETRY[ggml_type]
    return (numel + be - 1) // be * bb


def _as_u8(data) -> np.ndarray:
    return np.frombuffer(data, dtype=np.uint8) if not isinstance(data, np.ndarray) else data.view(np.uint8).reshape(-1)


def _blocks(data, ggml_type: int, numel: int) -> np.ndarray:
    be, bb = BLOCK_GEOMETRY[ggml_type]
    n_blocks = (numel + be - 1) // be
    raw = _as_u8(data)
    if raw.size < n_blocks * bb:
        raise ValueError(f"Data too short: {raw.size} < {n_blocks * bb}")
    return raw[: n_blocks * bb].reshape(n_blocks, bb)


def _scale_f64(blocks: np.ndarray, col: int) -> np.ndarray:
    # np.frombuffer(..., float16)[0] -> float(...) widens exactly (gguf_loader.py:455-456)
    return np.ascontiguousarray(blocks[:, col:col + 2]).view("<f2").astype(np.float64)


def decode_f32(ggml_type: int, data, numel: int) -> np.ndarray:
    """The six decode functions of gguf_loader.py:407-554; returns float32[numel]."""
    if ggml_type & GGML_ORDER:
        base = ggml_type & ~GGML_ORDER
        if base not in (Q4_0, Q4_1):
            raise NotImplementedError(f"ggml element order applies to Q4_0/Q4_1, not type {base}")
        n_blocks = -(-numel // 32)
        v = decode_f32(base, data, n_blocks * 32).reshape(n_blocks, 16, 2)
        # interleaved slot 2j holds the low nibble of byte j, slot 2j+1 the high nibble
        return np.concatenate([v[:, :, 0], v[:, :, 1]], axis=1).reshape(-1)[:numel].copy()
    if ggml_type == F32:      # :407-410
        return _as_u8(data)[: numel * 4].view("<f4").copy()
    if ggml_type == F16:      # :413-416  exact widening
        return _as_u8(data)[: numel * 2].view("<f2").astype(np.float32)
    if ggml_type == BF16:     # :419-427  u16 << 16 reinterpreted
        return (_as_u8(data)[: numel * 2].view("<u2").astype(np.uint32) << 16).view(np.float32)
    blk = _blocks(data, ggml_type, numel)
    n_blocks = blk.shape[0]
    if ggml_type == Q8_0:     # :538-552  float32(int8) * d, float32 multiply
        d = _scale_f64(blk, 0).astype(np.float32)
        q = blk[:, 2:].view(np.int8).astype(np.float32)
        return (q * d).reshape(-1)[:numel]
    out = np.empty((n_blocks, 16, 2), dtype=np.float32)
    if ggml_type == Q4_0:     # :451-474  low nibble -> even slot, high nibble -> odd slot
        d = _scale_f64(blk, 0)
        qs = blk[:, 2:].astype(np.int16)
        out[:, :, 0] = ((qs & 0x0F) - 8) * d          # int16 * float64 -> float64 -> float32 store
        out[:, :, 1] = (((qs >> 4) & 0x0F) - 8) * d
        return out.reshape(-1)[:numel]
    if ggml_type == Q4_1:     # :496-517  q*d + m in float64, one rounding to float32
        d = _scale_f64(blk, 0)
        m = _scale_f64(blk, 2)
        qs = blk[:, 4:].astype(np.int16)
        out[:, :, 0] = (qs & 0x0F) * d + m
        out[:, :, 1] = ((qs >> 4) & 0x0F) * d + m
        return out.reshape(-1)[:numel]
    raise NotImplementedError(f"Dequantization not implemented for type {ggml_type}")


def cast_f32(values: np.ndarray, out_dtype: str) -> np.ndarray:
    """``tensor.to(dtype)`` on CPU (gguf_loader.py:378): one round-to-nearest-even.

    Returns float32 for "f32", float16 for "f16" and the raw bfloat16 bit
    patterns as uint16 for "bf16" (NumPy has no bfloat16 type).
    """
    v = np.ascontiguousarray(values, dtype=np.float32)
    if out_dtype == "f32":
        return v
    if out_dtype == "f16":
        with np.errstate(over="ignore"):
            return v.astype(np.float16)
    if out_dtype == "bf16":
        u = v.view(np.uint32)
        nan = (u & 0x7FFFFFFF) > 0x7F800000
        r = ((u.astype(np.uint64) + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
        r[nan] = ((u[nan] >> 16) | 0x0040).astype(np.uint16)
        return r
    raise ValueError(out_dtype)


def widen(values: np.ndarray, dtype: str) -> np.ndarray:
    """16-bit result back to float32 (exact)."""
    if dtype == "f32":
        return values.astype(np.float32, copy=False)
    if dtype == "f16":
        return values.astype(np.float32)
    if dtype == "bf16":
        return (values.astype(np.uint32) << 16).view(np.float32)
    raise ValueError(dtype)


def read_tensor(ggml_type: int, data, numel: int, out_dtype: str = "f32", via_dtype: str | None = None) -> np.ndarray:
    """Arithmetic of ``GGUFReader.read_tensor`` (gguf_loader.py:355-378), flat.

    ``via_dtype`` reproduces ``param.copy_(tensor)`` in ``patch_context``
    (gguf_loader.py:746, :758-759): the tensor is first rounded to ``via_dtype``
    and then converted to the parameter's ``out_dtype``.
    """
    v = decode_f32(ggml_type, data, numel)
    if via_dtype is not None and via_dtype != out_dtype:
        v = widen(cast_f32(v, via_dtype), via_dtype)
    return cast_f32(v, out_dtype)
