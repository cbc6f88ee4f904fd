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
# Formats the reference names but cannot decode (gguf_loader.py:37-46).  Their oracle restates ggml's
# published dequantize_row_* routines and is pinned to outputs of the gguf-py package (tests/golden).
Q5_0, Q5_1, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K = 6, 7, 10, 11, 12, 13, 14
BLOCK_GEOMETRY = {F32: (1, 4), F16: (1, 2), BF16: (1, 2), Q4_0: (32, 18), Q4_1: (32, 20), Q8_0: (32, 34),
                  Q5_0: (32, 22), Q5_1: (32, 24), Q2_K: (256, 84), Q3_K: (256, 110), Q4_K: (256, 144),
                  Q5_K: (256, 176), Q6_K: (256, 210)}
TYPE_NAMES = {F32: "F32", F16: "F16", BF16: "BF16", Q4_0: "Q4_0", Q4_1: "Q4_1", Q8_0: "Q8_0", Q5_0: "Q5_0", Q5_1: "Q5_1",
              Q2_K: "Q2_K", Q3_K: "Q3_K", Q4_K: "Q4_K", Q5_K: "Q5_K", Q6_K: "Q6_K"}


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
    if ggml_type in (Q5_0, Q5_1, Q2_K, Q3_K, Q4_K, Q5_K, Q6_K):
        return _decode_extra(ggml_type, blk).reshape(-1)[:numel]
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


def _f16_col(blk: np.ndarray, off: int) -> np.ndarray:
    return np.ascontiguousarray(blk[:, off:off + 2]).view("<f2").astype(np.float32).reshape(-1, 1)


def _decode_extra(t: int, blk: np.ndarray) -> np.ndarray:
    """Q5_0/Q5_1 and the K-quants, element by element index math; float32 arithmetic throughout.
    Every product formed before the last operation is exact, so the result is one rounding."""
    n = blk.shape[0]
    b = blk.astype(np.uint32)
    f32 = np.float32
    if t in (Q5_0, Q5_1):
        o = 2 if t == Q5_0 else 4
        e = np.arange(32)
        qh = np.ascontiguousarray(blk[:, o:o + 4]).view("<u4").reshape(n, 1)
        byte = b[:, o + 4 + (e & 15)]
        nib = np.where(e < 16, byte & 15, byte >> 4)
        q = (nib | (((qh >> e.astype(np.uint32)) & 1) << 4)).astype(np.int32)
        d = _f16_col(blk, 0)
        if t == Q5_0:
            return (d * (q - 16).astype(f32)).astype(f32)
        return (d * q.astype(f32) + _f16_col(blk, 2)).astype(f32)
    e = np.arange(256)
    sb, l = e >> 5, e & 31
    if t in (Q4_K, Q5_K):
        s = b[:, 4:16]
        j = np.arange(8)
        sc = np.where(j < 4, s[:, j % 4] & 63, (s[:, 8 + j % 4] & 15) | ((s[:, j % 4] >> 6) << 4))
        mn = np.where(j < 4, s[:, 4 + j % 4] & 63, (s[:, 8 + j % 4] >> 4) | ((s[:, 4 + j % 4] >> 6) << 4))
        qs_off = 16 if t == Q4_K else 48
        byte = b[:, qs_off + 32 * (sb >> 1) + l]
        q = np.where(sb & 1, byte >> 4, byte & 15)
        if t == Q5_K:
            q = q | (((b[:, 16 + l] >> sb.astype(np.uint32)) & 1) << 4)
        dl = (_f16_col(blk, 0) * sc.astype(f32)).astype(f32)
        ml = (_f16_col(blk, 2) * mn.astype(f32)).astype(f32)
        return (dl[:, sb] * q.astype(f32) - ml[:, sb]).astype(f32)
    if t == Q6_K:
        half, r = sb >> 2, sb & 3
        lo = b[:, 64 * half + 32 * (r & 1) + l]
        hi = b[:, 128 + 32 * half + l]
        q = (np.where(r >> 1, lo >> 4, lo & 15) | (((hi >> (2 * r).astype(np.uint32)) & 3) << 4)).astype(np.int32) - 32
        sc = blk[:, 192:208].view(np.int8).astype(f32)
        dl = (_f16_col(blk, 208) * sc).astype(f32)
        return (dl[:, e >> 4] * q.astype(f32)).astype(f32)
    half, r = e >> 7, (e >> 5) & 3
    if t == Q2_K:
        q = (b[:, 16 + 32 * half + l] >> (2 * r).astype(np.uint32)) & 3
        s = b[:, 0:16]
        dl = (_f16_col(blk, 80) * (s & 15).astype(f32)).astype(f32)
        ml = (_f16_col(blk, 82) * (s >> 4).astype(f32)).astype(f32)
        return (dl[:, e >> 4] * q.astype(f32) - ml[:, e >> 4]).astype(f32)
    if t == Q3_K:
        ql = (b[:, 32 + 32 * half + l] >> (2 * r).astype(np.uint32)) & 3
        hb = (b[:, l] >> sb.astype(np.uint32)) & 1
        q = (ql | (hb << 2)).astype(np.int32) - 4
        j = np.arange(16)
        s = b[:, 96:108]
        low = np.where(j < 8, s[:, j % 8] & 15, s[:, j % 8] >> 4)
        high = (s[:, 8 + (j & 3)] >> (2 * (j >> 2)).astype(np.uint32)) & 3
        sc = (low | (high << 4)).astype(np.int32) - 32
        dl = (_f16_col(blk, 108) * sc.astype(f32)).astype(f32)
        return (dl[:, e >> 4] * q.astype(f32)).astype(f32)
    raise NotImplementedError(t)


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
