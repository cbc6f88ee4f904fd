"""Per-block Python loop port of the reference's quantized decode.

Test infrastructure only.  The reference decodes Q4_0/Q4_1/Q8_0 with one
Python-level iteration per 32-element block and a handful of tiny NumPy calls
inside it (src/phfe/inference/gguf_loader.py:451-474, :496-517, :538-552); that
loop, not the arithmetic, is what its CPU time is made of.  This port keeps
that cost structure -- one interpreter iteration and the same number of small
array operations per block -- so that timing it on the host cores of the GPU
machine stands in for timing the reference itself, which is not installed
there.  It is single-threaded because the reference is.
"""
from __future__ import annotations

import numpy as np

from .np_oracle import BLOCK_GEOMETRY, F16, F32, BF16, Q4_0, Q4_1, Q8_0, cast_f32, decode_f32


def decode_f32_loop(ggml_type: int, data: bytes, numel: int) -> np.ndarray:
    if ggml_type in (F32, F16, BF16):
        return decode_f32(ggml_type, data, numel)  # the reference is vectorised for these too
    per_block, stride = BLOCK_GEOMETRY[ggml_type]
    count = -(-numel // per_block)
    if len(data) < count * stride:
        raise ValueError(f"Data too short: {len(data)} < {count * stride}")
    result = np.zeros(count * per_block, dtype=np.float32)
    at = 0
    for k in range(count):
        lo_end = k * per_block
        if ggml_type == Q8_0:
            scale = float(np.frombuffer(data[at:at + 2], dtype=np.float16)[0])
            quants = np.frombuffer(data[at + 2:at + stride], dtype=np.int8)
            result[lo_end:lo_end + per_block] = quants.astype(np.float32) * scale
        else:
            scale = float(np.frombuffer(data[at:at + 2], dtype=np.float16)[0])
            if ggml_type == Q4_1:
                floor = float(np.frombuffer(data[at + 2:at + 4], dtype=np.float16)[0])
                packed = np.frombuffer(data[at + 4:at + stride], dtype=np.uint8).astype(np.int16)
                even = (packed & 15) * scale + floor
                odd = ((packed >> 4) & 15) * scale + floor
            else:
                packed = np.frombuffer(data[at + 2:at + stride], dtype=np.uint8).astype(np.int16)
                even = ((packed & 15) - 8) * scale
                odd = (((packed >> 4) & 15) - 8) * scale
            pair = np.empty(per_block, dtype=np.float32)
            pair[0::2] = even
            pair[1::2] = odd
            result[lo_end:lo_end + per_block] = pair
        at += stride
    return result[:numel]


def read_tensor_loop(ggml_type: int, data: bytes, numel: int, out_dtype: str = "f32") -> np.ndarray:
    return cast_f32(decode_f32_loop(ggml_type, data, numel), out_dtype)
