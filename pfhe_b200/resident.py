"""Decode packed GGUF tensors that already sit in device memory.

The reference keeps packed bytes on the GPU in ``StreamingGGUFLoader.stream_tensor_raw``
and decodes them with chains of torch ops (src/phfe/inference/gguf_cuda.py:52-116,
:231-245).  Here a whole batch goes through ``pfhe_dequant_launch_batch``: one
kernel launch per 32 quantised tensors.
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence, Tuple

import torch

from . import _native
from .gguf_loader import QUANT_INFO, _TORCH_TO_OUT


def decode_resident(items: Sequence[Tuple[torch.Tensor, int, Tuple[int, ...]]], dtype: torch.dtype = torch.float16,
                    out: Optional[Sequence[torch.Tensor]] = None) -> List[torch.Tensor]:
    """items: (packed uint8 CUDA tensor, ggml type, torch shape) per tensor.

    Returns one decoded tensor per item (``out[i]`` when given), all queued on
    the current stream of the tensors' device.
    """
    if dtype not in _TORCH_TO_OUT:
        raise ValueError(f"unsupported output dtype {dtype}")
    if not items:
        return []
    device = items[0][0].device
    descs = (_native.TensorDesc * len(items))()
    results: List[torch.Tensor] = []
    for i, (raw, ggml_type, shape) in enumerate(items):
        if raw.device != device or raw.dtype != torch.uint8 or not raw.is_contiguous():
            raise ValueError("packed tensors must be contiguous uint8 tensors on one CUDA device")
        if (ggml_type & ~_native.TYPE_FLAG_GGML_ORDER) not in QUANT_INFO:
            raise NotImplementedError(f"Dequantization not implemented for type {ggml_type}")
        numel = 1
        for s in shape:
            numel *= s
        dst = out[i] if out is not None else torch.empty(shape, dtype=dtype, device=device)
        if dst.dtype != dtype or dst.numel() != numel or not dst.is_contiguous() or dst.device != device:
            raise ValueError("out tensors must be contiguous, of the requested dtype and element count")
        descs[i] = _native.TensorDesc(ggml_type, _TORCH_TO_OUT[dtype], raw.data_ptr(), raw.numel(), dst.data_ptr(),
                                      dst.numel() * dst.element_size(), numel)
        results.append(dst)
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device).cuda_stream
        _native.check(_native.lib().pfhe_dequant_launch_batch(descs, len(items), stream))
    return results
