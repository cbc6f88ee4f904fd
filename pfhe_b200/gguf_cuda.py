"""Drop-in for ``phfe.inference.gguf_cuda`` (reference src/phfe/inference/gguf_cuda.py).

The reference module streams GGUF tensors to the GPU as raw bytes and dequantises them there with
chains of torch ops (``dequant_q8_0_cuda`` :52-80, ``dequant_q4_0_cuda`` :83-116,
``StreamingGGUFLoader`` :119-245), and keeps weights quantised in ``QuantizedTensor`` /
``QuantizedLinear`` (:247-401).  Same names, arguments and results here; the work is done by the
library's kernels:

* ``dequant_q8_0_cuda`` / ``dequant_q4_0_cuda``: one decode launch, bits as the reference's
  ``(q * scale)`` in fp32 rounded to fp16; like the reference they decode ``numel // 32`` whole
  blocks.
* ``StreamingGGUFLoader.stream_tensor``: packed bytes through the pinned ring, decoded straight
  into the result.  The reference decodes quantised and BF16 tensors to fp16 first and converts to
  the loader's dtype afterwards; that double rounding is reproduced.  Additions: Q4_1, the ggml
  formats of ``QUANT_INFO`` and element counts that are not multiples of 32 load too (the reference
  raises for them, and ``stream_tensors`` skips them).
* ``stream_tensor_raw``: ``GGUFReader.read_tensor_packed``.
* ``QuantizedTensor``, ``quantized_matmul_q8_0`` / ``_q4_0``, ``QuantizedLinear``: ``pfhe_b200.quantized``.
"""
from __future__ import annotations

import logging
from dataclasses import dataclass
from pathlib import Path
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from .gguf_loader import GGML_TYPE_F16, GGML_TYPE_F32, GGML_TYPE_Q4_0, GGML_TYPE_Q8_0, QUANT_INFO, GGUFReader, _cuda_device_for
from .quantized import QuantizedLinear, QuantizedTensor, quantized_matmul_q4_0, quantized_matmul_q8_0  # noqa: F401  (re-exported)
from .resident import decode_resident

logger = logging.getLogger(__name__)

QK4_0 = 32
QK8_0 = 32


@dataclass
class TensorMeta:
    """Minimal tensor metadata for streaming (reference :26-32)."""
    shape: Tuple[int, ...]
    dtype: int
    offset: int
    nbytes: int


def _dequant_blocks(raw: torch.Tensor, numel: int, device: str, ggml_type: int, block_bytes: int) -> torch.Tensor:
    n_blocks = numel // 32
    want, cuda_dev = _cuda_device_for(device)
    on_host = raw.device.type != "cuda"
    if on_host:
        raw = raw.to(cuda_dev, non_blocking=True)
    packed = raw.reshape(-1).view(torch.uint8)[: n_blocks * block_bytes].contiguous()
    if packed.numel() < n_blocks * block_bytes:
        raise ValueError(f"Data too short: {packed.numel()} < {n_blocks * block_bytes}")
    if n_blocks == 0:
        out = torch.empty(0, dtype=torch.float16, device=raw.device)
    else:
        out = decode_resident([(packed, ggml_type, (n_blocks * 32,))], torch.float16)[0][:numel]
    return out.to(want) if on_host and want.type != "cuda" else out


def dequant_q8_0_cuda(raw: torch.Tensor, numel: int, device: str) -> torch.Tensor:
    """Q8_0 bytes (a uint8 tensor) to a flat fp16 tensor on the GPU (reference :52-80)."""
    return _dequant_blocks(raw, numel, device, GGML_TYPE_Q8_0, 2 + QK8_0)


def dequant_q4_0_cuda(raw: torch.Tensor, numel: int, device: str) -> torch.Tensor:
    """Q4_0 bytes to a flat fp16 tensor on the GPU, low nibble first within each byte (reference :83-116)."""
    return _dequant_blocks(raw, numel, device, GGML_TYPE_Q4_0, 2 + QK4_0 // 2)


class StreamingGGUFLoader:
    """Streams GGUF tensors to the GPU and decodes them there (reference :119-245).

        with StreamingGGUFLoader(path, device="cuda") as loader:
            for name, tensor in loader.stream_tensors():
                ...
    """

    def __init__(self, path: str, device: str = "cuda", dtype: torch.dtype = torch.float16):
        self.path = Path(path)
        self.device = device
        self.dtype = dtype
        self._reader: Optional[GGUFReader] = None
        self._tensor_metas: Optional[Dict[str, TensorMeta]] = None
        self._data_offset: Optional[int] = None

    def open(self):
        self._reader = GGUFReader(self.path)
        self._reader.__enter__()
        self._tensor_metas = {name: TensorMeta(shape=info.shape, dtype=info.dtype, offset=info.offset, nbytes=info.nbytes)
                              for name, info in self._reader.tensors.items()}
        self._data_offset = self._reader.header.tensor_data_offset
        logger.info(f"Opened {self.path}: {len(self._tensor_metas)} tensors")

    def close(self):
        if self._reader is not None:
            self._reader.__exit__(None, None, None)
            self._reader = None

    def __enter__(self):
        self.open()
        return self

    def __exit__(self, *args):
        self.close()

    @property
    def tensor_names(self) -> List[str]:
        return list(self._tensor_metas.keys())

    def stream_tensor(self, name: str) -> torch.Tensor:
        """One tensor, decoded on the GPU, in the loader's dtype (reference :179-220)."""
        meta = self._tensor_metas[name]
        if meta.dtype not in QUANT_INFO:
            raise ValueError(f"Unsupported dtype {meta.dtype} for tensor {name}")
        # F32 and F16 sources are converted once; everything else is decoded to fp16 and then
        # converted, as `dequant_*_cuda(...)` / `.to(torch.float16)` followed by `.to(self.dtype)` do.
        via = self.dtype if meta.dtype in (GGML_TYPE_F32, GGML_TYPE_F16) else torch.float16
        _, cuda_dev = _cuda_device_for(self.device)
        out = torch.empty(meta.shape, dtype=self.dtype, device=cuda_dev)
        self._reader.read_tensor(name, dtype=via, out=out)
        return out if torch.device(self.device).type == "cuda" else out.to(self.device)

    def stream_tensors(self) -> Iterator[Tuple[str, torch.Tensor]]:
        """(name, tensor) for every tensor; a tensor that fails to load is logged and skipped (reference :222-229)."""
        for name in self._tensor_metas:
            try:
                tensor = self.stream_tensor(name)
                yield name, tensor
            except Exception as e:       # the reference's behaviour: warn and go on
                logger.warning(f"Failed to load {name}: {e}")

    def stream_tensor_raw(self, name: str) -> torch.Tensor:
        """The tensor's packed bytes on the GPU, undecoded (reference :231-240)."""
        self._tensor_metas[name]         # KeyError for an unknown name, as in the reference
        _, cuda_dev = _cuda_device_for(self.device)
        return self._reader.read_tensor_packed(name, device=str(cuda_dev))

    def get_tensor_meta(self, name: str) -> TensorMeta:
        return self._tensor_metas[name]
