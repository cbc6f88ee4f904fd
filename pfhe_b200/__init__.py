"""pfhe_b200: B200-native GGUF block decode behind phfe's loader API.

The public names mirror ``phfe.inference`` (reference
src/phfe/inference/__init__.py:51-62) for the GGUF loading path.
"""
from .gguf_loader import (
    GGUFHeader,
    GGUFModelPatcher,
    GGUFReader,
    GGUFTensorInfo,
    StreamingDequantizer,
    inspect_gguf,
    load_gguf_tensors,
    print_gguf_info,
    streaming_dequant_context,
    tensor_loading_context,
)

__all__ = [
    "GGUFReader", "GGUFTensorInfo", "GGUFHeader", "GGUFModelPatcher", "StreamingDequantizer",
    "tensor_loading_context", "streaming_dequant_context", "load_gguf_tensors", "inspect_gguf", "print_gguf_info",
]
