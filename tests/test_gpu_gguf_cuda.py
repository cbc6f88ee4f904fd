"""The mirror of the reference's gguf_cuda module against what that module itself produced
(tests/golden/gguf_cuda_stream.npz, made by running the reference with device="cpu")."""
import os

import numpy as np
import pytest
import torch

from conftest import assert_same_bits
from gpu_util import to_bits
from oracle import np_oracle
from pfhe_b200 import gguf_cuda, gguf_loader as gl

pytestmark = pytest.mark.gpu

DT = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
TYPES = {"Q4_0": 2, "Q8_0": 8}


@pytest.fixture(scope="module")
def golden(golden_dir):
    return np.load(os.path.join(golden_dir, "gguf_cuda_stream.npz"))


@pytest.mark.parametrize("key", list(DT))
def test_stream_tensor_matches_the_reference_loader(golden_dir, golden, key):
    path = os.path.join(golden_dir, "mini.gguf")
    seen = 0
    with gl.GGUFReader(path) as r:
        names = list(r.tensors)
    with gguf_cuda.StreamingGGUFLoader(path, device="cuda", dtype=DT[key]) as sl:
        assert sl.tensor_names == names
        for name in sl.tensor_names:
            t = sl.stream_tensor(name)
            meta = sl.get_tensor_meta(name)
            assert t.is_cuda and t.dtype == DT[key] and tuple(t.shape) == tuple(meta.shape)
            if f"{name}|{key}" in golden.files:
                assert_same_bits(to_bits(t.reshape(-1)), golden[f"{name}|{key}"], key, name)
                seen += 1
            else:                           # what the reference cannot stream (Q4_1, ragged counts) loads here: decode -> fp16 -> dtype
                assert f"{name}|{key}|unsupported" in golden.files
                with gl.GGUFReader(path) as r:
                    raw, info = r.read_tensor_raw(name), r.tensors[name]
                want = np_oracle.read_tensor(info.dtype, np.frombuffer(raw, dtype=np.uint8), info.numel, key, via_dtype="f16")
                assert_same_bits(to_bits(t.reshape(-1)), want.reshape(-1), key, name)
        assert [n for n, _ in sl.stream_tensors()] == sl.tensor_names
        raw = sl.stream_tensor_raw("token_embd.weight")
        with gl.GGUFReader(path) as r:
            assert raw.dtype == torch.uint8 and raw.is_cuda and bytes(raw.cpu().numpy()) == r.read_tensor_raw("token_embd.weight")
        with pytest.raises(KeyError):
            sl.stream_tensor("nope")
    assert seen == 5


@pytest.mark.parametrize("fmt", list(TYPES))
@pytest.mark.parametrize("numel", [32, 100, 4096 + 31])
@pytest.mark.parametrize("where", ["cuda", "cpu"])
def test_dequant_functions_match_the_reference(golden, fmt, numel, where):
    raw = torch.from_numpy(golden[f"fn|{fmt}|{numel}|raw"].copy())
    want = golden[f"fn|{fmt}|{numel}|out"]
    fn = gguf_cuda.dequant_q4_0_cuda if fmt == "Q4_0" else gguf_cuda.dequant_q8_0_cuda
    out = fn(raw.cuda() if where == "cuda" else raw, numel, "cuda")
    assert out.is_cuda and out.dtype == torch.float16 and out.numel() == numel // 32 * 32 == want.size
    assert_same_bits(to_bits(out), want, "f16", f"{fmt} {numel}")


def test_module_surface():
    for name in ("TensorMeta", "dequant_q8_0_cuda", "dequant_q4_0_cuda", "StreamingGGUFLoader", "QuantizedTensor",
                 "quantized_matmul_q8_0", "quantized_matmul_q4_0", "QuantizedLinear", "QK4_0", "QK8_0"):
        assert hasattr(gguf_cuda, name)
