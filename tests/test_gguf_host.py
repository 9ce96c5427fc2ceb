"""GGUF container: host-side reader / writer (candle-core/src/quantized/gguf_file.rs).  No GPU."""
import io
import struct

import numpy as np
import pytest

from candle_b200 import gguf
from candle_b200.errors import CandleError
from helpers import make_qtable


def _sample():
    rng = np.random.default_rng(3)
    q8 = make_qtable(rng, "q8_0", 10, 64)   # 10 x 64 -> 2 blocks of 34 bytes per row
    q4 = make_qtable(rng, "q4_0", 7, 96)
    f32 = rng.standard_normal((5, 3)).astype(np.float32)
    meta = [
        ("general.architecture", gguf.Value("String", "llama")),
        ("llama.block_count", gguf.Value("U32", 2)),
        ("llama.rope.freq_base", gguf.Value("F32", 10000.0)),
        ("flag", gguf.Value("Bool", True)),
        ("tokens", gguf.Value("Array", [gguf.Value("String", s) for s in ("<s>", "</s>", "a")])),
        ("scores", gguf.Value("Array", [gguf.Value("F32", v) for v in (0.0, -1.5)])),
        ("empty", gguf.Value("Array", [])),
        ("big", gguf.Value("U64", 2**40)), ("neg", gguf.Value("I64", -5)), ("small", gguf.Value("I8", -3)),
    ]
    tensors = [("token_embd.weight", 8, (10, 64), q8), ("other.weight", 2, (7, 96), q4), ("norm.weight", 0, (5, 3), f32)]
    return meta, tensors


def test_write_then_read_round_trip():
    meta, tensors = _sample()
    buf = io.BytesIO()
    gguf.write(buf, meta, tensors)
    raw = buf.getvalue()
    assert raw[:4] == b"GGUF" and struct.unpack("<I", raw[4:8])[0] == 2
    buf.seek(0)
    c = gguf.Content.read(buf)
    assert c.version == 2 and c.tensor_data_offset % 32 == 0
    assert {k: (v.type, v.value) for k, v in c.metadata.items() if v.type != "Array"} == {
        k: (v.type, v.value) for k, v in meta if v.type != "Array"}
    assert [v.value for v in c.metadata["tokens"].value] == ["<s>", "</s>", "a"]
    assert c.metadata["empty"].value == [] and c.metadata["big"].to_u64() == 2**40
    with pytest.raises(CandleError, match="not a u64"):
        c.metadata["neg"].to_u64()
    for name, dtype, shape, data in tensors:
        info = c.tensor_info(name)
        assert (info.ggml_dtype, info.shape) == (dtype, shape) and info.offset % 32 == 0
        assert np.array_equal(c.tensor_raw(buf, name), np.ascontiguousarray(data).reshape(-1).view(np.uint8))
    with pytest.raises(CandleError, match="cannot find tensor info for nope"):
        c.tensor_info("nope")
    # writing what was read gives the same bytes (metadata keeps its types, tensors their order)
    again = io.BytesIO()
    gguf.write(again, list(c.metadata.items()), [(n, i.ggml_dtype, i.shape, c.tensor_raw(buf, n))
                                                  for n, i in c.tensor_infos.items()])
    assert again.getvalue() == raw


def test_versions_alignment_and_errors():
    # version 1: 32-bit counts, lengths and dimensions; a custom alignment; a NUL-terminated string
    body = struct.pack("<IIII", 0x46554747, 1, 1, 2)
    body += struct.pack("<I", 17) + b"general.alignment" + struct.pack("<II", 4, 64)
    body += struct.pack("<I", 4) + b"name" + struct.pack("<I", 8) + struct.pack("<I", 4) + b"ab\0\0"
    body += struct.pack("<I", 1) + b"t" + struct.pack("<I", 2) + struct.pack("<II", 32, 3) + struct.pack("<IQ", 8, 0)
    data = np.arange(3 * 34, dtype=np.uint8)
    pad = -len(body) % 64
    f = io.BytesIO(body + b"\0" * pad + data.tobytes())
    c = gguf.Content.read(f)
    assert c.version == 1 and c.tensor_data_offset == len(body) + pad and c.metadata["name"].value == "ab"
    assert c.tensor_info("t").shape == (3, 32)  # stored innermost-first
    assert np.array_equal(c.tensor_raw(f, "t"), data)
    with pytest.raises(CandleError, match="unknown magic"):
        gguf.Content.read(io.BytesIO(b"GGML" + b"\0" * 20))
    with pytest.raises(CandleError, match="unsupported magic/version"):
        gguf.Content.read(io.BytesIO(struct.pack("<II", 0x46554747, 4) + b"\0" * 16))
    with pytest.raises(CandleError, match="failed to fill whole buffer"):
        gguf.Content.read(io.BytesIO(struct.pack("<IIQ", 0x46554747, 3, 1)))
    with pytest.raises(CandleError, match="multiple value-types"):
        gguf.write(io.BytesIO(), [("x", gguf.Value("Array", [gguf.Value("U8", 1), gguf.Value("I8", 1)]))], [])
    with pytest.raises(CandleError, match="do not match shape"):
        gguf.write(io.BytesIO(), [], [("t", 8, (2, 32), np.zeros(10, np.uint8))])
    with pytest.raises(CandleError, match="not divisible by the block size"):
        gguf.TensorInfo(8, (3, 5), 0).size_in_bytes
