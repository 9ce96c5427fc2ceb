"""Legacy GGML container: host-side reader (candle-core/src/quantized/ggml_file.rs).  No GPU.

candle holds no fixture for this format, so the reader is pinned by restating ``ggml_file.rs`` and by
hand-assembled byte strings (built here with ``struct``, independently of the module's own writer) for
each magic, plus round trips through the writer."""
import io
import struct

import numpy as np
import pytest

from candle_b200 import CandleError, ggml_file
from helpers import make_qtable


def hand_built(magic_value, version, align, rng):
    """A two-tensor file assembled field by field as ggml_file.rs reads it."""
    q = make_qtable(rng, "q4_0", 6, 64)          # shape [6, 64] -> stored dims (64, 6)
    f32 = rng.standard_normal(5).astype("<f4")   # shape [5]
    out = io.BytesIO()
    out.write(struct.pack("<I", magic_value))
    if version is not None:
        out.write(struct.pack("<I", version))
    out.write(struct.pack("<7I", 3, 64, 256, 8, 2, 8, 2))
    for word, score in ((b"<s>", 0.0), (b"\xe2\x96\x81the", -3.5), (b"", 1.25)):
        out.write(struct.pack("<I", len(word)) + word + struct.pack("<f", score))
    for name, dtype, dims, data in ((b"tok_embeddings.weight", 2, (64, 6), q.tobytes()), (b"norm.weight", 0, (5,), f32.tobytes())):
        out.write(struct.pack("<3I", len(dims), len(name), dtype))
        out.write(struct.pack("<%dI" % len(dims), *dims))
        out.write(name)
        if align:
            out.write(b"\0" * ((32 - out.tell() % 32) % 32))
        out.write(data)
    return out.getvalue(), q, f32


@pytest.mark.parametrize("magic_value,version,name,align", [
    (0x67676D6C, None, "GgmlUnversioned", False), (0x67676D66, 1, "GgmfV1", False), (0x67676A74, 1, "GgjtV1", True),
    (0x67676A74, 2, "GgjtV2", True), (0x67676A74, 3, "GgjtV3", True)])
def test_reads_every_magic(magic_value, version, name, align):
    rng = np.random.default_rng(5)
    blob, q, f32 = hand_built(magic_value, version, align, rng)
    c = ggml_file.Content.read(io.BytesIO(blob))
    assert c.magic == name and ggml_file.align32(c.magic) == align
    assert c.hparams == ggml_file.HParams(3, 64, 256, 8, 2, 8, 2)
    assert c.vocab == [(b"<s>", 0.0), (b"\xe2\x96\x81the", -3.5), (b"", 1.25)]
    assert set(c.tensors) == {"tok_embeddings.weight", "norm.weight"}
    t = c.tensors["tok_embeddings.weight"]
    assert t.ggml_dtype == 2 and t.shape == (6, 64) and np.array_equal(t.data, q.reshape(-1))
    n = c.tensors["norm.weight"]
    assert n.ggml_dtype == 0 and n.shape == (5,) and np.array_equal(n.data.view("<f4"), f32)
    # remove() hands a tensor out once (ggml_file.rs:258-263)
    assert c.remove("norm.weight") is n
    with pytest.raises(CandleError, match="cannot find tensor with name 'norm.weight'"):
        c.remove("norm.weight")


def test_round_trip_through_the_writer():
    rng = np.random.default_rng(6)
    q8 = make_qtable(rng, "q8_0", 4, 96)
    hp = ggml_file.HParams(2, 96, 256, 4, 1, 24, 7)
    vocab = [(b"a", 0.5), (b"bc", -1.0)]
    for magic in ("GgmlUnversioned", "GgmfV1", "GgjtV3"):
        buf = io.BytesIO()
        ggml_file.write(buf, magic, hp, vocab, [("x", 8, (4, 96), q8.tobytes()), ("y", 1, (2, 3), b"\x00\x3c" * 6)])
        c = ggml_file.Content.read(io.BytesIO(buf.getvalue()))
        assert c.magic == magic and c.hparams == hp and c.vocab == vocab
        assert c.tensors["x"].shape == (4, 96) and np.array_equal(c.tensors["x"].data, q8.reshape(-1))
        assert c.tensors["y"].shape == (2, 3) and c.tensors["y"].data.tobytes() == b"\x00\x3c" * 6


def test_errors_follow_candle():
    with pytest.raises(CandleError, match="unknown magic 46554747"):
        ggml_file.Content.read(io.BytesIO(struct.pack("<II", 0x46554747, 3)))           # a GGUF file
    with pytest.raises(CandleError, match="unsupported magic/version Ggjt/4"):
        ggml_file.Content.read(io.BytesIO(struct.pack("<II", 0x67676A74, 4) + b"\0" * 28))
    with pytest.raises(CandleError, match="unsupported magic/version Ggla/1"):          # LoRA adapter files: no reader
        ggml_file.Content.read(io.BytesIO(struct.pack("<II", 0x67676C61, 1) + b"\0" * 28))
    head = struct.pack("<I", 0x67676D6C) + struct.pack("<7I", 0, 32, 0, 0, 0, 0, 0)
    bad_dtype = head + struct.pack("<3I", 1, 1, 4) + struct.pack("<I", 32) + b"w"
    with pytest.raises(CandleError, match="unknown dtype for tensor 4"):
        ggml_file.Content.read(io.BytesIO(bad_dtype))
    ragged = head + struct.pack("<3I", 1, 1, 2) + struct.pack("<I", 40) + b"w" + b"\0" * (40 * 18 // 32)
    with pytest.raises(CandleError, match="Error creating tensor w: the number of elements 40 is not divisible by the block size 32"):
        ggml_file.Content.read(io.BytesIO(ragged))
    q8k = head + struct.pack("<3I", 1, 1, 15) + struct.pack("<I", 256) + b"w" + b"\0" * 292
    with pytest.raises(CandleError, match="quantized type Q8K is not supported yet"):
        ggml_file.Content.read(io.BytesIO(q8k))
    with pytest.raises(CandleError, match="failed to fill whole buffer"):               # truncated payload
        ggml_file.Content.read(io.BytesIO(head + struct.pack("<3I", 1, 1, 2) + struct.pack("<I", 32) + b"w" + b"\0" * 5))


@pytest.mark.gpu
def test_gpu_lookup_from_a_legacy_file(cb):
    import torch

    import oracle
    from helpers import ids_tensor, to_oracle

    rng = np.random.default_rng(7)
    q = make_qtable(rng, "q4_0", 50, 256)
    buf = io.BytesIO()
    ggml_file.write(buf, "GgjtV3", ggml_file.HParams(0, 256, 0, 0, 0, 0, 2), [], [("tok_embeddings.weight", 2, (50, 256), q.tobytes())])
    c = ggml_file.Content.read(io.BytesIO(buf.getvalue()))
    table = c.tensor("tok_embeddings.weight", "cuda")
    ids = rng.integers(0, 50, size=(33,)).astype(np.uint32)
    got = table.embedding(ids_tensor(ids), torch.bfloat16)
    assert np.array_equal(to_oracle(got), oracle.qembedding(q, "q4_0", ids, "bf16"))
