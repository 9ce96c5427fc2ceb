"""Reader for the legacy GGML container (the pre-GGUF llama.cpp format), host only.

Mirrors ``candle_core::quantized::ggml_file`` (candle-core/src/quantized/ggml_file.rs): the magic
and, except for the unversioned ``ggml`` magic, a version (:35-60); seven 32-bit hyper-parameters
(:74-99); ``n_vocab`` tokens, each a length-prefixed byte string followed by an f32 score -- read
for every magic, as candle does (:106-117); then tensors until the end of the file, each with its
dimensions stored innermost-first and reversed on read, its name, and -- for the ``ggjt`` magics
only -- padding to the next multiple of 32 bytes before the data (:188-219).  Element counts must
be whole blocks (:143-149).  Tensor payloads stay raw bytes on the host; ``Content.tensor`` moves
a block-quantised one to the GPU for the lookups.  There is no writer in the reference, and none
here beyond ``write`` for tests and fixtures, which emits exactly what ``Content.read`` accepts.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass, field

import numpy as np

from .errors import CandleError
from .gguf import GGML_TYPES

# ggml_file.rs:20-29; ggla (LoRA adapters) and ggsn (session files) are known magics without a reader
_MAGIC_NAMES = {0x67676A74: "Ggjt", 0x67676C61: "Ggla", 0x67676D66: "Ggmf", 0x67676D6C: "Ggml", 0x6767736E: "Ggsn"}
_VERSIONED = {("Ggmf", 1): "GgmfV1", ("Ggjt", 1): "GgjtV1", ("Ggjt", 2): "GgjtV2", ("Ggjt", 3): "GgjtV3"}
_MAGIC_VALUES = {"GgmlUnversioned": (0x67676D6C, None), "GgmfV1": (0x67676D66, 1), "GgjtV1": (0x67676A74, 1),
                 "GgjtV2": (0x67676A74, 2), "GgjtV3": (0x67676A74, 3)}
# types `qtensor_from_ggml` accepts (ggml_file.rs:152-185): no Q8_1, no Q8K
_LOADABLE = {0, 1, 2, 3, 6, 7, 8, 10, 11, 12, 13, 14}


def _read_exact(f, n: int) -> bytes:
    data = f.read(n)
    if len(data) != n:
        raise CandleError("failed to fill whole buffer")
    return data


def _u32(f) -> int:
    return struct.unpack("<I", _read_exact(f, 4))[0]


def align32(magic: str) -> bool:
    """``VersionedMagic::align32`` (ggml_file.rs:62-67)."""
    return magic.startswith("Ggjt")


def read_magic(f) -> str:
    value = _u32(f)
    name = _MAGIC_NAMES.get(value)
    if name is None:
        raise CandleError(f"unknown magic {value:08x}")
    if name == "Ggml":
        return "GgmlUnversioned"
    version = _u32(f)
    versioned = _VERSIONED.get((name, version))
    if versioned is None:
        raise CandleError(f"ggml: unsupported magic/version {name}/{version}")
    return versioned


@dataclass
class HParams:
    n_vocab: int
    n_embd: int
    n_mult: int
    n_head: int
    n_layer: int
    n_rot: int
    ftype: int

    @classmethod
    def read(cls, f) -> "HParams":
        return cls(*struct.unpack("<7I", _read_exact(f, 28)))


@dataclass
class RawTensor:
    """One tensor of the file: ggml type id, shape (outermost first) and its bytes."""
    ggml_dtype: int
    shape: tuple
    data: np.ndarray

    def to_qtensor(self, device):
        import torch

        from .quantized import GgmlDType, QTensor

        try:
            dtype = GgmlDType(self.ggml_dtype)
        except ValueError:
            raise CandleError(f"no device decoder for ggml type {GGML_TYPES[self.ggml_dtype][0]}") from None
        return QTensor.from_raw(torch.from_numpy(self.data), dtype, self.shape, device=device)


def _read_one_tensor(f, magic: str):
    n_dims, name_len, dtype = struct.unpack("<3I", _read_exact(f, 12))
    if dtype not in GGML_TYPES:
        raise CandleError(f"unknown dtype for tensor {dtype}")
    dims = list(struct.unpack("<%dI" % n_dims, _read_exact(f, 4 * n_dims)))
    dims.reverse()
    name = _read_exact(f, name_len).decode("utf-8", errors="replace")
    if align32(magic):
        pos = f.tell()
        f.seek((32 - pos % 32) % 32, 1)
    tname, block, nbytes = GGML_TYPES[dtype]
    elems = int(np.prod(dims, dtype=np.int64)) if dims else 1
    size_in_bytes = elems * nbytes // block
    raw = np.frombuffer(_read_exact(f, size_in_bytes), dtype=np.uint8).copy()
    if elems % block != 0:
        raise CandleError(f"Error creating tensor {name}: the number of elements {elems} is not divisible by the "
                          f"block size {block}")
    if dtype not in _LOADABLE:
        raise CandleError(f"Error creating tensor {name}: quantized type {tname} is not supported yet")
    return name, RawTensor(dtype, tuple(dims), raw)


@dataclass
class Content:
    magic: str
    hparams: HParams
    vocab: list = field(default_factory=list)    # [(token bytes, score)]
    tensors: dict = field(default_factory=dict)  # name -> RawTensor

    @classmethod
    def read(cls, f) -> "Content":
        last_position = f.seek(0, 2)
        f.seek(0)
        magic = read_magic(f)
        hparams = HParams.read(f)
        vocab = []
        for _ in range(hparams.n_vocab):
            word = _read_exact(f, _u32(f))
            vocab.append((word, struct.unpack("<f", _read_exact(f, 4))[0]))
        tensors = {}
        while f.tell() != last_position:
            name, tensor = _read_one_tensor(f, magic)
            tensors[name] = tensor
        return cls(magic, hparams, vocab, tensors)

    def remove(self, name: str) -> RawTensor:
        if name not in self.tensors:
            raise CandleError(f"cannot find tensor with name '{name}'")
        return self.tensors.pop(name)

    def tensor(self, name: str, device):
        """A block-quantised tensor as a GPU-resident ``QTensor`` (the file keeps it)."""
        if name not in self.tensors:
            raise CandleError(f"cannot find tensor with name '{name}'")
        return self.tensors[name].to_qtensor(device)


def write(f, magic: str, hparams: HParams, vocab, tensors) -> None:
    """The byte layout ``Content.read`` parses; ``tensors`` is an iterable of (name, ggml type id,
    shape outermost-first, bytes).  For fixtures: the reference only reads this format."""
    value, version = _MAGIC_VALUES[magic]
    f.write(struct.pack("<I", value))
    if version is not None:
        f.write(struct.pack("<I", version))
    f.write(struct.pack("<7I", hparams.n_vocab, hparams.n_embd, hparams.n_mult, hparams.n_head, hparams.n_layer,
                        hparams.n_rot, hparams.ftype))
    if len(vocab) != hparams.n_vocab:
        raise CandleError(f"{len(vocab)} tokens for n_vocab = {hparams.n_vocab}")
    for word, score in vocab:
        f.write(struct.pack("<I", len(word)))
        f.write(word)
        f.write(struct.pack("<f", score))
    for name, dtype, shape, data in tensors:
        encoded = name.encode("utf-8")
        f.write(struct.pack("<3I", len(shape), len(encoded), dtype))
        f.write(struct.pack("<%dI" % len(shape), *reversed(shape)))
        f.write(encoded)
        if align32(magic):
            f.write(b"\0" * ((32 - f.tell() % 32) % 32))
        f.write(bytes(data))
