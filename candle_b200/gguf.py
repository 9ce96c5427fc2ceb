"""Reader and writer for GGUF files, the container the quantised tables of this path come in.

Mirrors ``candle_core::quantized::gguf_file`` (candle-core/src/quantized/gguf_file.rs): versions 1
to 3 are read (v1 has 32-bit counts and lengths, :34-46, 92-98, 394-407), version 2 is written
(:496-546), tensor data starts at the next multiple of ``general.alignment`` (default 32, :448-460),
dimensions are stored innermost-first and reversed on read (:410-427).  Metadata values keep their
GGUF type so that a file can be written back unchanged.  Tensor payloads stay raw bytes on the
host; ``TensorInfo.to_qtensor`` moves a block-quantised one to the GPU for the lookups.
"""
from __future__ import annotations

import struct
from dataclasses import dataclass

import numpy as np

from .errors import CandleError

DEFAULT_ALIGNMENT = 32
_MAGICS = (0x46554747, 0x47475546)

# ggml type id -> (name, elements per block, bytes per block); candle-core/src/quantized/mod.rs:152-256
GGML_TYPES = {
    0: ("F32", 1, 4), 1: ("F16", 1, 2), 2: ("Q4_0", 32, 18), 3: ("Q4_1", 32, 20), 6: ("Q5_0", 32, 22),
    7: ("Q5_1", 32, 24), 8: ("Q8_0", 32, 34), 9: ("Q8_1", 32, 36), 10: ("Q2K", 256, 84), 11: ("Q3K", 256, 110),
    12: ("Q4K", 256, 144), 13: ("Q5K", 256, 176), 14: ("Q6K", 256, 210), 15: ("Q8K", 256, 292),
}

# GGUF value types, gguf_file.rs:331-370
_SCALARS = {0: ("U8", "<B"), 1: ("I8", "<b"), 2: ("U16", "<H"), 3: ("I16", "<h"), 4: ("U32", "<I"), 5: ("I32", "<i"),
            6: ("F32", "<f"), 10: ("U64", "<Q"), 11: ("I64", "<q"), 12: ("F64", "<d")}
_T_BOOL, _T_STRING, _T_ARRAY = 7, 8, 9
_TYPE_IDS = {name: tid for tid, (name, _) in _SCALARS.items()} | {"Bool": _T_BOOL, "String": _T_STRING, "Array": _T_ARRAY}


@dataclass
class Value:
    """A metadata value with its GGUF type name (``U8`` .. ``F64``, ``Bool``, ``String``, ``Array``);
    an array holds ``Value`` items of one type."""

    type: str
    value: object

    def to_u64(self) -> int:
        # gguf_file.rs:214-223: unsigned types and bool widen to u64
        if self.type in ("U64", "U8", "U16", "U32", "Bool"):
            return int(self.value)
        raise CandleError(f"not a u64 or upcastable to u64 {self}")


def _read_exact(f, n: int) -> bytes:
    b = f.read(n)
    if len(b) != n:
        raise CandleError("failed to fill whole buffer")  # std::io::Read::read_exact's message
    return b


def _read_len(f, version: int) -> int:
    return struct.unpack("<I", _read_exact(f, 4))[0] if version == 1 else struct.unpack("<Q", _read_exact(f, 8))[0]


def _read_string(f, version: int) -> str:
    raw = _read_exact(f, _read_len(f, version))
    return raw.rstrip(b"\0").decode("utf-8", errors="replace")  # :100-108: stray NULs dropped, lossy utf-8


def _read_value(f, tid: int, version: int) -> Value:
    if tid in _SCALARS:
        name, fmt = _SCALARS[tid]
        return Value(name, struct.unpack(fmt, _read_exact(f, struct.calcsize(fmt)))[0])
    if tid == _T_BOOL:
        b = _read_exact(f, 1)[0]
        if b > 1:
            raise CandleError(f"unexpected bool value {b}")
        return Value("Bool", bool(b))
    if tid == _T_STRING:
        return Value("String", _read_string(f, version))
    if tid == _T_ARRAY:
        item = struct.unpack("<I", _read_exact(f, 4))[0]
        n = _read_len(f, version)
        return Value("Array", [_read_value(f, item, version) for _ in range(n)])
    raise CandleError(f"unrecognized value-type {tid:#08x}")


@dataclass
class TensorInfo:
    ggml_dtype: int
    shape: tuple
    offset: int

    @property
    def size_in_bytes(self) -> int:
        _, block, nbytes = GGML_TYPES[self.ggml_dtype]
        elems = int(np.prod(self.shape, dtype=np.int64)) if self.shape else 1
        if elems % block != 0:
            raise CandleError(f"the number of elements {elems} is not divisible by the block size {block}")
        return elems // block * nbytes

    def read_raw(self, f, tensor_data_offset: int) -> np.ndarray:
        """The tensor's bytes as they are in the file (gguf_file.rs:57-81)."""
        f.seek(tensor_data_offset + self.offset)
        return np.frombuffer(_read_exact(f, self.size_in_bytes), dtype=np.uint8).copy()

    def to_qtensor(self, f, tensor_data_offset: int, device):
        """A block-quantised tensor as a GPU-resident ``QTensor`` for ``cb200_qembedding`` and friends."""
        import torch

        from .quantized import GgmlDType, QTensor

        try:
            dtype = GgmlDType(self.ggml_dtype)
        except ValueError:
            raise CandleError(f"no device decoder for ggml type {GGML_TYPES[self.ggml_dtype][0]}") from None
        return QTensor.from_raw(torch.from_numpy(self.read_raw(f, tensor_data_offset)), dtype, self.shape, device=device)


@dataclass
class Content:
    version: int
    metadata: dict
    tensor_infos: dict
    tensor_data_offset: int

    @classmethod
    def read(cls, f) -> "Content":
        magic, version = struct.unpack("<II", _read_exact(f, 8))
        if magic not in _MAGICS:
            raise CandleError(f"unknown magic 0x{magic:08x}")
        if version not in (1, 2, 3):
            raise CandleError(f"gguf: unsupported magic/version Gguf/{version}")
        tensor_count = _read_len(f, version)
        kv_count = _read_len(f, version)
        metadata = {}
        for _ in range(kv_count):
            key = _read_string(f, version)
            tid = struct.unpack("<I", _read_exact(f, 4))[0]
            metadata[key] = _read_value(f, tid, version)
        infos = {}
        for _ in range(tensor_count):
            name = _read_string(f, version)
            n_dims = struct.unpack("<I", _read_exact(f, 4))[0]
            fmt = "<%dI" % n_dims if version == 1 else "<%dQ" % n_dims
            dims = list(struct.unpack(fmt, _read_exact(f, struct.calcsize(fmt))))
            dims.reverse()
            dtype, offset = struct.unpack("<IQ", _read_exact(f, 12))
            if dtype not in GGML_TYPES:
                raise CandleError(f"unknown dtype for tensor {dtype}")
            infos[name] = TensorInfo(dtype, tuple(dims), offset)
        position = f.tell()
        alignment = DEFAULT_ALIGNMENT
        a = metadata.get("general.alignment")
        if a is not None and a.type in ("U8", "U16", "U32", "I8", "I16", "I32") and a.value >= 0:
            alignment = int(a.value)
        if alignment <= 0:
            raise CandleError("general.alignment must be positive")
        return cls(version, metadata, infos, -(-position // alignment) * alignment)

    def tensor_info(self, name: str) -> TensorInfo:
        if name not in self.tensor_infos:
            raise CandleError(f"cannot find tensor info for {name}")
        return self.tensor_infos[name]

    def tensor_raw(self, f, name: str) -> np.ndarray:
        return self.tensor_info(name).read_raw(f, self.tensor_data_offset)

    def tensor(self, f, name: str, device):
        return self.tensor_info(name).to_qtensor(f, self.tensor_data_offset, device)


def _write_string(f, s: str) -> None:
    b = s.encode("utf-8")
    f.write(struct.pack("<Q", len(b)) + b)


def _write_value(f, v: Value) -> None:
    if v.type in _TYPE_IDS and _TYPE_IDS[v.type] in _SCALARS:
        f.write(struct.pack(_SCALARS[_TYPE_IDS[v.type]][1], v.value))
    elif v.type == "Bool":
        f.write(struct.pack("<B", 1 if v.value else 0))
    elif v.type == "String":
        _write_string(f, v.value)
    elif v.type == "Array":
        kinds = {item.type for item in v.value}
        if len(kinds) > 1:
            raise CandleError(f"multiple value-types in the same array {sorted(kinds)}")
        item_type = kinds.pop() if kinds else "U32"  # an empty array is written as U32, :311-313
        f.write(struct.pack("<IQ", _TYPE_IDS[item_type], len(v.value)))
        for item in v.value:
            _write_value(f, item)
    else:
        raise CandleError(f"unknown value type {v.type}")


def write(f, metadata, tensors) -> None:
    """``gguf_file::write`` (:496-546): version 2, every tensor padded to 32 bytes.  ``metadata`` is a
    list of ``(key, Value)``; ``tensors`` a list of ``(name, ggml type id, shape, raw bytes)``."""
    f.write(struct.pack("<IIQQ", 0x46554747, 2, len(tensors), len(metadata)))
    for key, value in metadata:
        _write_string(f, key)
        f.write(struct.pack("<I", _TYPE_IDS[value.type]))
        _write_value(f, value)
    offset, offsets = 0, []
    for name, dtype, shape, raw in tensors:
        raw = np.ascontiguousarray(raw).reshape(-1).view(np.uint8)
        if TensorInfo(dtype, tuple(shape), 0).size_in_bytes != raw.size:
            raise CandleError(f"tensor {name}: {raw.size} bytes do not match shape {list(shape)} of {GGML_TYPES[dtype][0]}")
        _write_string(f, name)
        f.write(struct.pack("<I", len(shape)))
        for dim in reversed(shape):
            f.write(struct.pack("<Q", dim))
        f.write(struct.pack("<IQ", dtype, offset))
        offsets.append(offset)
        offset += raw.size + (31 - (31 + raw.size) % 32)
    pos = f.tell()
    f.write(b"\0" * (31 - (31 + pos) % 32))
    start = f.tell()
    for off, (name, dtype, shape, raw) in zip(offsets, tensors):
        if start + off != f.tell():
            raise CandleError(f"internal error, unexpected current position {start} {off} {f.tell()}")
        raw = np.ascontiguousarray(raw).reshape(-1).view(np.uint8)
        f.write(raw.tobytes())
        f.write(b"\0" * (31 - (31 + raw.size) % 32))
