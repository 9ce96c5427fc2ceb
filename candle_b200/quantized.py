"""The slice of ``candle_core::quantized`` the lookup path needs: a ``QTensor`` of 32-element
blocks (Q4_0, Q4_1, Q5_0, Q5_1, Q8_0) or 256-element K-quant super-blocks (Q2K .. Q8K) resident on the GPU (candle-core/src/quantized/mod.rs:35-38, quantized/cuda.rs:9-20) with
``dequantize`` / ``dequantize_f16`` (mod.rs:361-382) and a row lookup."""
from __future__ import annotations

import enum

import torch

from . import _cabi
from .errors import CandleError
from .ops import _DTYPES, _ID_DTYPES, _ids_checks, _ptr, _same_device, _stream, new_status, raise_for_status


class GgmlDType(enum.Enum):
    """ggml type ids (candle-core/src/quantized/mod.rs:152-171) with ``block_size`` / ``type_size`` as in
    ``GgmlDType::block_size`` / ``type_size`` (mod.rs:210-252)."""

    Q4_0 = _cabi.QTYPE_Q4_0
    Q4_1 = _cabi.QTYPE_Q4_1
    Q5_0 = _cabi.QTYPE_Q5_0
    Q5_1 = _cabi.QTYPE_Q5_1
    Q8_0 = _cabi.QTYPE_Q8_0
    Q2K = _cabi.QTYPE_Q2K
    Q3K = _cabi.QTYPE_Q3K
    Q4K = _cabi.QTYPE_Q4K
    Q5K = _cabi.QTYPE_Q5K
    Q6K = _cabi.QTYPE_Q6K
    Q8K = _cabi.QTYPE_Q8K

    @property
    def block_size(self) -> int:
        return 256 if self.value >= 10 else 32

    @property
    def type_size(self) -> int:
        return {2: 18, 3: 20, 6: 22, 7: 24, 8: 34, 10: 84, 11: 110, 12: 144, 13: 176, 14: 210, 15: 292}[self.value]


class QTensor:
    """Raw blocks + logical shape.  ``data`` is a contiguous uint8 CUDA tensor."""

    def __init__(self, data: torch.Tensor, dtype: GgmlDType, shape):
        shape = tuple(int(d) for d in shape)
        if not shape or shape[-1] % dtype.block_size != 0:
            # check_shape, candle-core/src/quantized/mod.rs:304-316
            raise CandleError(
                f"quantized tensor must have their last dim divisible by block size {list(shape)} {dtype.block_size}"
            )
        n = 1
        for d in shape:
            n *= d
        want = n // dtype.block_size * dtype.type_size
        if data.dtype != torch.uint8 or not data.is_contiguous() or data.numel() != want:
            raise CandleError(f"QTensor storage must be {want} contiguous bytes for shape {list(shape)}")
        if not data.is_cuda:
            raise CandleError("candle_b200 runs on Device::Cuda only: there is no CPU fallback")
        self.data, self.dtype, self.shape = data.reshape(-1), dtype, shape

    @classmethod
    def from_raw(cls, raw: torch.Tensor, dtype: GgmlDType, shape, device=None) -> "QTensor":
        """``qtensor_from_ggml`` for already-read bytes (candle-core/src/quantized/ggml_file.rs:120-188)."""
        data = raw.reshape(-1).to(device or raw.device).contiguous()
        return cls(data, dtype, shape)

    def elem_count(self) -> int:
        n = 1
        for d in self.shape:
            n *= d
        return n

    def dequantize(self, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        """``QTensor::dequantize`` (f32) or, for f16 / bf16, dequantize followed by ``to_dtype``."""
        if dtype not in _DTYPES:
            raise CandleError(f"unsupported dtype {dtype} for dequantize")
        out = torch.empty(self.shape, dtype=dtype, device=self.data.device)
        _cabi.call("cb200_dequantize", _ptr(self.data), self.dtype.value, _ptr(out), self.elem_count(),
                   _DTYPES[dtype], _stream(self.data))
        return out

    def dequantize_f16(self) -> torch.Tensor:
        return self.dequantize(torch.float16)

    def embedding(self, ids: torch.Tensor, dtype: torch.dtype = torch.float32, *, check: bool = True,
                  status: torch.Tensor | None = None, vocab_range: tuple[int, int] | None = None,
                  vocab: int | None = None) -> torch.Tensor:
        """Rows ``ids`` decoded to ``dtype``: ``dequantize().to_dtype(dtype).embedding(ids)`` without
        the decoded table.  With ``vocab_range=(begin, end)`` this tensor holds only that slice of
        a ``vocab``-row table and ids outside it give rows of zero bits (see cb200_qembedding)."""
        if len(self.shape) != 2:
            raise CandleError("embedding expects a rank-2 table")
        if dtype not in _DTYPES:
            raise CandleError(f"unsupported dtype {dtype} for embedding")
        flat = _ids_checks(ids.reshape(-1))
        _same_device(self.data, flat)
        local_vocab, hidden = self.shape
        begin, end = vocab_range if vocab_range is not None else (0, local_vocab)
        total = vocab if vocab is not None else end
        if end - begin != local_vocab:
            raise CandleError(f"vocab shard [{begin}, {end}) does not match the table's {local_vocab} rows")
        out = torch.empty(list(ids.shape) + [hidden], dtype=dtype, device=self.data.device)
        st = status if status is not None else (new_status(self.data.device) if check else None)
        _cabi.call("cb200_qembedding", _ptr(self.data), self.dtype.value, _ptr(flat), _ptr(out), total, hidden,
                   flat.shape[0], _DTYPES[dtype], _ID_DTYPES[flat.dtype], begin, end, _ptr(st), _stream(self.data))
        if check:
            raise_for_status(st)
        return out
