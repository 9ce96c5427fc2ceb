"""Module-level mirrors: ``candle_nn::{Embedding, LayerNorm, RmsNorm}`` (candle-nn/src/embedding.rs,
candle-nn/src/layer_norm.rs) and a quantised embedding in the style of
candle-transformers/src/quantized_nn.rs:12-36."""
from __future__ import annotations

import torch

from . import ops
from .errors import CandleError
from .quantized import QTensor


class Embedding:
    def __init__(self, embeddings: torch.Tensor, hidden_size: int):
        self._embeddings, self._hidden_size = embeddings, hidden_size

    def embeddings(self) -> torch.Tensor:
        return self._embeddings

    def hidden_size(self) -> int:
        return self._hidden_size

    def forward(self, indexes: torch.Tensor, *, check: bool = True) -> torch.Tensor:
        # candle-nn/src/embedding.rs:29-36
        final_dims = list(indexes.shape) + [self._hidden_size]
        values = ops.index_select(self._embeddings, indexes.reshape(-1), 0, check=check)
        return values.reshape(final_dims)

    __call__ = forward


class LayerNorm:
    """``LayerNorm::new`` / ``new_no_bias`` / ``rms_norm`` (candle-nn/src/layer_norm.rs:71-106)."""

    def __init__(self, weight: torch.Tensor, bias: torch.Tensor | None, eps: float, remove_mean: bool = True):
        self._weight, self._bias, self.eps, self.remove_mean = weight, bias, eps, remove_mean

    @classmethod
    def new(cls, weight, bias, eps):
        return cls(weight, bias, eps, True)

    @classmethod
    def new_no_bias(cls, weight, eps):
        return cls(weight, None, eps, True)

    @classmethod
    def rms_norm(cls, weight, eps):
        return cls(weight, None, eps, False)

    def weight(self):
        return self._weight

    def bias(self):
        return self._bias

    def forward(self, x: torch.Tensor, *, residual: torch.Tensor | None = None) -> torch.Tensor:
        # candle-nn/src/layer_norm.rs:108-136: the fused op iff the input is contiguous, the mean is
        # removed and there is a bias; otherwise the composite chain (f32 inside, one rounding, weight
        # and bias applied in the tensor's dtype), which rounds differently for f16 / bf16.
        if x.is_contiguous() and self.remove_mean and self._bias is not None:
            return ops.layer_norm(x, self._weight, self._bias, self.eps, residual=residual)
        if residual is not None:
            raise CandleError("a fused residual is only available on the fused norm paths")
        return ops._norm_slow(x, self._weight, self._bias, self.eps, self.remove_mean)

    __call__ = forward


class RmsNorm:
    """``RmsNorm::new(weight, eps)`` (candle-nn/src/layer_norm.rs:138-194)."""

    def __init__(self, weight: torch.Tensor, eps: float):
        self._inner = LayerNorm.rms_norm(weight, eps)

    def into_inner(self) -> LayerNorm:
        return self._inner

    def forward_diff(self, xs: torch.Tensor) -> torch.Tensor:
        # layer_norm.rs:176-178: always the inner LayerNorm, i.e. the composite chain
        return self._inner.forward(xs)

    def forward(self, xs: torch.Tensor, *, residual: torch.Tensor | None = None) -> torch.Tensor:
        # layer_norm.rs:186-194: only this entry point uses the fused rms-norm op
        if xs.is_contiguous():
            return ops.rms_norm(xs, self._inner.weight(), self._inner.eps, residual=residual)
        return self._inner.forward(xs, residual=residual)

    __call__ = forward


class QEmbedding:
    """Embedding whose table stays quantised on the device; rows are decoded per lookup.

    candle dequantises the whole table at load instead
    (candle-transformers/src/models/quantized_llama.rs:378-379); the values are the same."""

    def __init__(self, table: QTensor, dtype: torch.dtype = torch.float32):
        if len(table.shape) != 2:
            raise CandleError("QEmbedding expects a rank-2 QTensor")
        self._table, self._dtype = table, dtype

    def hidden_size(self) -> int:
        return self._table.shape[1]

    def forward(self, indexes: torch.Tensor, *, check: bool = True) -> torch.Tensor:
        return self._table.embedding(indexes, self._dtype, check=check)

    __call__ = forward
