"""candle_b200: candle's normalisation + embedding path on B200 (sm_100a).

The package is the Python-side mirror of the candle front ends for this path
(``candle_nn::ops::{rms_norm, layer_norm}``, ``candle_nn::{LayerNorm, RmsNorm, Embedding}``,
``Tensor::index_select``, ``QTensor::dequantize``) on top of the C ABI in ``include/candle_b200.h``.
torch supplies device memory and streams only; every result is computed by the CUDA kernels in
``csrc/``.  Importing the package needs the built library -- there is no CPU fallback.
"""
from . import _cabi  # noqa: F401  (fails loudly when the extension is missing)
from .errors import CandleError, InvalidIndex
from .ops import (
    FLAG_FAST_SUM,
    FLAG_FORCE_GENERIC,
    FLAG_FORCE_LANEROW,
    FLAG_FORCE_REPLAY,
    embedding_rms_norm,
    index_select,
    layer_norm,
    layer_norm_slow,
    qembedding_rms_norm,
    rms_norm,
    rms_norm_rows,
    rms_norm_slow,
    rope,
    rope_i,
    rope_thd,
    softmax_last_dim,
)
from .host_pipeline import PinnedNormPipeline
from .nn import Embedding, LayerNorm, QEmbedding, RmsNorm
from .quantized import GgmlDType, QTensor

__all__ = [
    "CandleError", "InvalidIndex", "rms_norm", "layer_norm", "rms_norm_slow", "layer_norm_slow", "rms_norm_rows", "softmax_last_dim", "rope", "rope_i", "rope_thd", "index_select", "embedding_rms_norm",
    "qembedding_rms_norm", "PinnedNormPipeline", "Embedding", "LayerNorm", "RmsNorm", "QEmbedding", "QTensor", "GgmlDType",
    "FLAG_FAST_SUM", "FLAG_FORCE_LANEROW", "FLAG_FORCE_GENERIC", "FLAG_FORCE_REPLAY",
]
