"""ctypes front end of the CPU oracle (``candle_cpu_oracle.c``).

TEST INFRASTRUCTURE ONLY.  Nothing in the ``candle_b200`` package imports this module; it may be
used by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of ``bench.py``.

Arrays are numpy arrays.  f16 / bf16 data travels as ``uint16`` bit patterns (numpy has no
bfloat16); ``dtype`` arguments are the strings ``"f32"``, ``"f16"``, ``"bf16"``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libcandle_cpu_oracle.so")

DTYPES = {"f32": 0, "f16": 1, "bf16": 2}
ID_DTYPES = {np.dtype(np.uint8): 0, np.dtype(np.uint32): 1, np.dtype(np.int64): 2}
QTYPES = {"q4_0": 2, "q4_1": 3, "q5_0": 6, "q5_1": 7, "q8_0": 8,
          "q2k": 10, "q3k": 11, "q4k": 12, "q5k": 13, "q6k": 14, "q8k": 15}  # ggml type ids
BLOCK_BYTES = {"q4_0": 18, "q4_1": 20, "q5_0": 22, "q5_1": 24, "q8_0": 34,
               "q2k": 84, "q3k": 110, "q4k": 144, "q5k": 176, "q6k": 210, "q8k": 292}
QK = 32
QK_K = 256


def block_elems(qtype: str) -> int:
    """Elements per block: 256 for the K-quant super-blocks, 32 otherwise."""
    return QK_K if qtype.endswith("k") else QK


class InvalidIndex(IndexError):
    """Mirror of candle's ``Error::InvalidIndex { index, size, op }``."""

    def __init__(self, index: int, size: int, op: str = "index-select"):
        super().__init__(f"invalid index {index} with dim size {size} in {op}")
        self.index, self.size, self.op = index, size, op


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile; returns the path of the shared library."""
    srcs = [os.path.join(_HERE, f) for f in ("candle_cpu_oracle.c", "candle_cpu_kquants.h", "Makefile")]
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(f) for f in srcs):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        i64, vp, f32, ci = ctypes.c_int64, ctypes.c_void_p, ctypes.c_float, ctypes.c_int
        L.oracle_rms_norm.argtypes = [ci, vp, vp, vp, i64, i64, f32, ci]
        L.oracle_layer_norm.argtypes = [ci, vp, vp, vp, vp, i64, i64, f32, ci]
        L.oracle_add.argtypes = [ci, vp, vp, vp, i64, ci]
        L.oracle_cast_from_f32.argtypes = [ci, vp, vp, i64, ci]
        L.oracle_cast_to_f32.argtypes = [ci, vp, vp, i64, ci]
        L.oracle_index_select.argtypes = [i64, ci, vp, vp, i64, vp, i64, i64, i64, i64, ctypes.POINTER(i64)]
        L.oracle_dequantize.argtypes = [ci, vp, vp, i64, ci]
        L.oracle_quantize.argtypes = [ci, vp, vp, i64]
        L.oracle_qembedding.argtypes = [ci, ci, ci, vp, vp, vp, i64, i64, i64, ctypes.POINTER(i64), ci]
        L.oracle_norm_slow.argtypes = [ci, vp, vp, vp, vp, i64, i64, ctypes.c_double, ci, ci]
        L.oracle_avx_vec_sum.argtypes = [vp, i64]
        L.oracle_avx_vec_sum.restype = f32
        L.oracle_softmax_last_dim.argtypes = [ci, vp, vp, i64, i64, ci]
        L.oracle_rope.argtypes = [ci, ci, vp, vp, vp, vp, i64, i64, i64, i64, ci]
        L.oracle_max_threads.restype = ci
        L.oracle_bf16_from_f32.argtypes = [f32]
        L.oracle_bf16_from_f32.restype = ctypes.c_uint16
        L.oracle_f16_from_f32.argtypes = [f32]
        L.oracle_f16_from_f32.restype = ctypes.c_uint16
        L.oracle_bf16_to_f32.argtypes = [ctypes.c_uint16]
        L.oracle_bf16_to_f32.restype = f32
        L.oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
        L.oracle_f16_to_f32.restype = f32
        _lib = L
    return _lib


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def _np_dtype(dtype: str):
    return np.float32 if dtype == "f32" else np.uint16


def _check(arr: np.ndarray, dtype: str, name: str) -> np.ndarray:
    want = _np_dtype(dtype)
    if arr.dtype != want:
        raise TypeError(f"{name}: expected {want} storage for {dtype}, got {arr.dtype}")
    return np.ascontiguousarray(arr)


def _ptr(a: np.ndarray) -> ctypes.c_void_p:
    return ctypes.c_void_p(a.ctypes.data)


def _rc(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"oracle {what} failed with code {rc}")


def cast_from_f32(x: np.ndarray, dtype: str, threads: int = 0) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    y = np.empty(x.shape, dtype=_np_dtype(dtype))
    _rc(lib().oracle_cast_from_f32(DTYPES[dtype], _ptr(x), _ptr(y), x.size, threads), "cast_from_f32")
    return y


def cast_to_f32(x: np.ndarray, dtype: str, threads: int = 0) -> np.ndarray:
    x = _check(x, dtype, "x")
    y = np.empty(x.shape, dtype=np.float32)
    _rc(lib().oracle_cast_to_f32(DTYPES[dtype], _ptr(x), _ptr(y), x.size, threads), "cast_to_f32")
    return y


def add(a: np.ndarray, b: np.ndarray, dtype: str, threads: int = 1) -> np.ndarray:
    """``a + b`` rounded to ``dtype`` (candle's sequential binary map; ``threads=1`` mirrors it)."""
    a, b = _check(a, dtype, "a"), _check(b, dtype, "b")
    if a.shape != b.shape:
        raise ValueError("shape mismatch in add")
    out = np.empty_like(a)
    _rc(lib().oracle_add(DTYPES[dtype], _ptr(a), _ptr(b), _ptr(out), a.size, threads), "add")
    return out


def rms_norm(x: np.ndarray, alpha: np.ndarray, eps: float, dtype: str, threads: int = 0) -> np.ndarray:
    x, alpha = _check(x, dtype, "x"), _check(alpha, dtype, "alpha")
    cols = x.shape[-1]
    if alpha.shape != (cols,):
        raise ValueError(f"shape mismatch in rms-norm {x.shape} {alpha.shape}")
    rows = x.size // cols if cols else 0
    y = np.empty_like(x)
    _rc(lib().oracle_rms_norm(DTYPES[dtype], _ptr(x), _ptr(alpha), _ptr(y), rows, cols, eps, threads), "rms_norm")
    return y


def layer_norm(x: np.ndarray, gamma: np.ndarray, beta: np.ndarray, eps: float, dtype: str, threads: int = 0) -> np.ndarray:
    x, gamma, beta = _check(x, dtype, "x"), _check(gamma, dtype, "gamma"), _check(beta, dtype, "beta")
    cols = x.shape[-1]
    if gamma.shape != (cols,) or beta.shape != (cols,):
        raise ValueError(f"shape mismatch in layer-norm src: {x.shape} alpha: {gamma.shape} beta: {beta.shape}")
    rows = x.size // cols if cols else 0
    y = np.empty_like(x)
    _rc(
        lib().oracle_layer_norm(DTYPES[dtype], _ptr(x), _ptr(gamma), _ptr(beta), _ptr(y), rows, cols, eps, threads),
        "layer_norm",
    )
    return y


def norm_slow(x: np.ndarray, weight: np.ndarray, bias: np.ndarray | None, eps: float, dtype: str,
              remove_mean: bool = True, threads: int = 0) -> np.ndarray:
    """candle's composite norm (``LayerNorm::forward`` off the fused path, ``ops::rms_norm_slow`` /
    ``layer_norm_slow``): f32 internally, AVX-ordered row sums, one rounding to ``dtype``, then the
    weight (and bias) applied in ``dtype``."""
    x, weight = _check(x, dtype, "x"), _check(weight, dtype, "weight")
    cols = x.shape[-1]
    if bias is not None:
        bias = _check(bias, dtype, "bias")
    if weight.shape != (cols,) or (bias is not None and bias.shape != (cols,)):
        raise ValueError("shape mismatch in the composite norm")
    rows = x.size // cols if cols else 0
    y = np.empty_like(x)
    _rc(lib().oracle_norm_slow(DTYPES[dtype], _ptr(x), _ptr(weight), _ptr(bias) if bias is not None else None,
                               _ptr(y), rows, cols, float(eps), 1 if remove_mean else 0, threads), "norm_slow")
    return y


def avx_vec_sum(row: np.ndarray) -> float:
    """candle's ``vec_sum`` in its AVX order over one f32 row."""
    row = np.ascontiguousarray(row, dtype=np.float32)
    return float(lib().oracle_avx_vec_sum(_ptr(row), row.size))


def softmax_last_dim(x: np.ndarray, dtype: str, threads: int = 0) -> np.ndarray:
    """``candle_nn::ops::softmax_last_dim`` (candle-nn/src/ops.rs:289-435, CPU path)."""
    x = _check(x, dtype, "x")
    cols = x.shape[-1]
    rows = x.size // cols if cols else 0
    y = np.empty_like(x)
    _rc(lib().oracle_softmax_last_dim(DTYPES[dtype], _ptr(x), _ptr(y), rows, cols, threads), "softmax_last_dim")
    return y


ROPE_VARIANTS = {"rope_i": 0, "rope": 1, "rope_thd": 2}


def rope(variant: str, x: np.ndarray, cos: np.ndarray, sin: np.ndarray, dtype: str, threads: int = 0) -> np.ndarray:
    """``candle_nn::rotary_emb::{rope_i, rope, rope_thd}`` (CPU paths).  ``x`` is ``[b, h, t, d]``
    (``[b, t, h, d]`` for ``rope_thd``), ``cos`` / ``sin`` are ``[>= t, d / 2]``."""
    x, cos, sin = _check(x, dtype, "x"), _check(cos, dtype, "cos"), _check(sin, dtype, "sin")
    if x.ndim != 4:
        raise ValueError("rope expects a rank-4 tensor")
    if variant == "rope_thd":
        b, t, h, d = x.shape
    else:
        b, h, t, d = x.shape
    if cos.shape != sin.shape or cos.ndim != 2 or cos.shape[1] * 2 != d or cos.shape[0] < t:
        raise ValueError(f"inconsistent last dim size in rope {x.shape} {cos.shape} {sin.shape}")
    y = np.empty_like(x)
    _rc(lib().oracle_rope(ROPE_VARIANTS[variant], DTYPES[dtype], _ptr(x), _ptr(cos), _ptr(sin), _ptr(y), b, h, t, d,
                          threads), "rope")
    return y


def index_select(src: np.ndarray, ids: np.ndarray, dim: int = 0) -> np.ndarray:
    """``Tensor::index_select``: ids must be rank 1 (u8 / u32 / i64), may be a strided view."""
    src = np.ascontiguousarray(src)
    if ids.ndim != 1:
        raise ValueError(f"unexpected number of dims: expected 1, got {ids.ndim}")
    if ids.dtype not in ID_DTYPES:
        raise TypeError(f"unsupported ids dtype {ids.dtype}")
    stride = ids.strides[0] // ids.itemsize if ids.size else 1
    shape = list(src.shape)
    src_dim = shape[dim]
    left = int(np.prod(shape[:dim], dtype=np.int64))
    right = int(np.prod(shape[dim + 1 :], dtype=np.int64))
    shape[dim] = ids.shape[0]
    dst = np.zeros(shape, dtype=src.dtype)
    bad = ctypes.c_int64(0)
    rc = lib().oracle_index_select(
        src.itemsize, ID_DTYPES[ids.dtype], _ptr(src), ctypes.c_void_p(ids.ctypes.data), stride, _ptr(dst),
        left, src_dim, right, ids.shape[0], ctypes.byref(bad),
    )
    if rc == -2:
        raise InvalidIndex(bad.value & (2**64 - 1), src_dim)
    _rc(rc, "index_select")
    return dst


def embedding(table: np.ndarray, ids: np.ndarray) -> np.ndarray:
    """``Embedding::forward``: flatten ids, index_select on dim 0, reshape to ids.shape + [hidden]."""
    flat = np.ascontiguousarray(ids).reshape(-1)
    return index_select(table, flat, 0).reshape(tuple(ids.shape) + (table.shape[1],))


def quantize(x: np.ndarray, qtype: str) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    be = block_elems(qtype)
    if x.shape[-1] % be:
        raise ValueError(f"last dim {x.shape[-1]} is not divisible by {be}")
    nb = x.size // be
    out = np.zeros(nb * BLOCK_BYTES[qtype], dtype=np.uint8)
    _rc(lib().oracle_quantize(QTYPES[qtype], _ptr(x), _ptr(out), x.size), "quantize")
    return out.reshape(x.shape[:-1] + (x.shape[-1] // be * BLOCK_BYTES[qtype],))


def dequantize(blocks: np.ndarray, qtype: str, threads: int = 1) -> np.ndarray:
    """Raw block bytes ``[..., n_blocks * block_bytes]`` -> f32 ``[..., n_blocks * 32]``."""
    blocks = np.ascontiguousarray(blocks, dtype=np.uint8)
    bb, be = BLOCK_BYTES[qtype], block_elems(qtype)
    if blocks.shape[-1] % bb:
        raise ValueError("byte length is not a whole number of blocks")
    k = blocks.size // bb * be
    y = np.empty(blocks.shape[:-1] + (blocks.shape[-1] // bb * be,), dtype=np.float32)
    _rc(lib().oracle_dequantize(QTYPES[qtype], _ptr(blocks), _ptr(y), k, threads), "dequantize")
    return y


def qembedding(qtable: np.ndarray, qtype: str, ids: np.ndarray, out_dtype: str, threads: int = 0) -> np.ndarray:
    """Rows ``ids`` of a quantised ``[vocab, hidden/32*block_bytes]`` byte table, decoded to ``out_dtype``."""
    qtable = np.ascontiguousarray(qtable, dtype=np.uint8)
    vocab = qtable.shape[0]
    hidden = qtable.shape[1] // BLOCK_BYTES[qtype] * block_elems(qtype)
    flat = np.ascontiguousarray(ids).reshape(-1)
    out = np.empty((flat.size, hidden), dtype=_np_dtype(out_dtype))
    bad = ctypes.c_int64(0)
    rc = lib().oracle_qembedding(
        QTYPES[qtype], DTYPES[out_dtype], ID_DTYPES[flat.dtype], _ptr(qtable), _ptr(flat), _ptr(out),
        vocab, hidden, flat.size, ctypes.byref(bad), threads,
    )
    if rc == -2:
        raise InvalidIndex(bad.value & (2**64 - 1), vocab)
    _rc(rc, "qembedding")
    return out.reshape(tuple(ids.shape) + (hidden,))
