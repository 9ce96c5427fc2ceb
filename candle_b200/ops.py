"""Front ends with the names, argument meaning and error behaviour of candle's own.

``rms_norm`` / ``layer_norm`` mirror ``candle_nn::ops::{rms_norm, layer_norm}``
(candle-nn/src/ops.rs:641-652, 896-909) plus the checks their ``cuda_fwd`` performs
(:536-543, 770-781); ``index_select`` mirrors ``Tensor::index_select``
(candle-core/src/tensor.rs:1568-1589).  The optional ``residual`` argument fuses the
``(x + residual)?`` the models compute just before the norm
(candle-transformers/src/models/llama.rs:446-450, bert.rs:301).
"""
from __future__ import annotations

import torch

from . import _cabi
from ._cabi import FLAG_FAST_SUM, FLAG_FORCE_GENERIC, FLAG_FORCE_LANEROW, FLAG_FORCE_REPLAY  # noqa: F401
from .errors import CandleError, InvalidIndex

_DTYPES = {torch.float32: _cabi.DTYPE_F32, torch.float16: _cabi.DTYPE_F16, torch.bfloat16: _cabi.DTYPE_BF16}
_DTYPE_NAMES = {torch.float32: "F32", torch.float16: "F16", torch.bfloat16: "BF16"}
_ID_DTYPES = {
    torch.uint8: _cabi.ID_U8,
    torch.uint32: _cabi.ID_U32,
    torch.int32: _cabi.ID_U32,  # the bit pattern is read as u32: negative values fail the bounds check
    torch.int64: _cabi.ID_I64,
}


def _dims(t: torch.Tensor) -> str:
    return str(list(t.shape))


def _ptr(t: torch.Tensor | None):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor):
    return torch.cuda.current_stream(t.device).cuda_stream


def _same_device(*ts: torch.Tensor) -> None:
    first = ts[0]
    if not first.is_cuda:
        raise CandleError("candle_b200 runs on Device::Cuda only: there is no CPU fallback")
    for t in ts[1:]:
        if t is not None and t.device != first.device:
            raise CandleError(f"device mismatch in op, lhs: {first.device}, rhs: {t.device}")


def new_status(device) -> torch.Tensor:
    """A zeroed ``cb200_status`` record (4 x int64 = 32 bytes) in device memory."""
    return torch.zeros(4, dtype=torch.int64, device=device)


def raise_for_status(status: torch.Tensor, op: str = "index-select") -> None:
    """Synchronises on the status record and raises what candle's CPU backend would have raised."""
    code_word, position, index, size = status.cpu().tolist()
    code = code_word & 0xFFFFFFFF
    if code == _cabi.STATUS_INVALID_INDEX:
        raise InvalidIndex(index & (2**64 - 1), size, op, position)
    if code == _cabi.STATUS_WAIT_TIMEOUT:
        raise CandleError(f"device-side wait timed out at row {position} in {op}")


def _norm_checks(name: str, xs: torch.Tensor, params: list[tuple[str, torch.Tensor]], residual):
    if xs.dtype not in _DTYPES or any(p.dtype != xs.dtype for _, p in params):
        raise CandleError(f"unsupported dtype for rmsnorm {_DTYPE_NAMES.get(xs.dtype, xs.dtype)}")
    if not xs.is_contiguous():
        raise CandleError("input has to be contiguous")
    for pname, p in params:
        if not p.is_contiguous():
            raise CandleError(f"{pname} has to be contiguous")
    if residual is not None:
        if residual.shape != xs.shape or residual.dtype != xs.dtype:
            raise CandleError(f"shape mismatch in binary op add, lhs: {_dims(xs)}, rhs: {_dims(residual)}")
        if not residual.is_contiguous():
            raise CandleError("input has to be contiguous")
    _same_device(xs, *[p for _, p in params], residual)


def _out_check(out: torch.Tensor | None, xs: torch.Tensor) -> torch.Tensor:
    if out is None:
        return torch.empty_like(xs)
    if out.shape != xs.shape or out.dtype != xs.dtype or out.device != xs.device or not out.is_contiguous():
        raise CandleError(f"out must be a contiguous tensor like the input, got {_dims(out)} for {_dims(xs)}")
    return out


def rms_norm(xs: torch.Tensor, alpha: torch.Tensor, eps: float, *, residual: torch.Tensor | None = None,
             return_sum: bool = False, flags: int = 0, out: torch.Tensor | None = None,
             status: torch.Tensor | None = None):
    """``candle_nn::ops::rms_norm(xs, alpha, eps)``; with ``residual`` the norm of ``xs + residual``.

    Returns ``y`` (``out`` when given), or ``(y, xs + residual)`` when ``return_sum`` is set.  A
    ``status`` record (``new_status``) receives device-side problems (a bounded wait that ran out).
    """
    if xs.dim() == 0:
        raise CandleError("unexpected rank, expected: at least 1, got: 0")
    if alpha.dim() != 1:
        raise CandleError(f"unexpected rank, expected: 1, got: {alpha.dim()} ({_dims(alpha)})")
    if xs.shape[-1] != alpha.shape[0]:
        raise CandleError(f"shape mismatch in rms-norm {_dims(xs)} {_dims(alpha)}")
    _norm_checks("rms-norm", xs, [("alpha", alpha)], residual)
    cols = xs.shape[-1]
    rows = xs.numel() // cols if cols else 0
    y = _out_check(out, xs)
    h = torch.empty_like(xs) if return_sum else None
    _cabi.call("cb200_rms_norm_checked", _ptr(xs), _ptr(residual), _ptr(alpha), _ptr(y), _ptr(h), rows, cols,
               float(eps), _DTYPES[xs.dtype], flags, _ptr(status), _stream(xs))
    return (y, h) if return_sum else y


def layer_norm(xs: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor, eps: float, *,
               residual: torch.Tensor | None = None, return_sum: bool = False, flags: int = 0,
               out: torch.Tensor | None = None, status: torch.Tensor | None = None):
    """``candle_nn::ops::layer_norm(xs, alpha, beta, eps)``; with ``residual`` the norm of ``xs + residual``."""
    if xs.dim() == 0:
        raise CandleError("unexpected rank, expected: at least 1, got: 0")
    if alpha.dim() != 1 or beta.dim() != 1:
        bad = alpha if alpha.dim() != 1 else beta
        raise CandleError(f"unexpected rank, expected: 1, got: {bad.dim()} ({_dims(bad)})")
    if xs.shape[-1] != alpha.shape[0] or xs.shape[-1] != beta.shape[0]:
        raise CandleError(f"shape mismatch in layer-norm src: {_dims(xs)} alpha: {_dims(alpha)} beta: {_dims(beta)}")
    _norm_checks("layer-norm", xs, [("alpha", alpha), ("beta", beta)], residual)
    cols = xs.shape[-1]
    rows = xs.numel() // cols if cols else 0
    y = _out_check(out, xs)
    h = torch.empty_like(xs) if return_sum else None
    _cabi.call("cb200_layer_norm_checked", _ptr(xs), _ptr(residual), _ptr(alpha), _ptr(beta), _ptr(y), _ptr(h), rows,
               cols, float(eps), _DTYPES[xs.dtype], flags, _ptr(status), _stream(xs))
    return (y, h) if return_sum else y


def _norm_slow(xs: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, eps: float, remove_mean: bool):
    """candle's composite norm chain (candle-nn/src/layer_norm.rs:115-135) in one launch."""
    if xs.dim() == 0:
        raise CandleError("unexpected rank, expected: at least 1, got: 0")
    if xs.dtype not in _DTYPES:
        raise CandleError(f"unsupported dtype for rmsnorm {_DTYPE_NAMES.get(xs.dtype, xs.dtype)}")
    cols = xs.shape[-1]
    for p in (weight, bias):
        if p is None:
            continue
        if p.dtype != xs.dtype:
            raise CandleError(f"dtype mismatch in mul, lhs: {_DTYPE_NAMES[xs.dtype]}, rhs: {_DTYPE_NAMES.get(p.dtype, p.dtype)}")
        if p.dim() != 1 or p.shape[0] != cols:
            raise CandleError(f"shape mismatch in broadcast_mul, lhs: {_dims(xs)}, rhs: {_dims(p)}")
    _same_device(xs, weight, bias)
    # the chain starts with to_dtype, which reads a strided input into a contiguous tensor
    xs = xs if xs.is_contiguous() else xs.contiguous()
    weight = weight if weight.is_contiguous() else weight.contiguous()
    if bias is not None and not bias.is_contiguous():
        bias = bias.contiguous()
    rows = xs.numel() // cols if cols else 0
    y = torch.empty_like(xs)
    _cabi.call("cb200_layer_norm_slow", _ptr(xs), _ptr(weight), _ptr(bias), _ptr(y), rows, cols, float(eps),
               _DTYPES[xs.dtype], 1 if remove_mean else 0, _stream(xs))
    return y


def rms_norm_slow(x: torch.Tensor, alpha: torch.Tensor, eps: float) -> torch.Tensor:
    """``candle_nn::ops::rms_norm_slow`` (candle-nn/src/ops.rs:628-639)."""
    return _norm_slow(x, alpha, None, eps, False)


def layer_norm_slow(x: torch.Tensor, alpha: torch.Tensor, beta: torch.Tensor, eps: float) -> torch.Tensor:
    """``candle_nn::ops::layer_norm_slow`` (candle-nn/src/ops.rs:876-894)."""
    return _norm_slow(x, alpha, beta, eps, True)


def _ids_checks(ids: torch.Tensor) -> torch.Tensor:
    if ids.dim() != 1:
        raise CandleError(f"unexpected number of dims: expected 1, got {ids.dim()}, shape {_dims(ids)}")
    if ids.dtype not in _ID_DTYPES:
        raise CandleError(f"unsupported dtype {ids.dtype} for index-select ids (expected U8, U32 or I64)")
    return ids if ids.is_contiguous() else ids.contiguous()  # the CPU op honours an ids stride


def index_select(t: torch.Tensor, ids: torch.Tensor, dim: int, *, check: bool = True,
                 status: torch.Tensor | None = None) -> torch.Tensor:
    """``Tensor::index_select(ids, dim)``.  With ``check`` the call synchronises and raises
    ``InvalidIndex`` like the CPU backend; pass ``check=False`` and a ``status`` record to defer."""
    if not t.is_contiguous():
        raise CandleError("index-select requires contiguous tensors")
    ids = _ids_checks(ids)
    _same_device(t, ids)
    dim = dim if dim >= 0 else dim + t.dim()
    if not 0 <= dim < t.dim():
        raise CandleError(f"dim out of range in index-select: {dim} for shape {_dims(t)}")
    shape = list(t.shape)
    left = 1
    for d in shape[:dim]:
        left *= d
    right = 1
    for d in shape[dim + 1:]:
        right *= d
    src_dim = shape[dim]
    shape[dim] = ids.shape[0]
    out = torch.empty(shape, dtype=t.dtype, device=t.device)
    st = status if status is not None else (new_status(t.device) if check else None)
    _cabi.call("cb200_index_select", _ptr(t), _ptr(ids), _ptr(out), left, src_dim, right, ids.shape[0],
               t.element_size(), _ID_DTYPES[ids.dtype], _ptr(st), _stream(t))
    if check:
        raise_for_status(st)
    return out


def embedding_rms_norm(table: torch.Tensor, ids: torch.Tensor, alpha: torch.Tensor, eps: float, *,
                       return_gathered: bool = False, flags: int = 0, check: bool = True,
                       status: torch.Tensor | None = None):
    """``rms_norm(Embedding::forward(ids), alpha, eps)`` in one launch (ids of any shape)."""
    if table.dim() != 2 or not table.is_contiguous():
        raise CandleError("index-select requires contiguous tensors")
    if alpha.dim() != 1 or alpha.shape[0] != table.shape[1]:
        raise CandleError(f"shape mismatch in rms-norm {list(ids.shape) + [table.shape[1]]} {_dims(alpha)}")
    _norm_checks("rms-norm", table, [("alpha", alpha)], None)
    flat = _ids_checks(ids.reshape(-1))
    _same_device(table, flat, alpha)
    vocab, hidden = table.shape
    final = list(ids.shape) + [hidden]
    y = torch.empty(final, dtype=table.dtype, device=table.device)
    g = torch.empty(final, dtype=table.dtype, device=table.device) if return_gathered else None
    st = status if status is not None else (new_status(table.device) if check else None)
    _cabi.call("cb200_embedding_rms_norm", _ptr(table), _ptr(flat), _ptr(alpha), _ptr(y), _ptr(g), vocab, hidden,
               flat.shape[0], float(eps), _DTYPES[table.dtype], _ID_DTYPES[flat.dtype], flags, _ptr(st),
               _stream(table))
    if check:
        raise_for_status(st)
    return (y, g) if return_gathered else y


def qembedding_rms_norm(qtensor, ids: torch.Tensor, alpha: torch.Tensor, eps: float, *,
                        return_gathered: bool = False, flags: int = 0, check: bool = True,
                        status: torch.Tensor | None = None, vocab_range: tuple[int, int] | None = None,
                        vocab: int | None = None):
    """Rows ``ids`` of a block-quantised table decoded to ``alpha.dtype`` and RMS-normalised: one launch
    for Q4_0 / Q8_0 and the K-quant formats at the usual row lengths, lookup followed by the norm otherwise."""
    from .quantized import QTensor  # local import: quantized imports this module

    if not isinstance(qtensor, QTensor) or len(qtensor.shape) != 2:
        raise CandleError("qembedding expects a rank-2 QTensor")
    if alpha.dtype not in _DTYPES:
        raise CandleError(f"unsupported dtype for rmsnorm {alpha.dtype}")
    local_vocab, hidden = qtensor.shape
    if alpha.dim() != 1 or alpha.shape[0] != hidden or not alpha.is_contiguous():
        raise CandleError(f"shape mismatch in rms-norm {list(ids.shape) + [hidden]} {_dims(alpha)}")
    flat = _ids_checks(ids.reshape(-1))
    _same_device(qtensor.data, flat, alpha)
    begin, end = vocab_range if vocab_range is not None else (0, local_vocab)
    total = vocab if vocab is not None else end
    if end - begin != local_vocab:
        raise CandleError(f"vocab shard [{begin}, {end}) does not match the table's {local_vocab} rows")
    final = list(ids.shape) + [hidden]
    y = torch.empty(final, dtype=alpha.dtype, device=alpha.device)
    g = torch.empty(final, dtype=alpha.dtype, device=alpha.device) if return_gathered else None
    st = status if status is not None else (new_status(alpha.device) if check else None)
    _cabi.call("cb200_qembedding_rms_norm", _ptr(qtensor.data), qtensor.dtype.value, _ptr(flat), _ptr(alpha), _ptr(y),
               _ptr(g), total, hidden, flat.shape[0], float(eps), _DTYPES[alpha.dtype], _ID_DTYPES[flat.dtype],
               begin, end, flags, _ptr(st), _stream(alpha))
    if check:
        raise_for_status(st)
    return (y, g) if return_gathered else y


def qembedding_rms_norm_owner(qtensor, ids: torch.Tensor, alpha: torch.Tensor, eps: float, dst_ptrs, *,
                              vocab_range: tuple[int, int], vocab: int, flags: int = 0,
                              status: torch.Tensor | None = None) -> None:
    """Owner-writes-to-all step of a vocabulary-sharded lookup + RMS norm: the ids inside
    ``vocab_range`` are decoded from this rank's slice ``qtensor``, normalised, and stored into every
    buffer of ``dst_ptrs`` (device addresses of ``[ids.numel(), hidden]`` buffers of ``alpha.dtype``:
    this rank's own first, then the peers' mapped ones).  Ids owned by other ranks are skipped; the
    caller synchronises the ranks before reading.  Invalid ids are recorded in ``status``."""
    import ctypes

    from .quantized import QTensor  # local import: quantized imports this module

    if not isinstance(qtensor, QTensor) or len(qtensor.shape) != 2:
        raise CandleError("qembedding expects a rank-2 QTensor")
    if alpha.dtype not in _DTYPES:
        raise CandleError(f"unsupported dtype for rmsnorm {alpha.dtype}")
    local_vocab, hidden = qtensor.shape
    if alpha.dim() != 1 or alpha.shape[0] != hidden or not alpha.is_contiguous():
        raise CandleError(f"shape mismatch in rms-norm {list(ids.shape) + [hidden]} {_dims(alpha)}")
    flat = _ids_checks(ids.reshape(-1))
    _same_device(qtensor.data, flat, alpha)
    begin, end = vocab_range
    if end - begin != local_vocab:
        raise CandleError(f"vocab shard [{begin}, {end}) does not match the table's {local_vocab} rows")
    ptrs = [int(p) for p in dst_ptrs]
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    _cabi.call("cb200_qembedding_rms_norm_owner", _ptr(qtensor.data), qtensor.dtype.value, _ptr(flat), _ptr(alpha),
               ctypes.cast(arr, ctypes.c_void_p), len(ptrs), vocab, hidden, flat.shape[0], float(eps),
               _DTYPES[alpha.dtype], _ID_DTYPES[flat.dtype], begin, end, flags, _ptr(status), _stream(alpha))


def qembedding_rms_norm_row_owner(qtensor, ids: torch.Tensor, alpha: torch.Tensor, eps: float, dst_ptrs, row_bounds, *,
                                  vocab_range: tuple[int, int], vocab: int, flags: int = 0,
                                  status: torch.Tensor | None = None) -> None:
    """Row-owner step of a vocabulary-sharded lookup + RMS norm: the ids inside ``vocab_range`` are
    decoded from this rank's slice ``qtensor`` and normalised, and each finished row is stored into
    the one buffer whose block of token rows contains it.  ``dst_ptrs[r]`` is the device address of
    rank r's ``[row_bounds[r + 1] - row_bounds[r], hidden]`` buffer (rank order; peers' buffers mapped
    into this process), ``row_bounds`` the ``len(dst_ptrs) + 1`` block limits from 0 to ``ids.numel()``.
    Ids owned by other ranks are skipped; the caller synchronises the ranks before reading."""
    import ctypes

    from .quantized import QTensor  # local import: quantized imports this module

    if not isinstance(qtensor, QTensor) or len(qtensor.shape) != 2:
        raise CandleError("qembedding expects a rank-2 QTensor")
    if alpha.dtype not in _DTYPES:
        raise CandleError(f"unsupported dtype for rmsnorm {alpha.dtype}")
    local_vocab, hidden = qtensor.shape
    if alpha.dim() != 1 or alpha.shape[0] != hidden or not alpha.is_contiguous():
        raise CandleError(f"shape mismatch in rms-norm {list(ids.shape) + [hidden]} {_dims(alpha)}")
    flat = _ids_checks(ids.reshape(-1))
    _same_device(qtensor.data, flat, alpha)
    begin, end = vocab_range
    if end - begin != local_vocab:
        raise CandleError(f"vocab shard [{begin}, {end}) does not match the table's {local_vocab} rows")
    ptrs = [int(p) for p in dst_ptrs]
    bounds = [int(b) for b in row_bounds]
    if len(bounds) != len(ptrs) + 1:
        raise CandleError(f"{len(ptrs)} destinations need {len(ptrs) + 1} row bounds, got {len(bounds)}")
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    barr = (ctypes.c_int64 * len(bounds))(*bounds)
    _cabi.call("cb200_qembedding_rms_norm_row_owner", _ptr(qtensor.data), qtensor.dtype.value, _ptr(flat), _ptr(alpha),
               ctypes.cast(arr, ctypes.c_void_p), len(ptrs), ctypes.cast(barr, ctypes.c_void_p), vocab, hidden,
               flat.shape[0], float(eps), _DTYPES[alpha.dtype], _ID_DTYPES[flat.dtype], begin, end, flags, _ptr(status),
               _stream(alpha))


def softmax_last_dim(xs: torch.Tensor) -> torch.Tensor:
    """``candle_nn::ops::softmax_last_dim`` (candle-nn/src/ops.rs:289-435)."""
    if xs.dtype not in _DTYPES:
        raise CandleError(f"unsupported dtype for softmax {_DTYPE_NAMES.get(xs.dtype, xs.dtype)}")
    if not xs.is_contiguous():
        raise CandleError("input has to be contiguous")
    _same_device(xs)
    if xs.dim() == 0:
        raise CandleError("unexpected rank, expected: at least 1, got: 0")
    cols = xs.shape[-1]
    rows = xs.numel() // cols if cols else 0
    y = torch.empty_like(xs)
    _cabi.call("cb200_softmax_last_dim", _ptr(xs), _ptr(y), rows, cols, _DTYPES[xs.dtype], _stream(xs))
    return y


def _rope(variant: int, name: str, xs: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    # the checks of rotary_emb.rs:203-228 (rope_i), 457-482 (rope), 706-731 (rope_thd)
    if xs.dim() != 4:
        raise CandleError(f"unexpected rank, expected: 4, got: {xs.dim()} ({_dims(xs)})")
    if cos.dim() != 2 or sin.dim() != 2:
        bad = cos if cos.dim() != 2 else sin
        raise CandleError(f"unexpected rank, expected: 2, got: {bad.dim()} ({_dims(bad)})")
    if variant == _cabi.ROPE_THD:
        b, seq_len, h, n_embd = xs.shape
    else:
        b, h, seq_len, n_embd = xs.shape
    if cos.shape[1] * 2 != n_embd or sin.shape[1] * 2 != n_embd or seq_len > cos.shape[0] or seq_len > sin.shape[0]:
        raise CandleError(f"inconsistent last dim size in rope {_dims(xs)} {_dims(cos)} {_dims(sin)}")
    if not xs.is_contiguous():
        raise CandleError("xs has to be contiguous in rope")
    if not cos.is_contiguous():
        raise CandleError("cos has to be contiguous in rope")
    if not sin.is_contiguous():
        raise CandleError("sin has to be contiguous in rope")
    if xs.dtype not in _DTYPES or cos.dtype != xs.dtype or sin.dtype != xs.dtype:
        raise CandleError(f"unsupported dtype for rope {xs.dtype} {cos.dtype} {sin.dtype}")
    _same_device(xs, cos, sin)
    dst = torch.empty_like(xs)
    _cabi.call("cb200_rope", _ptr(xs), _ptr(cos), _ptr(sin), _ptr(dst), b, h, seq_len, n_embd, _DTYPES[xs.dtype], variant,
               _stream(xs))
    return dst


def rope_i(xs: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``candle_nn::rotary_emb::rope_i``: interleaved pairs, ``xs`` is ``[b, h, t, d]``."""
    return _rope(_cabi.ROPE_INTERLEAVED, "rope-i", xs, cos, sin)


def rope(xs: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``candle_nn::rotary_emb::rope``: pairs ``(x[k], x[k + d/2])``, ``xs`` is ``[b, h, t, d]``."""
    return _rope(_cabi.ROPE_HALF, "rope", xs, cos, sin)


def rope_thd(xs: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``candle_nn::rotary_emb::rope_thd``: as ``rope`` for ``xs`` laid out ``[b, t, h, d]``."""
    return _rope(_cabi.ROPE_THD, "rope-thd", xs, cos, sin)


def rms_norm_rows(xs: torch.Tensor, rows: torch.Tensor, alpha: torch.Tensor, eps: float, *, check: bool = True,
                  status: torch.Tensor | None = None) -> torch.Tensor:
    """RMS norm of the selected rows only: ``rms_norm(xs, alpha, eps).index_select(rows, 0)`` without
    normalising the rows nobody reads.  The final norm of a decoder is followed by a slice that keeps
    the last token of each sequence (candle-transformers/src/models/quantized_llama.rs:507-508: norm of
    all rows, then ``x.i((.., seq_len - 1, ..))``); with ``rows`` = those positions in the flattened
    ``[b * t, hidden]`` activations this reads and writes ``b`` rows instead of ``b * t``.  Rows are
    independent, so the values are the same."""
    if xs.dim() != 2:
        raise CandleError(f"unexpected rank, expected: 2, got: {xs.dim()} ({_dims(xs)})")
    return embedding_rms_norm(xs, rows, alpha, eps, check=check, status=status)


def qembedding_route_rows(qtensor, ids: torch.Tensor, dst_ptrs, row_bounds, *, vocab_range: tuple[int, int], vocab: int,
                          status: torch.Tensor | None = None) -> None:
    """Routing step of a vocabulary-sharded lookup with row-sharded consumers: for every id inside
    ``vocab_range`` the raw block row of this rank's slice ``qtensor`` is copied into the staging buffer
    of the rank whose block of token rows holds the id's position (``dst_ptrs`` in rank order,
    ``row_bounds`` the block limits).  After the ranks' barrier each staging buffer is a
    ``[rows_r, hidden]`` table of blocks in token order, ready for a local lookup + norm."""
    import ctypes

    from .quantized import QTensor  # local import: quantized imports this module

    if not isinstance(qtensor, QTensor) or len(qtensor.shape) != 2:
        raise CandleError("qembedding expects a rank-2 QTensor")
    local_vocab, hidden = qtensor.shape
    flat = _ids_checks(ids.reshape(-1))
    _same_device(qtensor.data, flat)
    begin, end = vocab_range
    if end - begin != local_vocab:
        raise CandleError(f"vocab shard [{begin}, {end}) does not match the table's {local_vocab} rows")
    ptrs = [int(p) for p in dst_ptrs]
    bounds = [int(b) for b in row_bounds]
    if len(bounds) != len(ptrs) + 1:
        raise CandleError(f"{len(ptrs)} destinations need {len(ptrs) + 1} row bounds, got {len(bounds)}")
    arr = (ctypes.c_void_p * len(ptrs))(*ptrs)
    barr = (ctypes.c_int64 * len(bounds))(*bounds)
    _cabi.call("cb200_qembedding_route_rows", _ptr(qtensor.data), qtensor.dtype.value, _ptr(flat),
               ctypes.cast(arr, ctypes.c_void_p), len(ptrs), ctypes.cast(barr, ctypes.c_void_p), vocab, hidden,
               flat.shape[0], _ID_DTYPES[flat.dtype], begin, end, _ptr(status), _stream(flat))
