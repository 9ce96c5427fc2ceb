"""ctypes binding of ``libcandle_b200.so`` -- the same C ABI a Rust ``extern "C"`` block would bind.

There is no fallback: if the library has not been built the import of this module fails.
"""
from __future__ import annotations

import ctypes
import os

from .build import LIB_PATH

# name -> argtypes, in the order of include/candle_b200.h
_vp, _i64, _i32, _f32, _int = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float, ctypes.c_int
SIGNATURES = {
    "cb200_version": [],
    "cb200_last_error": [],
    "cb200_rms_norm": [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _int, _int, _vp],
    "cb200_layer_norm": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _int, _int, _vp],
    "cb200_rms_norm_checked": [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _int, _int, _vp, _vp],
    "cb200_layer_norm_checked": [_vp, _vp, _vp, _vp, _vp, _vp, _i64, _i32, _f32, _int, _int, _vp, _vp],
    "cb200_layer_norm_slow": [_vp, _vp, _vp, _vp, _i64, _i32, _f32, _int, _int, _vp],
    "cb200_softmax_last_dim": [_vp, _vp, _i64, _i32, _int, _vp],
    "cb200_rope": [_vp, _vp, _vp, _vp, _i64, _i32, _i32, _i32, _int, _int, _vp],
    "cb200_selftest_wait_expiry": [_int],
    "cb200_index_select": [_vp, _vp, _vp, _i64, _i64, _i64, _i64, _i32, _int, _vp, _vp],
    "cb200_embedding": [_vp, _vp, _vp, _i64, _i32, _i64, _int, _int, _vp, _vp],
    "cb200_dequantize": [_vp, _int, _vp, _i64, _int, _vp],
    "cb200_qembedding": [_vp, _int, _vp, _vp, _i64, _i32, _i64, _int, _int, _i64, _i64, _vp, _vp],
    "cb200_embedding_rms_norm": [_vp, _vp, _vp, _vp, _vp, _i64, _i32, _i64, _f32, _int, _int, _int, _vp, _vp],
    "cb200_qembedding_rms_norm": [
        _vp, _int, _vp, _vp, _vp, _vp, _i64, _i32, _i64, _f32, _int, _int, _i64, _i64, _int, _vp, _vp,
    ],
    "cb200_qembedding_rms_norm_owner": [
        _vp, _int, _vp, _vp, _vp, _int, _i64, _i32, _i64, _f32, _int, _int, _i64, _i64, _int, _vp, _vp,
    ],
    "cb200_qembedding_route_rows": [_vp, _int, _vp, _vp, _int, _vp, _i64, _i32, _i64, _int, _i64, _i64, _vp, _vp],
    "cb200_qembedding_rms_norm_row_owner": [
        _vp, _int, _vp, _vp, _vp, _int, _vp, _i64, _i32, _i64, _f32, _int, _int, _i64, _i64, _int, _vp, _vp,
    ],
}

DTYPE_F32, DTYPE_F16, DTYPE_BF16 = 0, 1, 2
ID_U8, ID_U32, ID_I64 = 0, 1, 2
QTYPE_Q4_0, QTYPE_Q4_1, QTYPE_Q5_0, QTYPE_Q5_1, QTYPE_Q8_0 = 2, 3, 6, 7, 8
QTYPE_Q2K, QTYPE_Q3K, QTYPE_Q4K, QTYPE_Q5K, QTYPE_Q6K, QTYPE_Q8K = 10, 11, 12, 13, 14, 15
FLAG_FAST_SUM, FLAG_FORCE_LANEROW, FLAG_FORCE_GENERIC, FLAG_FORCE_REPLAY = 1, 0x100, 0x200, 0x400
STATUS_OK, STATUS_INVALID_INDEX, STATUS_WAIT_TIMEOUT = 0, 1, 2
ROPE_INTERLEAVED, ROPE_HALF, ROPE_THD = 0, 1, 2


class CandleB200Error(RuntimeError):
    """A negative return code from the C ABI, carrying cb200_last_error()."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{message} (code {code})")
        self.code = code


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build the CUDA extension first (python -m candle_b200.build); "
            "there is no CPU fallback"
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError here = the library does not export a declared symbol
        fn.argtypes = argtypes
        fn.restype = ctypes.c_char_p if name == "cb200_last_error" else ctypes.c_int
    return lib


lib = _load()


def call(name: str, *args) -> None:
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise CandleB200Error(rc, lib.cb200_last_error().decode())
