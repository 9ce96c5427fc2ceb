"""ctypes binding of ``libcandle_b200_nccl.so`` (include/candle_b200_nccl.h)."""
from __future__ import annotations

import ctypes
import os

from . import _cabi  # noqa: F401  (loads libcandle_b200.so first: the NCCL library links against it)
from .build import NCCL_LIB_PATH

_vp, _i64, _i32, _f32, _int, _sz = (ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32, ctypes.c_float, ctypes.c_int,
                                   ctypes.c_size_t)
SIGNATURES = {
    "cb200_nccl_unique_id": [_vp],
    "cb200_nccl_comm_init": [ctypes.POINTER(_vp), _int, _vp, _int],
    "cb200_nccl_comm_init_timeout": [ctypes.POINTER(_vp), _int, _vp, _int, _int],
    "cb200_nccl_comm_destroy": [_vp],
    "cb200_sharded_qembedding_rms_norm": [
        _vp, _vp, _int, _vp, _vp, _vp, _vp, _sz, _i64, _i32, _i64, _f32, _int, _int, _i64, _i64, _int, _vp, _vp,
    ],
    "cb200_sharded_qembedding_rms_norm_static": [
        _vp, _vp, _int, _vp, _vp, _vp, _i64, _i32, _i64, _f32, _int, _int, _i64, _i64, _int, _vp, _vp,
    ],
}
UNIQUE_ID_BYTES = 128
STATIC_SCRATCH_BYTES = 32 * 1024 * 1024
E_TIMEOUT = -6


def _load() -> ctypes.CDLL:
    if not os.path.exists(NCCL_LIB_PATH):
        raise ImportError(f"{NCCL_LIB_PATH} is missing: build it first (python -m candle_b200.build)")
    import torch  # noqa: F401  (brings torch's libnccl.so.2 into the process before ours asks for it)

    lib = ctypes.CDLL(NCCL_LIB_PATH)
    for name, argtypes in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = ctypes.c_int
    return lib


lib = _load()


def call(name: str, *args) -> None:
    rc = getattr(lib, name)(*args)
    if rc != 0:
        raise _cabi.CandleB200Error(rc, f"{name} failed (see stderr)")


def unique_id() -> bytes:
    buf = ctypes.create_string_buffer(UNIQUE_ID_BYTES)
    call("cb200_nccl_unique_id", ctypes.cast(buf, _vp))
    return buf.raw


def comm_init(nranks: int, uid: bytes, rank: int) -> ctypes.c_void_p:
    comm = _vp()
    buf = ctypes.create_string_buffer(uid, UNIQUE_ID_BYTES)
    call("cb200_nccl_comm_init", ctypes.byref(comm), nranks, ctypes.cast(buf, _vp), rank)
    return comm


def comm_init_timeout(nranks: int, uid: bytes, rank: int, timeout_ms: int) -> ctypes.c_void_p:
    """``comm_init`` that gives up (error code ``E_TIMEOUT``) when the ranks have not all joined in time."""
    comm = _vp()
    buf = ctypes.create_string_buffer(uid, UNIQUE_ID_BYTES)
    call("cb200_nccl_comm_init_timeout", ctypes.byref(comm), nranks, ctypes.cast(buf, _vp), rank, timeout_ms)
    return comm


def comm_destroy(comm) -> None:
    call("cb200_nccl_comm_destroy", comm)
