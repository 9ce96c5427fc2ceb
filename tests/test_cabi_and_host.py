"""CPU-only checks: the built library exports every symbol the header declares, the ctypes
signatures agree with the header, and the front ends reject bad calls before touching a device."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built_lib():
    from candle_b200 import build

    return build.build()  # no-op when up to date


def header_functions(only=None):
    """name -> number of parameters, parsed from every include/*.h (or just the file `only`)."""
    out = {}
    inc = os.path.join(ROOT, "include")
    for fn in sorted(os.listdir(inc)):
        if not fn.endswith(".h") or (only is not None and fn != only):
            continue
        text = open(os.path.join(inc, fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"CB200_API\s+[\w\s\*]+?\b(cb200_\w+)\s*\(([^;]*?)\)\s*;", text, flags=re.S):
            params = m.group(2).strip()
            out[m.group(1)] = 0 if params in ("", "void") else params.count(",") + 1
    return out


def test_library_exports_every_declared_symbol(built_lib):
    from candle_b200 import build

    lib = ctypes.CDLL(built_lib)
    declared = header_functions("candle_b200.h")
    assert len(declared) >= 10
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/candle_b200.h but not exported"
    assert lib.cb200_version() == 100
    nccl_path = build.build_nccl()
    import torch  # noqa: F401  (its libnccl.so.2 satisfies the dependency, as in a real process)

    nccl_lib = ctypes.CDLL(nccl_path)
    declared = header_functions("candle_b200_nccl.h")
    assert len(declared) >= 4
    for name in declared:
        assert hasattr(nccl_lib, name), f"{name} is declared in include/candle_b200_nccl.h but not exported"
    assert len(header_functions()) == len(header_functions("candle_b200.h")) + len(declared)


def test_ctypes_signatures_match_the_header(built_lib):
    from candle_b200 import _cabi, _nccl

    for mod, header in ((_cabi, "candle_b200.h"), (_nccl, "candle_b200_nccl.h")):
        declared = header_functions(header)
        assert set(mod.SIGNATURES) == set(declared)
        for name, argtypes in mod.SIGNATURES.items():
            assert len(argtypes) == declared[name], name


def test_rust_ffi_declares_the_same_entry_points():
    """rust/candle-b200-kernels/src/ffi.rs (not compiled here) names every entry point of the headers with the
    same number of parameters; the self-test hook and the thin NCCL wrappers (cudarc has its own) are left out."""
    text = open(os.path.join(ROOT, "rust", "candle-b200-kernels", "src", "ffi.rs")).read()
    rust = {}
    for m in re.finditer(r"pub fn (cb200_\w+)\s*\(([^;]*?)\)\s*(?:->\s*[\w\s\*:]+)?;", text, flags=re.S):
        params = m.group(2).strip()
        rust[m.group(1)] = 0 if not params else len([p for p in params.split(",") if p.strip()])
    skipped = {"cb200_selftest_wait_expiry", "cb200_nccl_unique_id", "cb200_nccl_comm_init", "cb200_nccl_comm_init_timeout",
               "cb200_nccl_comm_destroy"}
    declared = {k: v for k, v in header_functions().items() if k not in skipped}
    assert set(rust) == set(declared), set(rust) ^ set(declared)
    for name, n in declared.items():
        assert rust[name] == n, name


def test_argument_validation_needs_no_device(built_lib):
    from candle_b200 import _cabi

    lib = _cabi.lib
    one = ctypes.c_void_p(16)  # never dereferenced: validation fails first
    assert lib.cb200_rms_norm(one, None, one, one, None, 4, 8, 1e-5, 7, 0, None) == -2  # bad dtype
    assert b"unsupported dtype" in lib.cb200_last_error()
    assert lib.cb200_rms_norm(one, None, one, one, None, -1, 8, 1e-5, 0, 0, None) == -1
    assert lib.cb200_rms_norm(None, None, one, one, None, 4, 8, 1e-5, 0, 0, None) == -1
    assert lib.cb200_rms_norm(one, None, one, one, None, 0, 8, 1e-5, 0, 0, None) == 0  # nothing to do
    assert lib.cb200_layer_norm(one, None, one, None, one, None, 4, 8, 1e-5, 0, 0, None) == -1  # beta missing
    assert lib.cb200_qembedding(one, 9, one, one, 10, 64, 4, 0, 1, 0, 10, None, None) == -2  # Q8_1 has no to_float
    assert lib.cb200_qembedding(one, 12, one, one, 10, 64, 4, 0, 1, 0, 10, None, None) == -1  # Q4K: hidden % 256
    assert b"not divisible by 256" in lib.cb200_last_error()
    assert lib.cb200_qembedding(one, 8, one, one, 10, 48, 4, 0, 1, 0, 10, None, None) == -1  # hidden % 32
    assert b"not divisible by 32" in lib.cb200_last_error()
    assert lib.cb200_qembedding(one, 8, one, one, 10, 64, 4, 0, 1, 5, 11, None, None) == -1  # shard outside vocab
    assert lib.cb200_dequantize(one, 2, one, 33, 0, None) == -1
    assert lib.cb200_index_select(one, one, one, 1, 4, 3, 2, 4, 9, None, None) == -2  # bad ids dtype
    assert lib.cb200_index_select(one, one, one, 1, 4, 3, 0, 4, 1, None, None) == 0  # empty ids


def test_front_ends_reject_bad_calls_on_the_host():
    import candle_b200 as cb

    x = torch.randn(4, 8)
    with pytest.raises(cb.CandleError, match="shape mismatch in rms-norm"):
        cb.rms_norm(x, torch.ones(7), 1e-5)
    with pytest.raises(cb.CandleError, match="shape mismatch in layer-norm"):
        cb.layer_norm(x, torch.ones(8), torch.ones(9), 1e-5)
    with pytest.raises(cb.CandleError, match="input has to be contiguous"):
        cb.rms_norm(x.t(), torch.ones(4), 1e-5)
    with pytest.raises(cb.CandleError, match="unsupported dtype for rmsnorm"):
        cb.rms_norm(x.double(), torch.ones(8, dtype=torch.float64), 1e-5)
    with pytest.raises(cb.CandleError, match="no CPU fallback"):
        cb.rms_norm(x, torch.ones(8), 1e-5)  # everything valid except the device
    with pytest.raises(cb.CandleError, match="block size"):
        cb.QTensor(torch.zeros(18, dtype=torch.uint8), cb.GgmlDType.Q4_0, (1, 33))
    assert cb.GgmlDType.Q8_0.type_size == 34 and cb.GgmlDType.Q4_0.type_size == 18


def test_partitioning_helpers():
    from candle_b200 import CandleError
    from candle_b200.parallel import row_shard, vocab_shard

    for rows in (0, 1, 7, 64, 65536, 65537):
        for world in (1, 2, 4, 8):
            parts = [row_shard(rows, r, world) for r in range(world)]
            assert parts[0][0] == 0 and parts[-1][1] == rows
            assert all(parts[i][1] == parts[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in parts]
            assert max(sizes) - min(sizes) <= 1
    assert vocab_shard(152064, 3, 8) == (57024, 76032)
    with pytest.raises(CandleError, match="not divisible"):
        vocab_shard(10, 0, 4)
    with pytest.raises(CandleError):
        row_shard(10, 4, 4)


def test_bench_workload_accounting():
    import sys

    sys.path.insert(0, ROOT)
    import bench

    rng = np.random.default_rng(0)
    ids = bench.zipf_ids(rng, 1000, 20000)
    assert ids.dtype == np.uint32 and ids.max() < 1000
    counts = np.bincount(ids, minlength=1000)
    assert counts[0] > counts[10] > counts[500]  # rank k -> id k-1: the head is hottest
    w = bench.Workload("c2")
    assert w.bytes_per_step == 3 * 16384 * 768 * 2 == 75497472
    w = bench.Workload("c5", rows_scale=1 / 64)
    assert w.rows == 1024 and w.bytes_per_step == 3 * 1024 * 8192 * 2
