"""Two host threads, each on a stream of its own, launching the same kernels with different shapes at the
same time: per-kernel attributes (dynamic shared-memory limit, carve-out) and the cached occupancy are
shared state inside the library, so every result is compared, 1000 iterations per thread, with the
result the same call gave single-threaded -- which is first checked against the CPU oracle."""
import threading

import numpy as np
import pytest
import torch

import oracle
from helpers import from_oracle, randn, to_oracle

pytestmark = pytest.mark.gpu
ITERATIONS = 1000


def _cases(cb, seed, shapes):
    """[(call, expected)] for (op, dtype, rows, hidden) shapes; expected = single-threaded result = oracle."""
    rng = np.random.default_rng(seed)
    out = []
    for op, dtype, rows, hidden in shapes:
        x, r = randn(rng, (rows, hidden), dtype), randn(rng, (rows, hidden), dtype)
        g, b = randn(rng, (hidden,), dtype, 1.0, 0.1), randn(rng, (hidden,), dtype, 0.0, 0.1)
        xt, rt, gt, bt = (from_oracle(v, dtype) for v in (x, r, g, b))
        h = oracle.add(x, r, dtype)
        if op == "rms":
            want = oracle.rms_norm(h, g, 1e-5, dtype)
            call = lambda xt=xt, rt=rt, gt=gt: cb.rms_norm(xt, gt, 1e-5, residual=rt)
        else:
            want = oracle.layer_norm(h, g, b, 1e-5, dtype)
            call = lambda xt=xt, rt=rt, gt=gt, bt=bt: cb.layer_norm(xt, gt, bt, 1e-5, residual=rt)
        expected = call()
        torch.cuda.synchronize()
        assert np.array_equal(to_oracle(expected), want), (op, dtype, rows, hidden)
        out.append((call, expected))
    return out


def test_two_threads_two_streams_same_kernels_different_shapes(cb):
    # the same kernel templates from both threads, with different row lengths (different dynamic shared
    # memory and carve-out per launch), interleaved with kernels only one of the threads uses
    shapes_a = [("rms", "bf16", 96, 8192), ("rms", "bf16", 300, 1024), ("ln", "bf16", 200, 768), ("rms", "f32", 64, 4096)]
    shapes_b = [("rms", "bf16", 128, 4096), ("rms", "bf16", 77, 2048), ("ln", "bf16", 150, 1536), ("rms", "f32", 100, 1024),
                ("rms", "f16", 64, 8192)]
    work = [_cases(cb, 1, shapes_a), _cases(cb, 2, shapes_b)]
    errors, mismatches = [], [None, None]
    start = threading.Barrier(2)

    def run(k):
        try:
            stream = torch.cuda.Stream()
            bad = torch.zeros((), dtype=torch.int64, device="cuda")
            start.wait()
            with torch.cuda.stream(stream):
                for i in range(ITERATIONS):
                    call, expected = work[k][i % len(work[k])]
                    y = call()
                    bad += (y.view(torch.uint8) != expected.view(torch.uint8)).any()
            stream.synchronize()
            mismatches[k] = int(bad.item())
        except Exception as exc:  # surfaced by the assertion below
            errors.append(f"thread {k}: {type(exc).__name__}: {exc}")

    threads = [threading.Thread(target=run, args=(k,)) for k in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert mismatches == [0, 0], mismatches
