import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def kats():
    with open(os.path.join(ROOT, "tests", "golden", "candle_kats.json")) as f:
        return json.load(f)


@pytest.fixture(scope="session")
def cb():
    """The package under test, for the GPU tests: there is no CPU path to fall back on."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import candle_b200

    return candle_b200


def round4(a):
    """candle's test_utils::to_vec*_round(t, 4): f32::round(t * 1e4) / 1e4 evaluated in f32."""
    a = np.asarray(a, dtype=np.float32)
    b = np.float32(10.0) ** np.int32(4)
    t = (a * b).astype(np.float32)
    r = np.where(t >= 0, np.floor(t + np.float32(0.5)), np.ceil(t - np.float32(0.5))).astype(np.float32)
    return (r / b).astype(np.float32)
