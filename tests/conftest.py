import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def golden():
    cache = {}

    def load(name):
        if name not in cache:
            cache[name] = dict(np.load(os.path.join(GOLDEN, name)))
        return cache[name]
    return load


def synth_images(seed, shape):
    """Uniform [0,1) float32 from numpy's frozen legacy bit-stream (same as the fixture generator)."""
    return np.random.RandomState(seed).random_sample(shape).astype(np.float32)


def kaiming_weight(rs, cout, cin, V):
    return (rs.standard_normal((cout, cin * V)) * np.sqrt(2.0 / (cin * V))).astype(np.float32)
