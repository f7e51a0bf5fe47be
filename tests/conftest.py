import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
GOLDEN = os.path.join(ROOT, "tests", "golden")


@pytest.fixture(autouse=True)
def _inference_mode_by_default(request):
    """Tests run with gradients disabled, as inference callers do; tests marked `autograd` keep them enabled."""
    import torch
    if request.node.get_closest_marker("autograd") is not None:
        yield
    else:
        with torch.no_grad():
            yield


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")
    config.addinivalue_line("markers", "autograd: the test runs with gradients enabled")


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


# The shipped foveated AlexNet (config/fovi_alexnet.yaml of the reference: base_lowres, a=0.5, 64x64 resources) and the
# deterministic parameters the golden generator gave the reference model; same as in golden/make_golden.py.
ALEXNET_SHIPPED = dict(in_res=64, in_channels=3, features_per_layer=[96, 256, 384, 384, 256], stride_per_layer=[2, 1, 1, 1, 1],
                       pool_after=[0, 1, 4], k_per_layer=[121, 25, 9, 9, 9], out_res=1, auto_match_cart_resources=1, fov=16.0, cmf_a=0.5,
                       norm_type="force_batch", ref_frame_mult=2, sample_cortex=True)


def seed_alexnet(model, seed):
    import torch
    f32 = np.float32
    for i, block in enumerate(model.layers):
        if not hasattr(block, "conv"):
            continue
        rs = np.random.RandomState(seed + i)
        cout, fan = block.conv.weight.shape
        dev = block.conv.weight.device
        put = lambda t, a: t.copy_(torch.from_numpy(a.astype(f32)).to(dev))  # noqa: E731
        with torch.no_grad():
            put(block.conv.weight, rs.standard_normal((cout, fan)) * np.sqrt(2.0 / fan))
            put(block.norm.weight, 0.5 + rs.random_sample(cout))
            put(block.norm.bias, 0.2 * rs.standard_normal(cout))
            put(block.norm.running_mean, 0.1 * rs.standard_normal(cout))
            put(block.norm.running_var, 0.5 + rs.random_sample(cout))
    if getattr(model, "n_classes", None) is not None:
        rs = np.random.RandomState(seed + 100)
        w = model.classifier.weight
        with torch.no_grad():
            w.copy_(torch.from_numpy((rs.standard_normal(tuple(w.shape)) / np.sqrt(w.shape[1])).astype(f32)).to(w.device))
            model.classifier.bias.copy_(torch.from_numpy((0.1 * rs.standard_normal(w.shape[0])).astype(f32)).to(w.device))
