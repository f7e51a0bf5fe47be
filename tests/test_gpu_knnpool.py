"""GPU: KNN pooling kernel against the outputs recorded from the reference and the oracle."""
import numpy as np
import pytest
import torch

from conftest import synth_images
from oracle import fovi_oracle as oracle

pytestmark = pytest.mark.gpu
f32 = np.float32


def test_pooling_layer_matches_reference(golden):
    from fovi_b200.coords import SamplingCoords, get_in_out_coords
    from fovi_b200.knn import KNNPoolingLayer
    g = golden("pool_a0p5.npz")
    c = SamplingCoords(16, 0.5, 53)
    ic, oc, _ = get_in_out_coords(53, 16, 0.5, 2, auto_match_cart_resources=1, in_cart_res=64, in_coords=c)
    x = torch.from_numpy(synth_images(5, (2, 4, len(ic))) - f32(0.5)).cuda()
    for mode, key, exact in (("max", "out", True), ("avg", "out_avg", False), ("sum", "out_sum", False)):
        pool = KNNPoolingLayer(9, ic, oc, mode=mode, device="cuda")
        assert np.array_equal(pool.knn_indices.numpy(), g["knn_idx"])            # table bit-exact vs the reference
        y = pool(x)
        assert y.shape == (2, 4, 964)
        if exact:
            assert np.array_equal(y.cpu().numpy(), g[key])
        else:
            np.testing.assert_allclose(y.cpu().numpy(), g[key], rtol=1e-6, atol=1e-7)
        yp = pool.forward_points(x.permute(0, 2, 1).contiguous())                # channels-last gives the same numbers
        assert torch.equal(yp.permute(0, 2, 1), y)


def test_pooling_edge_cases():
    from fovi_b200 import ops
    rs = np.random.RandomState(3)
    B, C, Nin, Nout, K = 3, 5, 13, 6, 4
    x = rs.standard_normal((B, C, Nin)).astype(f32)
    x[0, 0, 2] = np.nan                                        # a NaN input is skipped like a pad
    idx = rs.randint(0, Nin + 1, (K, Nout)).astype(np.int32)
    idx[:, 0] = Nin                                            # a point whose neighbours are all pads
    idx[0, 1] = 2
    plan = ops.KnnPoolPlan(idx, Nin)
    xd = torch.from_numpy(x).cuda()
    ymax = plan.forward(xd, "max").cpu().numpy()
    g = oracle._pool_gather(x, idx)
    want = np.where(np.isnan(g), -np.inf, g).max(2)
    assert np.array_equal(ymax, want) and np.all(np.isneginf(ymax[:, :, 0]))
    ysum = plan.forward(xd, "sum").cpu().numpy()
    np.testing.assert_allclose(ysum, oracle.knn_pool_sum(x, idx), rtol=1e-6, atol=1e-6)
    assert np.all(ysum[:, :, 0] == 0)
    yavg = plan.forward(xd, "avg").cpu().numpy()
    assert np.all(np.isnan(yavg[:, :, 0]))
    np.testing.assert_allclose(yavg[:, :, 1:], oracle.knn_pool_avg(x, idx)[:, :, 1:], rtol=1e-6, atol=1e-6)
    # bf16, channels-last
    xb = torch.from_numpy(np.nan_to_num(x)).cuda().to(torch.bfloat16).permute(0, 2, 1).contiguous()
    yb = plan.forward(xb, "max", ops.ACT_BNC)
    wantb = np.where(np.isnan(oracle._pool_gather(xb.float().permute(0, 2, 1).cpu().numpy(), idx)), -np.inf,
                     oracle._pool_gather(xb.float().permute(0, 2, 1).cpu().numpy(), idx)).max(2)
    assert np.array_equal(yb.float().permute(0, 2, 1).cpu().numpy(), wantb)


@pytest.mark.parametrize("mode", ["max", "avg", "sum"])
def test_vectorised_channels_last_kernel_equals_scalar_kernel(mode):
    """bf16 channels-last with a multiple of 8 channels takes the 16-byte-load kernel: same numbers as the scalar one
    (run here on float32 copies of the same bf16 values), pads and NaN inputs included."""
    from fovi_b200 import ops
    rs = np.random.RandomState(11)
    B, C, Nin, Nout, K = 5, 24, 37, 19, 9
    x = torch.from_numpy(rs.standard_normal((B, Nin, C)).astype(f32)).to(torch.bfloat16)
    x[1, 3, 5] = float("nan")
    x[2, :, 7] = float("nan")                                   # a channel that is NaN everywhere in one row
    idx = rs.randint(0, Nin + 1, (K, Nout)).astype(np.int32)
    idx[:, 0] = Nin
    plan = ops.KnnPoolPlan(idx, Nin)
    y = plan.forward(x.cuda(), mode, ops.ACT_BNC)
    ref = plan.forward(x.float().cuda(), mode, ops.ACT_BNC).to(torch.bfloat16)        # scalar kernel, float32 in and out
    assert y.dtype == torch.bfloat16 and y.shape == (B, Nout, C)
    a, b = y.float().cpu().numpy(), ref.float().cpu().numpy()
    assert np.array_equal(np.isnan(a), np.isnan(b))
    assert np.array_equal(np.nan_to_num(a, nan=0.0, posinf=1e30, neginf=-1e30), np.nan_to_num(b, nan=0.0, posinf=1e30, neginf=-1e30))
