"""GPU: gradient of KNNPoolingLayer with respect to its input (fovi_knnpool_backward) against the gradients the reference's
autograd produced on CPU (tests/golden/pool_backward_small.npz) and against the oracle."""
import numpy as np
import pytest
import torch

from oracle import fovi_oracle as oracle

pytestmark = [pytest.mark.gpu, pytest.mark.autograd]


class _Pts:
    def __init__(self, n):
        self.shape = (n, 2)
        self.dtype = torch.float32


@pytest.mark.parametrize("mode", ["max", "avg", "sum", "gaussian"])
@pytest.mark.parametrize("layout", ["bcn", "bnc"])
def test_pool_gradient_matches_reference_autograd(golden, mode, layout):
    from fovi_b200 import ops
    g = golden("pool_backward_small.npz")
    plan = ops.KnnPoolPlan(g["knn_idx_pad"], int(g["n_in"]))
    if mode == "gaussian":
        plan.set_weights(g["weights"])
    x, gy = torch.from_numpy(g["x"]).cuda(), torch.from_numpy(g[f"{mode}_gy"]).cuda()
    if layout == "bcn":
        y = plan.forward(x, mode, ops.ACT_BCN)
        dx = plan.backward(x, gy, mode, ops.ACT_BCN)
    else:
        y = plan.forward(x.permute(0, 2, 1).contiguous(), mode, ops.ACT_BNC).permute(0, 2, 1)
        dx = plan.backward(x.permute(0, 2, 1).contiguous(), gy.permute(0, 2, 1).contiguous(), mode, ops.ACT_BNC).permute(0, 2, 1)
    assert np.abs(y.cpu().numpy() - g[f"{mode}_y"]).max() < 1e-5
    assert np.abs(dx.cpu().numpy() - g[f"{mode}_dx"]).max() < 1e-5
    want = oracle.knn_pool_backward(g["x"], g["knn_idx_pad"], g[f"{mode}_gy"], mode, g["weights"] if mode == "gaussian" else None)
    assert np.abs(dx.cpu().numpy() - want).max() < 1e-5


def test_pooling_layer_is_differentiable_and_bf16():
    """The module: gradients flow through forward() and forward_points(); bf16 activations give the float32 result to bf16 rounding."""
    from fovi_b200.coords import get_in_out_coords
    from fovi_b200.knn import KNNPoolingLayer
    ic, oc, _ = get_in_out_coords(24, 16, 1.0, 2, auto_match_cart_resources=0)
    pool = KNNPoolingLayer(9, ic, oc, mode="avg", device="cuda")
    rs = np.random.RandomState(2)
    x = rs.standard_normal((2, 8, ic.shape[0])).astype(np.float32)
    gy = rs.standard_normal((2, 8, oc.shape[0])).astype(np.float32)
    xt = torch.from_numpy(x).cuda().requires_grad_(True)
    pool(xt).backward(torch.from_numpy(gy).cuda())
    want = oracle.knn_pool_backward(x, pool.knn_indices_pad_token.numpy(), gy, "avg")
    assert np.abs(xt.grad.cpu().numpy() - want).max() < 1e-5
    xb = torch.from_numpy(x).cuda().permute(0, 2, 1).contiguous().to(torch.bfloat16).requires_grad_(True)
    pool.forward_points(xb).backward(torch.from_numpy(gy).cuda().permute(0, 2, 1).contiguous().to(torch.bfloat16))
    assert xb.grad.dtype == torch.bfloat16
    got = xb.grad.float().permute(0, 2, 1).cpu().numpy()
    assert np.abs(got - want).max() < 3e-2 * max(1.0, np.abs(want).max())
    with torch.no_grad():
        assert pool(torch.from_numpy(x).cuda()).grad_fn is None
