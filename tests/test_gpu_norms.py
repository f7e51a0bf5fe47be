"""GPU: the per-sample norm layers and 'gaussian' pooling against outputs recorded from the reference's own classes
(tests/golden/norms_small.npz) and against the oracle."""
import numpy as np
import pytest
import torch

from oracle import fovi_oracle as oracle

pytestmark = pytest.mark.gpu


def test_norm_layers_match_reference(golden):
    from fovi_b200 import norm
    g = golden("norms_small.npz")
    B, C, N = (int(v) for v in g["x_shape"])
    x = (np.random.RandomState(int(g["seed"])).standard_normal((B, C, N)) * 1.5 + 0.3).astype(np.float32)
    xd = torch.from_numpy(x).cuda()
    for name, cls, wshape in (("channel", norm.KNNChannelNorm, (C,)), ("coord", norm.KNNCoordNorm, (N,)), ("layer", norm.KNNLayerNorm, (C, N)),
                              ("group", norm.KNNGroupNorm, (C,))):
        layer = cls(N, C, device="cuda")
        assert sorted(layer.state_dict().keys()) == ["bias", "weight"] and tuple(layer.weight.shape) == wshape
        layer.load_state_dict({"weight": torch.from_numpy(g[f"{name}_w"]), "bias": torch.from_numpy(g[f"{name}_b"])})
        if name == "group":
            assert layer.num_groups == int(g["group_groups"])
        with torch.no_grad():
            y = layer(xd)
            assert np.abs(y.cpu().numpy() - g[f"{name}_out"]).max() < 1e-5, name                 # float32 in, float32 out
            # channels-last layout, bf16 in and out, ReLU fused: the oracle on the bf16-rounded input, rounded the same way
            xb = xd.to(torch.bfloat16).permute(0, 2, 1).contiguous()
            yp = layer.forward_points(xb, relu=True)
            ref = oracle.knn_norm(xb.float().permute(0, 2, 1).cpu().numpy(), name, g[f"{name}_w"], g[f"{name}_b"], eps=layer.eps,
                                  groups=int(g[f"{name}_groups"]))
            ref = np.maximum(ref, 0)
            got = yp.float().permute(0, 2, 1).cpu().numpy()
            assert yp.dtype == torch.bfloat16 and np.abs(got - ref).max() < 2e-2 * max(1.0, np.abs(ref).max()), name
        with torch.enable_grad():          # under autograd: the reference's torch calls, same numbers, with gradients
            xg = xd.clone().requires_grad_(True)
            yg = layer(xg)
            assert yg.grad_fn is not None and np.abs(yg.detach().cpu().numpy() - g[f"{name}_out"]).max() < 1e-5, name
            yg.square().sum().backward()
            assert xg.grad is not None and layer.weight.grad is not None and torch.isfinite(xg.grad).all()
            layer.weight.grad = layer.bias.grad = None
    assert norm.find_valid_num_groups(24, 32) == 6 and norm.find_valid_num_groups(96, 32) == 24 and norm.find_valid_num_groups(7, 32) == 1
    assert isinstance(norm.get_norm("layer_chan", N, C), norm.KNNChannelNorm) and isinstance(norm.get_norm("force_batch", N, C), norm.KNNBatchNorm)
    assert norm.get_norm("none", N, C) is None
    with pytest.raises(NotImplementedError):
        norm.get_norm("instance", N, C)


class _Pts:
    def __init__(self, n):
        self.shape = (n, 2)
        self.dtype = torch.float32


def test_gaussian_pooling_matches_reference(golden):
    from fovi_b200 import ops
    g = golden("norms_small.npz")
    n_in = int(g["pool_n_in"])
    plan = ops.KnnPoolPlan(g["pool_knn_idx_pad"], n_in)
    plan.set_weights(g["pool_weights"])
    x = torch.from_numpy(g["pool_x"]).cuda()
    y = plan.forward(x, "gaussian").cpu().numpy()
    assert np.allclose(y, g["pool_out"], rtol=1e-5, atol=1e-6, equal_nan=True)
    yb = plan.forward(x.permute(0, 2, 1).contiguous(), "gaussian", ops.ACT_BNC).permute(0, 2, 1).cpu().numpy()
    assert np.allclose(yb, g["pool_out"], rtol=1e-5, atol=1e-6, equal_nan=True)
    assert np.allclose(oracle.knn_pool_weighted(g["pool_x"], g["pool_knn_idx_pad"], g["pool_weights"]), g["pool_out"], rtol=1e-5, atol=1e-6)
    # the module computes the same weights from the neighbour distances
    from fovi_b200.knn import KNNPoolingLayer
    layer = KNNPoolingLayer.__new__(KNNPoolingLayer)
    torch.nn.Module.__init__(layer)
    layer.knn_distances, layer.gauss_sigma = torch.from_numpy(g["pool_distances"]), float(g["pool_sigma"])
    assert np.allclose(layer._compute_gaussian_weights().numpy(), g["pool_weights"], rtol=1e-6, atol=1e-8)


def test_alexnet_block_with_per_sample_norm():
    """conv -> layer norm -> ReLU -> pool on the kernels' layout equals the same steps done one by one."""
    from fovi_b200.alexnet import KNNAlexNetBlock
    from fovi_b200 import ops
    torch.manual_seed(0)
    blk = KNNAlexNetBlock(3, 32, 9, 16, 1.0, 20, 2, norm_type="channel", pool=True, pool_k=4, device="cuda", ref_frame_mult=1).eval()
    with torch.no_grad():
        blk.norm.weight.uniform_(0.5, 1.5); blk.norm.bias.normal_(0, 0.2)
        x = torch.randn(5, 3, blk.in_coords.shape[0], device="cuda")
        assert blk.points_path
        y = blk(x)
        h = blk.conv(x)                                              # [B, C, N] float32 (bf16 tensor-core result)
        ref = oracle.knn_norm(h.to(torch.bfloat16).float().cpu().numpy(), "channel", blk.norm.weight.cpu().numpy(), blk.norm.bias.cpu().numpy(), eps=blk.norm.eps)
        ref = torch.from_numpy(np.maximum(ref, 0)).to(torch.bfloat16).cuda()
        ref = blk.pool(ref)
    assert y.shape == ref.shape
    assert float((y.float() - ref.float()).abs().max()) < 3e-2 * max(1.0, float(ref.float().abs().max()))
