"""GPU: depthwise and depthwise-separable KNN convolution against outputs produced from the reference layers' own gather,
tap scatter and contraction (tests/golden/depthwise_small.npz) and against the oracle."""
import numpy as np
import pytest
import torch

from oracle import fovi_oracle as oracle

pytestmark = pytest.mark.gpu


class _Pts:
    def __init__(self, n):
        self.shape = (n, 2)
        self.dtype = torch.float32


def rel_max(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def _inputs(g):
    V = int(g["V"])
    rs = np.random.RandomState(int(g["seed"]))
    x = rs.standard_normal((4, 16, int(g["n_in"]))).astype(np.float32)
    w = (rs.standard_normal((16, V, 2)) * 0.2).astype(np.float32)
    b = (0.1 * rs.standard_normal(32)).astype(np.float32)
    pw = (rs.standard_normal((32, 32)) * 0.2).astype(np.float32)
    pb = (0.1 * rs.standard_normal(32)).astype(np.float32)
    return x, w, b, pw, pb


def _make(cls, g, **kw):
    n_in, n_out = int(g["n_in"]), g["knn_idx"].shape[1]
    return cls(16, 32, 9, _Pts(n_in), _Pts(n_out), device="cuda", tables_override=dict(knn_indices=g["knn_idx"], tap=g["tap"], V=int(g["V"])), **kw)


def test_depthwise_matches_reference_steps(golden):
    from fovi_b200.knn import KNNDepthwiseConvLayer, get_knn_conv_layer
    g = golden("depthwise_small.npz")
    x, w, b, _, _ = _inputs(g)
    assert get_knn_conv_layer("dw") is KNNDepthwiseConvLayer
    layer = _make(KNNDepthwiseConvLayer, g, bias=True)
    assert tuple(layer.weight.shape) == (16, int(g["V"]), 2) and sorted(layer.state_dict().keys()) == ["bias", "weight"]
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(w))
        layer.bias.copy_(torch.from_numpy(b))
        y = layer(torch.from_numpy(x).cuda())
    assert y.shape == g["dw_out"].shape
    assert rel_max(y.cpu().numpy(), g["dw_out"]) < 1e-5            # float32 in, float32 accumulate
    # bf16 activations in and out
    with torch.no_grad():
        yb = layer(torch.from_numpy(x).cuda().to(torch.bfloat16))
    xr = torch.from_numpy(x).to(torch.bfloat16).float().numpy()
    ref = oracle.knn_depthwise_forward(xr, g["knn_idx_pad"], g["tap"].astype(np.int64), w, b)
    assert yb.dtype == torch.bfloat16 and rel_max(yb.float().cpu().numpy(), ref) < 1e-2
    # no bias: the layer keeps working and adds nothing
    nb = _make(KNNDepthwiseConvLayer, g, bias=False)
    with torch.no_grad():
        nb.weight.copy_(torch.from_numpy(w))
        y0 = nb(torch.from_numpy(x).cuda())
    assert rel_max(y0.cpu().numpy(), g["dw_out"] - b[None, :, None]) < 1e-5
    with torch.enable_grad():
        assert layer(torch.from_numpy(x).cuda()).grad_fn is not None    # gradients enabled: differentiable (see the gradient test)


def test_depthwise_separable_matches_reference_steps(golden):
    from fovi_b200.knn import KNNDepthwiseSeparableConvLayer
    g = golden("depthwise_small.npz")
    x, w, _, pw, pb = _inputs(g)
    layer = _make(KNNDepthwiseSeparableConvLayer, g, bias=True)
    assert sorted(layer.state_dict().keys()) == ["bias", "dw_conv", "p_conv.bias", "p_conv.weight", "weight"]
    with torch.no_grad():
        layer.dw_conv.copy_(torch.from_numpy(w))
        layer.p_conv.weight.copy_(torch.from_numpy(pw))
        layer.p_conv.bias.copy_(torch.from_numpy(pb))
        y = layer(torch.from_numpy(x).cuda())
    assert y.shape == g["dwsep_out"].shape
    assert rel_max(y.cpu().numpy(), g["dwsep_out"]) < 1e-3          # the pointwise product may run in TF32
    # bf16 activations: the pointwise map runs on the tensor-core kernel (a KNNConv whose points are their own only neighbour)
    with torch.no_grad():
        yb = layer(torch.from_numpy(x).cuda().to(torch.bfloat16))
    assert yb.dtype == torch.bfloat16 and yb.shape == g["dwsep_out"].shape
    err = np.linalg.norm(yb.float().cpu().numpy() - g["dwsep_out"]) / np.linalg.norm(g["dwsep_out"])
    assert err < 1e-2, err
    layer._pw_plan.check()


@pytest.mark.autograd
def test_depthwise_gradients_match_reference_autograd(golden):
    """Input, filter and bias gradients of the depthwise layer, and all four parameter/input gradients of the separable
    layer, against autograd through the reference layers' own steps (float32 scatter-adds: 1e-4; the separable layer's
    pointwise map runs in bf16 on the tensor cores: 1e-2 relative L2)."""
    from fovi_b200.knn import KNNDepthwiseConvLayer, KNNDepthwiseSeparableConvLayer
    g = golden("depthwise_small.npz")
    x, w, b, pw, pb = _inputs(g)
    gy = torch.from_numpy(g["gy"]).cuda()
    rel = lambda a, r: float(np.linalg.norm(a - r) / max(np.linalg.norm(r), 1e-30))  # noqa: E731
    layer = _make(KNNDepthwiseConvLayer, g, bias=True)
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(w)); layer.bias.copy_(torch.from_numpy(b))
    xt = torch.from_numpy(x).cuda().requires_grad_()
    y = layer(xt)
    assert rel_max(y.detach().cpu().numpy(), g["dw_out"]) < 1e-5
    (y * gy).sum().backward()
    assert rel(xt.grad.cpu().numpy(), g["dw_dX"]) < 1e-4
    assert rel(layer.weight.grad.cpu().numpy(), g["dw_dW"]) < 1e-4
    assert rel(layer.bias.grad.cpu().numpy(), g["dw_db"]) < 1e-4
    sep = _make(KNNDepthwiseSeparableConvLayer, g, bias=True)
    with torch.no_grad():
        sep.dw_conv.copy_(torch.from_numpy(w)); sep.p_conv.weight.copy_(torch.from_numpy(pw)); sep.p_conv.bias.copy_(torch.from_numpy(pb))
    keys = sorted(sep.state_dict().keys())
    xt = torch.from_numpy(x).cuda().requires_grad_()
    y = sep(xt)
    assert sorted(sep.state_dict().keys()) == keys                      # the helper layer stays out of the module tree
    assert rel(y.detach().float().cpu().numpy(), g["dwsep_out"]) < 1e-2
    (y * gy).sum().backward()
    assert rel(xt.grad.cpu().numpy(), g["dwsep_dX"]) < 2e-2
    assert rel(sep.dw_conv.grad.cpu().numpy(), g["dwsep_dW"]) < 2e-2
    assert rel(sep.p_conv.weight.grad.cpu().numpy(), g["dwsep_dPW"]) < 1e-2
    assert rel(sep.p_conv.bias.grad.cpu().numpy(), g["dwsep_dPb"]) < 1e-2
