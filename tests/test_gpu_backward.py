"""GPU: gradients of KNNConvLayer (both contractions run on the forward tensor-core kernel) against the gradients the
reference's autograd produced on CPU in float32 (tests/golden/backward_small.npz) and against the oracle's backward."""
import numpy as np
import pytest
import torch

from conftest import kaiming_weight
from oracle import fovi_oracle as oracle

pytestmark = [pytest.mark.gpu, pytest.mark.autograd]
TOL = 1e-2          # relative L2, bf16 operands with float32 accumulation vs float32 reference


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


class _Pts:
    def __init__(self, n):
        self.shape = (n, 2)
        self.dtype = torch.float32


def _layer(g, c_in, c_out, bias=True):
    from fovi_b200.knn import KNNConvLayer
    n_in = int(g["n_in"])
    return KNNConvLayer(c_in, c_out, g["knn_idx"].shape[0], _Pts(n_in), _Pts(g["knn_idx"].shape[1]), device="cuda", bias=bias,
                        tables_override=dict(knn_indices=g["knn_idx"], tap=g["tap"], V=int(g["V"])))


def test_gradients_match_reference_autograd(golden):
    g = golden("backward_small.npz")
    V, n_in = int(g["V"]), int(g["n_in"])
    rs = np.random.RandomState(int(g["seed"]))
    w = kaiming_weight(rs, 32, 16, V)
    b = (0.1 * rs.standard_normal(32)).astype(np.float32)
    x = rs.standard_normal((5, 16, n_in)).astype(np.float32)
    gy = rs.standard_normal((5, 32, g["knn_idx"].shape[1])).astype(np.float32)
    layer = _layer(g, 16, 32)
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(w))
        layer.bias.copy_(torch.from_numpy(b))
    xt = torch.from_numpy(x).cuda().requires_grad_(True)
    y = layer(xt)
    assert y.requires_grad and rel_l2(y.detach().cpu().numpy(), g["y"]) < TOL
    y.backward(torch.from_numpy(gy).cuda())
    layer.plan.check()
    assert rel_l2(xt.grad.cpu().numpy(), g["dX"]) < TOL
    assert rel_l2(layer.weight.grad.cpu().numpy(), g["dW"]) < TOL
    assert rel_l2(layer.bias.grad.cpu().numpy(), g["dbias"]) < 1e-5
    assert layer.weight.grad.shape == layer.weight.shape and xt.grad.shape == xt.shape


def test_first_layer_weight_gradient(golden):
    """A 3-channel first layer (pair-layout forward): its weight gradient runs as one GEMM per output point (columns =
    neighbour x channel, contraction over the batch) followed by a scatter-add onto the taps; its input needs no gradient."""
    g = golden("config1.npz")
    V, n_in = int(g["V"]), int(g["n_in"])
    n_out = g["knn_idx_pad"].shape[1]
    rs = np.random.RandomState(3)
    w = kaiming_weight(rs, 64, 3, V)
    x = rs.standard_normal((70, 3, n_in)).astype(np.float32)          # 70 rows: the batch is padded to 128 for the contraction
    gy = rs.standard_normal((70, 64, n_out)).astype(np.float32)
    from fovi_b200.knn import KNNConvLayer
    layer = KNNConvLayer(3, 64, 49, _Pts(n_in), _Pts(n_out), device="cuda",
                         tables_override=dict(knn_indices=g["knn_idx"], tap=g["tap"], V=V))
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(w))
    y = layer(torch.from_numpy(x).cuda())
    y.backward(torch.from_numpy(gy).cuda())
    _, dW, _ = oracle.knnconv_backward(x[:8], g["knn_idx_pad"], g["tap"].astype(np.int64), V, w, gy[:8])
    # the oracle on 8 rows is the check of a second, smaller run (the full batch would take minutes in NumPy)
    layer.weight.grad = None
    y8 = layer(torch.from_numpy(x[:8]).cuda())
    y8.backward(torch.from_numpy(gy[:8]).cuda())
    assert rel_l2(layer.weight.grad.cpu().numpy(), dW) < TOL
    assert layer.grad_plans._few is not None                        # the per-point path ran
    assert layer.grad_plans.dw_plan(64)[0].n_out > V                # the per-tap path would cut its 3800-entry lists
    with pytest.raises(NotImplementedError):
        xt = torch.from_numpy(x[:8]).cuda().requires_grad_(True)
        layer(xt).sum().backward()


def test_optimizer_steps_reduce_a_regression_loss(golden):
    g = golden("backward_small.npz")
    n_in, n_out = int(g["n_in"]), g["knn_idx"].shape[1]
    torch.manual_seed(0)
    layer = _layer(g, 16, 32)
    teacher = _layer(g, 16, 32)
    x = torch.randn(64, 16, n_in, device="cuda")
    with torch.no_grad():
        target = teacher(x).float()
    opt = torch.optim.Adam(layer.parameters(), lr=0.01)
    losses = []
    for _ in range(20):
        opt.zero_grad()
        loss = ((layer(x).float() - target) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < 0.7 * losses[0], losses
    assert y_is_fresh(layer, x)


def y_is_fresh(layer, x):
    """The packed copy of the weights follows the optimizer's in-place updates."""
    with torch.no_grad():
        a = layer(x)
        layer.refresh_weights()
        b = layer(x)
    return torch.equal(a, b)


def test_stack_trains_in_the_kernel_layout():
    """KNNConvStack under autograd (channels-last between layers, ReLU fused) against the same layers called one by one
    with torch's ReLU between them."""
    from fovi_b200.coords import get_in_out_coords
    from fovi_b200.knn import KNNConvLayer, KNNConvStack
    torch.manual_seed(1)
    ic, oc, cart = get_in_out_coords(24, 16, 1.0, 2, auto_match_cart_resources=0)
    _, oc2, _ = get_in_out_coords(oc.resolution, 16, 1.0, 1, auto_match_cart_resources=0)
    layers = [KNNConvLayer(3, 16, 25, ic, oc, device="cuda", ref_frame_side_length=5, bias=True),
              KNNConvLayer(16, 32, 9, oc, oc2, device="cuda", ref_frame_side_length=3, bias=True),
              KNNConvLayer(32, 64, 9, oc2, oc2, device="cuda", ref_frame_side_length=3, bias=False)]
    stack = KNNConvStack(layers)
    x = torch.randn(6, 3, ic.shape[0], device="cuda")
    gy = torch.randn(6, 64, oc2.shape[0], device="cuda")

    y = stack(x)
    assert y.requires_grad and y.shape == gy.shape
    y.backward(gy)
    got = [p.grad.clone() for p in stack.parameters()]
    for p in stack.parameters():
        p.grad = None
    h = x
    for i, L in enumerate(layers):
        h = L(h if i == 0 else h.to(torch.bfloat16))
        if i < 2:
            h = torch.relu(h)
    assert rel_l2(y.detach().float().cpu().numpy(), h.detach().float().cpu().numpy()) < 1e-2
    h.float().backward(gy)
    for a, p in zip(got, stack.parameters()):
        assert rel_l2(a.float().cpu().numpy(), p.grad.float().cpu().numpy()) < 3e-2
    with torch.no_grad():
        y2 = stack(x)
    assert not y2.requires_grad and rel_l2(y2.float().cpu().numpy(), y.detach().float().cpu().numpy()) < 1e-2


@pytest.mark.parametrize("shape,perm,dtype", [
    ((70, 225, 64), (0, 2, 1), torch.bfloat16),     # channels-last activations seen as [B, C, N]: channels fast, paired accesses
    ((70, 64, 225), (0, 1, 2), torch.float32),      # [B, C, N] contiguous: points fast, odd extent -> scalar kernel
    ((33, 40, 6), (0, 1, 2), torch.float32),        # small, even fast extent, float32 pairs
    ((5, 7, 3), (0, 2, 1), torch.bfloat16),         # everything odd
])
def test_batch_to_inner_layouts(shape, perm, dtype):
    from fovi_b200 import ops
    torch.manual_seed(0)
    x = torch.randn(shape, device="cuda").to(dtype).permute(*perm)            # logical [B, I, J] with some strides
    B, I, J = x.shape
    bp, jp = -(-B // 64) * 64, J + 3
    y = ops.batch_to_inner(x, jp=jp, bp=bp)
    want = torch.zeros((I, jp, bp), dtype=torch.bfloat16, device="cuda")
    want[:, :J, :B] = x.permute(1, 2, 0).to(torch.bfloat16)
    assert torch.equal(y, want)


@pytest.mark.parametrize("shape,dtype", [((1000, 37, 64), torch.bfloat16), ((3, 5, 6), torch.float32), ((70000, 2), torch.float32)])
def test_column_sum(shape, dtype):
    from fovi_b200 import ops
    torch.manual_seed(2)
    x = torch.randn(shape, device="cuda").to(dtype)
    got = ops.column_sum(x)
    want = x.double().reshape(-1, shape[-1]).sum(0)
    assert got.dtype == torch.float32 and got.shape == (shape[-1],)
    scale = float(x.double().abs().reshape(-1, shape[-1]).sum(0).max())
    assert float((got.double() - want).abs().max()) <= 1e-5 * scale


def test_float32_layer_gradients_match_reference_autograd(golden):
    """precision='fp32': forward and both gradient contractions run on the exact float32 kernel; against the reference's
    autograd in float32 the agreement is at float32 rounding, not at bf16's."""
    from fovi_b200.knn import KNNConvLayer
    g = golden("backward_small.npz")
    V, n_in = int(g["V"]), int(g["n_in"])
    rs = np.random.RandomState(int(g["seed"]))
    w = kaiming_weight(rs, 32, 16, V)
    b = (0.1 * rs.standard_normal(32)).astype(np.float32)
    x = rs.standard_normal((5, 16, n_in)).astype(np.float32)
    gy = rs.standard_normal((5, 32, g["knn_idx"].shape[1])).astype(np.float32)
    layer = KNNConvLayer(16, 32, g["knn_idx"].shape[0], _Pts(n_in), _Pts(g["knn_idx"].shape[1]), device="cuda", bias=True, precision="fp32",
                         tables_override=dict(knn_indices=g["knn_idx"], tap=g["tap"], V=V))
    with torch.no_grad():
        layer.weight.copy_(torch.from_numpy(w))
        layer.bias.copy_(torch.from_numpy(b))
    xt = torch.from_numpy(x).cuda().requires_grad_(True)
    y = layer(xt)
    assert y.requires_grad and rel_l2(y.detach().cpu().numpy(), g["y"]) < 1e-5
    y.backward(torch.from_numpy(gy).cuda())
    assert rel_l2(xt.grad.cpu().numpy(), g["dX"]) < 1e-5
    assert rel_l2(layer.weight.grad.cpu().numpy(), g["dW"]) < 1e-5
    assert rel_l2(layer.bias.grad.cpu().numpy(), g["dbias"]) < 1e-5
    # parameters only (a plain input): the result still carries the graph
    layer.weight.grad = None
    y2 = layer(torch.from_numpy(x).cuda())
    assert y2.grad_fn is not None
    y2.backward(torch.from_numpy(gy).cuda())
    assert rel_l2(layer.weight.grad.cpu().numpy(), g["dW"]) < 1e-5


def test_float32_first_layer_trains():
    """A 3-channel float32 layer built from its own tables: gradients against the oracle's backward (float64)."""
    from fovi_b200.coords import get_in_out_coords
    from fovi_b200.knn import KNNConvLayer
    ic, oc, _ = get_in_out_coords(20, 16, 1.0, 2, auto_match_cart_resources=0)
    layer = KNNConvLayer(3, 16, 9, ic, oc, device="cuda", ref_frame_side_length=3, precision="fp32", bias=True)
    rs = np.random.RandomState(5)
    x = rs.standard_normal((3, 3, ic.shape[0])).astype(np.float32)
    gy = rs.standard_normal((3, 16, oc.shape[0])).astype(np.float32)
    xt = torch.from_numpy(x).cuda().requires_grad_(True)
    layer(xt).backward(torch.from_numpy(gy).cuda())
    idx = layer.knn_indices_pad_token.numpy().astype(np.int64)
    V = layer.ref_coords.shape[0]
    dX, dW, db = oracle.knnconv_backward(x.astype(np.float64), idx, layer.tap.numpy().astype(np.int64), V,
                                         layer.weight.detach().cpu().numpy().astype(np.float64), gy.astype(np.float64))
    assert rel_l2(xt.grad.cpu().numpy(), dX) < 1e-5 and rel_l2(layer.weight.grad.cpu().numpy(), dW) < 1e-5
    assert rel_l2(layer.bias.grad.cpu().numpy(), db) < 1e-5
