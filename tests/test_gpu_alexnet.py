"""GPU: the shipped foveated AlexNet (conv -> batch norm -> ReLU -> max pool blocks, average pooling, classifier) on the
kernels against the outputs the reference model produced on CPU in float32 with the same parameters."""
import numpy as np
import pytest
import torch

from conftest import ALEXNET_SHIPPED, seed_alexnet

pytestmark = pytest.mark.gpu


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="module")
def net():
    from fovi_b200.alexnet import KNNAlexNet
    m = KNNAlexNet(n_classes=10, device="cuda", **ALEXNET_SHIPPED)
    seed_alexnet(m, 300)
    return m.eval()


def test_point_counts_and_state_dict_names(net, golden):
    g = golden("alexnet_shipped.npz")
    counts = [net.layers[0].in_coords.shape[0]] + [L.out_coords.shape[0] for L in net.layers]
    assert counts == list(g["n_points"])
    names = set(net.state_dict().keys())
    for i in range(5):
        for leaf in ("conv.weight", "norm.weight", "norm.bias", "norm.running_mean", "norm.running_var", "norm.num_batches_tracked"):
            assert f"layers.{i}.{leaf}" in names
    assert {"classifier.weight", "classifier.bias"} <= names
    assert not any("conv.bias" in n for n in names)          # the reference blocks build their convs without bias


def test_blocks_and_logits_match_reference(net, golden):
    g = golden("alexnet_shipped.npz")
    x = np.random.RandomState(int(g["x_seed"])).standard_normal((3, 3, int(g["n_points"][0]))).astype(np.float32)
    assert net.points_path
    h = torch.from_numpy(x).cuda()
    for i, L in enumerate(net.layers):          # block by block, each fed the previous block's own (bf16-rounded) output
        h = L(h)
        ref = g[f"layer{i}_out_b0"]
        assert h.shape[1:] == ref.shape
        assert rel_l2(h[0].float().cpu().numpy(), ref) < 2e-2, i     # bf16 activations through up to six stages
    logits = net(torch.from_numpy(x).cuda()).float().cpu().numpy()
    assert logits.shape == (3, 10)
    assert rel_l2(logits, g["logits"]) < 2e-2
    feats = net.forward_points(__import__("fovi_b200").ops.pack_points(torch.from_numpy(x).cuda(), net.layers[0].conv.plan), 3)
    assert rel_l2(feats.permute(0, 2, 1).float().cpu().numpy(), g["features"]) < 2e-2


def test_first_block_alone_is_within_the_single_layer_bar(net, golden):
    g = golden("alexnet_shipped.npz")
    x = np.random.RandomState(int(g["x_seed"])).standard_normal((3, 3, int(g["n_points"][0]))).astype(np.float32)
    y = net.layers[0](torch.from_numpy(x).cuda())
    assert rel_l2(y[0].cpu().numpy(), g["layer0_out_b0"]) < 1e-2


def test_folded_operands_follow_parameter_updates(net):
    b = net.layers[2]
    wt0, bias0 = b.folded_operands()
    assert b.folded_operands()[0] is wt0                      # cached
    with torch.no_grad():
        b.norm.running_var.mul_(4.0)
    wt1, _ = b.folded_operands()
    assert wt1 is not wt0
    np.testing.assert_allclose(wt1.float().cpu().numpy(), 0.5 * wt0.float().cpu().numpy(), rtol=2e-2, atol=1e-6)
    with torch.no_grad():
        b.norm.running_var.div_(4.0)


def test_reloaded_parameters_reach_the_kernel(net):
    """Forward, load other batch-norm statistics and weights, forward again: the result is that of a block built fresh
    with the new parameters (the first block's plan is grouped, so its bias is repeated per member on the way in)."""
    from fovi_b200.alexnet import KNNAlexNet
    x = torch.randn(3, 3, net.layers[0].in_coords.shape[0], device="cuda")
    blk = net.layers[0]
    assert blk.conv.plan.group > 1
    y_old = blk(x).clone()
    old_state = {k: v.clone() for k, v in net.state_dict().items()}
    other = KNNAlexNet(n_classes=10, device="cuda", **ALEXNET_SHIPPED)
    seed_alexnet(other, 301)
    other.eval()
    want = other.layers[0](x)
    for _ in range(3):                                    # several refolds: freed temporaries get their addresses reused
        net.load_state_dict(other.state_dict())
        got = blk(x)
        assert torch.equal(got, want)
        net.load_state_dict(old_state)
        assert torch.equal(blk(x), y_old)
    assert not torch.equal(want, y_old)


def test_training_mode_is_refused(net):
    net.train()
    try:
        with pytest.raises(RuntimeError):
            net(torch.zeros(1, 3, net.layers[0].in_coords.shape[0], device="cuda"))
    finally:
        net.eval()


def test_foveated_alexnet_equals_sampler_then_network(net):
    from conftest import synth_images
    from fovi_b200.alexnet import FoveatedAlexNet
    from fovi_b200.sensing import RetinalTransform
    rt = RetinalTransform(resolution=64, start_res=256, fov=16, cmf_a=0.5, style="isotropic", sampler="grid_nn", fixation_size=256,
                          auto_match_cart_resources=1, device="cuda")
    assert len(rt.sampler.coords) == net.layers[0].in_coords.shape[0]
    B, F = 3, 4
    img = torch.from_numpy(synth_images(3, (B, 3, 256, 256))).cuda()
    fix = torch.from_numpy((0.25 + 0.5 * np.random.RandomState(4).random_sample((B, F, 2))).astype(np.float32)).cuda()
    model = FoveatedAlexNet(rt, net)
    per_fix = model(img, fix)
    assert per_fix.shape == (B, F, 10)
    # the reference's order of operations: one sensor call per fixation, the network on the '(f b)' batch
    x_fixs = torch.stack([rt(img, fix[:, f]) for f in range(F)], 1)                         # [B,F,3,N]
    flat = x_fixs.permute(1, 0, 2, 3).reshape(F * B, 3, -1)
    ref = net(flat).view(F, B, -1).permute(1, 0, 2)
    # the fused route rounds the sensor output to bf16 exactly as pack_points does, so the two agree to rounding of the classifier
    assert rel_l2(per_fix.cpu().numpy(), ref.float().cpu().numpy()) < 1e-3
    np.testing.assert_allclose(model(img, fix, fix_agg="mean").cpu().numpy(), per_fix.mean(1).cpu().numpy(), rtol=1e-6, atol=1e-6)


def _torch_block(x, conv, norm, pool, P, prefix):
    """The reference's formulation of one block in float32 torch ops (gather + tap-indexed weights + linear map,
    fovi/arch/knn.py:484-557; BatchNorm1d with batch statistics; ReLU; nan-aware pooling, knn.py:345-371) on the parameter
    tensors P[prefix + ...]."""
    import torch.nn.functional as F
    idx = conv.knn_indices_pad_token.to(x.device)                       # [K, n_out], pad == n_in
    tap = conv.tap.to(x.device)                                          # [n_out, K]
    V = conv.ref_coords.shape[0]
    co, ci = conv.out_channels, conv.in_channels
    xp = torch.cat([x, torch.zeros_like(x[:, :, :1])], 2)
    g = xp[:, :, idx]                                                    # [B, ci, K, n_out]
    w = P[prefix + "conv.weight"].view(co, ci, V)[:, :, tap]             # [co, ci, n_out, K]
    y = torch.einsum("bckn,ocnk->bon", g, w)
    if prefix + "conv.bias" in P:
        y = y + P[prefix + "conv.bias"][None, :, None]
    if norm is not None:
        y = F.batch_norm(y, None, None, P[prefix + "norm.weight"], P[prefix + "norm.bias"], True, 0.0, norm.eps)
    y = torch.relu(y)
    if pool is not None:
        pidx = pool.knn_indices_pad_token.to(x.device)
        yp = torch.cat([y, torch.full_like(y[:, :, :1], float("nan"))], 2)[:, :, pidx]     # [B, C, K, n_out]
        yp = torch.where(torch.isnan(yp), torch.full_like(yp, -float("inf")), yp)
        y = yp.max(2).values
    return y


@pytest.mark.autograd
def test_network_trains_with_batch_statistics():
    """KNNAlexNet in training mode: convolution gradients from the tensor-core kernels, batch norm with batch statistics,
    max pooling with its own gradient; the first step's gradients against torch autograd through the reference's
    formulation of the same network, and a few optimizer steps reduce the loss."""
    from fovi_b200.alexnet import KNNAlexNet
    torch.manual_seed(0)
    net = KNNAlexNet(in_res=24, in_channels=3, features_per_layer=[16, 32], stride_per_layer=[2, 1], pool_after=[0], k_per_layer=[9, 9],
                     n_classes=5, out_res=None, auto_match_cart_resources=0, fov=16.0, cmf_a=1.0, norm_type="batch", device="cuda").train()
    n0 = net.layers[0].in_coords.shape[0]
    x = torch.randn(12, 3, n0, device="cuda")
    target = torch.randint(0, 5, (12,), device="cuda")
    P = {n: p.detach().clone().float().requires_grad_(True) for n, p in net.named_parameters()}

    def ref_forward():
        h = x
        for i, blk in enumerate(net.layers):
            h = _torch_block(h, blk.conv, blk.norm, blk.pool, P, f"layers.{i}.")
        return torch.nn.functional.linear(h.reshape(h.shape[0], -1), P["classifier.weight"], P["classifier.bias"])

    loss = torch.nn.functional.cross_entropy(net(x), target)
    loss.backward()
    loss_ref = torch.nn.functional.cross_entropy(ref_forward(), target)
    loss_ref.backward()
    assert abs(loss.item() - loss_ref.item()) < 2e-2 * max(1.0, abs(loss_ref.item()))
    for name, p in net.named_parameters():
        q = P[name]
        assert p.grad is not None and torch.isfinite(p.grad).all(), name
        err = float((p.grad.float() - q.grad).norm() / q.grad.norm().clamp_min(1e-12))
        assert err < 1e-1, (name, err)     # bf16 activations through batch norm and a max pool, whose argmax can switch under bf16 rounding
    opt = torch.optim.SGD(net.parameters(), lr=0.05, momentum=0.9)
    first = None
    for _ in range(8):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(net(x), target)
        loss.backward()
        opt.step()
        first = loss.item() if first is None else first
    assert loss.item() < 0.7 * first
    net.eval()
    with torch.no_grad():
        assert net(x).shape == (12, 5)       # the inference path (folded running statistics) still runs after training
