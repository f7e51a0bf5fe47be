"""GPU: the module-level API (RetinalTransform / KNNConvLayer / patch embedding / KNNConvStack), built
from this package's own geometry and tables, against the outputs recorded from the reference."""
import numpy as np
import pytest
import torch

from conftest import synth_images, kaiming_weight
from oracle import fovi_oracle as oracle

pytestmark = pytest.mark.gpu
f32 = np.float32


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def test_config1_sensor_plus_knnconv_modules(golden):
    from fovi_b200.sensing import RetinalTransform
    from fovi_b200.knn import KNNConvLayer
    g = golden("config1.npz")
    rt = RetinalTransform(resolution=64, start_res=224, fov=16, cmf_a=2.78, style="isotropic", sampler="grid_bilinear",
                          fixation_size=224, auto_match_cart_resources=1, device="cuda")
    assert rt.resolution == 44 and len(rt.sampler.coords) == 3975
    x = torch.from_numpy(synth_images(0, (8, 3, 224, 224))).cuda()
    y = rt(x, None)
    assert y.shape == (8, 3, 3975) and np.array_equal(y.cpu().numpy(), g["sampled"])        # bit-exact vs the reference
    c = rt.sampler.coords
    w = kaiming_weight(np.random.RandomState(1), 64, 3, 49)
    for precision, tol in (("fp32", 1e-5), ("bf16", 1e-2)):
        layer = KNNConvLayer(3, 64, 49, c, c, device="cuda", ref_frame_side_length=7, bias=False, precision=precision)
        assert np.array_equal(layer.knn_indices.numpy(), g["knn_idx"]) and np.array_equal(layer.tap.numpy(), g["tap"])
        assert tuple(layer.weight.shape) == (64, 3 * 49) and layer.bias is None
        layer.weight.data.copy_(torch.from_numpy(w))
        out = layer(y)
        assert out.shape == (8, 64, 3975) and out.dtype == torch.float32
        assert rel_l2(out[0].cpu().numpy(), g["conv_out_b0"]) < tol
        np.testing.assert_allclose(out.double().sum((1, 2)).cpu().numpy(), g["conv_out_sum"], rtol=5e-3, atol=5e-2)
    rf = layer.local_rf
    assert rf.shape == (3975, 49, 49) and float(rf.sum()) == 3975 * 49
    # weight edits are picked up (the packed copy is rebuilt): tracked in-place updates automatically,
    # writes through .data after refresh_weights()
    with torch.no_grad():
        layer.weight.mul_(2)
    assert rel_l2(layer(y)[0].cpu().numpy(), 2 * g["conv_out_b0"]) < 1e-2
    layer.weight.data.mul_(0.5)
    layer.refresh_weights()
    assert rel_l2(layer(y)[0].cpu().numpy(), g["conv_out_b0"]) < 1e-2
    layer.load_state_dict({"weight": torch.from_numpy(3 * w)})
    assert rel_l2(layer(y)[0].cpu().numpy(), 3 * g["conv_out_b0"]) < 1e-2


def test_multi_fixation_forward_matches_loop(golden):
    from fovi_b200.sensing import RetinalTransform
    g = golden("config2_small.npz")
    rt = RetinalTransform(resolution=64, start_res=256, fov=16, cmf_a=1.0, sampler="grid_bilinear", fixation_size=256, device="cuda")
    x = torch.from_numpy(synth_images(0, (2, 3, 256, 256))).cuda()
    fix = torch.from_numpy(g["fix"]).cuda()
    y = rt(x, fix)                                                     # [B,F,C,N] in one launch
    assert np.array_equal(y.cpu().numpy(), g["a1_bilinear_near_zeros"])
    for f in range(3):                                                 # the reference's per-fixation call pattern
        assert torch.equal(rt(x, fix[:, f]), y[:, f])
    ysz = rt(x, fix, fixation_size=torch.from_numpy(g["sizes"]).cuda())
    assert np.array_equal(ysz.cpu().numpy(), g["a1_bilinear_near_sizes"])
    rt_nn = RetinalTransform(resolution=64, start_res=256, fov=16, cmf_a=1.0, sampler="grid_nn", fixation_size=256, device="cuda")
    assert np.array_equal(rt_nn(x, fix).cpu().numpy(), g["a1_nearest_near_zeros"])


def test_config4_partitioning_patch_embedding(golden):
    from fovi_b200.knn import KNNPartitioningPatchEmbedding
    g = golden("config4_patch_embed_p8.npz")
    pe = KNNPartitioningPatchEmbedding(3, 384, in_res=64, fov=16, cmf_a=2.78, in_cart_res=64, cart_patch_size=8, ref_frame_side_length=16,
                                       max_coord_val="auto", sample_cortex=True, bias=True, transposed=True, device="cuda")
    assert pe._k == g["knn_idx"].shape[0] == 105 and len(pe.out_coords) == 63
    assert np.array_equal(pe.out_coords.cartesian.cpu().numpy(), g["out_cartesian"])
    assert np.array_equal(pe.knn_indices.numpy(), g["knn_idx"]) and np.array_equal(pe.tap.numpy(), g["tap"])
    pe.weight.data.copy_(torch.from_numpy(kaiming_weight(np.random.RandomState(1), 384, 3, 256)))
    pe.bias.data.copy_(torch.from_numpy((0.1 * np.random.RandomState(2).standard_normal(384)).astype(f32)))
    x = torch.from_numpy(synth_images(0, (2, 3, 3975))).cuda()
    out = pe(x)
    assert out.shape == (2, 384, 63)
    assert rel_l2(out.cpu().numpy(), g["out_b2"]) < 1e-2


def test_config3_stack_module_end_to_end(golden):
    """Sensor -> five-layer stack through the module API, tables built by this package."""
    from fovi_b200.coords import auto_match_num_coords, get_in_out_coords
    from fovi_b200.knn import KNNConvLayer, KNNConvStack
    acts = golden("config3_acts_b2.npz")
    chans, strides, ks = [3, 64, 192, 384, 256, 256], [2, 2, 1, 1, 1], [121, 25, 9, 9, 9]
    in_res, cart_res = auto_match_num_coords(16, 1.0, 64, "isotropic", 1)
    rs = np.random.RandomState(1)
    layers = []
    for i in range(5):
        ic, oc, out_cart = get_in_out_coords(in_res, 16, 1.0, strides[i], auto_match_cart_resources=1, in_cart_res=cart_res)
        side = int(np.ceil(2 * np.sqrt(ks[i])))
        L = KNNConvLayer(chans[i], chans[i + 1], ks[i], ic, oc, device="cuda", ref_frame_side_length=side, bias=True)
        L.weight.data.copy_(torch.from_numpy(kaiming_weight(rs, chans[i + 1], chans[i], side * side)))
        layers.append(L)
        in_res, cart_res = oc.resolution, out_cart
    stack = KNNConvStack(layers)
    x = torch.from_numpy(synth_images(0, (2, 3, 4010))).cuda()
    out = stack(x)
    assert out.shape == (2, 256, 225) and out.dtype == torch.float32
    assert rel_l2(out.cpu().numpy(), acts["act4"]) < 1e-2
    out2 = stack(x)
    assert torch.equal(out, out2)
    # value semantics: a later call with the same batch size must not overwrite an earlier result
    keep = out.clone()
    other = stack(torch.from_numpy(synth_images(5, (2, 3, 4010))).cuda())
    assert out.data_ptr() != other.data_ptr() and torch.equal(out, keep) and not torch.equal(other, keep)


def test_cpu_tensors_are_refused(golden):
    from fovi_b200 import ops
    plan = ops.SamplerPlan(golden("sensor_a1.npz")["sampling_grid"])
    with pytest.raises(ValueError, match="no CPU path"):
        ops.sample(plan, torch.zeros(1, 3, 8, 8), torch.zeros(1, 1, 2), torch.zeros(1, 1, 2))


def test_fused_sample_knnconv_call_equals_two_calls(golden):
    from fovi_b200 import ops
    g, s = golden("config1.npz"), golden("sensor_a2p78.npz")
    V = int(g["V"])
    splan = ops.SamplerPlan(s["sampling_grid"])
    cplan = ops.KnnConvPlan(g["knn_idx_pad"], g["tap"], int(g["n_in"]), V, 3, 64)
    wt = cplan.pack_weights(torch.from_numpy(kaiming_weight(np.random.RandomState(1), 64, 3, V)).cuda())
    B, F = 5, 3
    x = torch.from_numpy(synth_images(2, (B, 3, 224, 224))).cuda()
    fix = torch.from_numpy((0.3 + 0.4 * np.random.RandomState(3).random_sample((B, F, 2))).astype(f32)).cuda()
    hw = torch.full((B, F, 2), 224.0, device="cuda")
    y, inter = ops.sample_knnconv_fused(splan, cplan, x, fix, hw, wt, relu=True, out_dtype=torch.float32)
    xin = ops.sample(splan, x, fix, hw, layout=ops.OUT_FB_PAIRS)
    want = cplan.forward(xin, wt, relu=True, out_dtype=torch.float32, batch=B * F)
    cplan.check()
    assert y.shape == (B * F, 3975, 64) and torch.equal(y, want)
    # ... and against the oracle: sampler bit-exact, rounded to bf16 like the intermediate, then the layer on bf16 operands
    w = kaiming_weight(np.random.RandomState(1), 64, 3, V)
    xs = oracle.retinal_sample(x.cpu().numpy(), s["sampling_grid"], fix.cpu().numpy(), hw.cpu().numpy())            # [B,F,C,N]
    xs = torch.from_numpy(xs).to(torch.bfloat16).float().numpy().transpose(1, 0, 2, 3).reshape(B * F, 3, -1)[:4]
    wr = torch.from_numpy(w).to(torch.bfloat16).float().numpy()
    ref = oracle.knnconv_forward_closed_form(xs, g["knn_idx_pad"], g["tap"].astype(np.int64), V, wr, relu=True)
    assert np.abs(y[:4].permute(0, 2, 1).cpu().numpy() - ref).max() < 2e-3 * max(1.0, np.abs(ref).max())
    yb, _ = ops.sample_knnconv_fused(splan, cplan, x, fix, hw, wt, relu=True, out_dtype=torch.float32, row_order="bf")
    assert torch.equal(yb.view(B, F, 3975, 64), y.view(F, B, 3975, 64).permute(1, 0, 2, 3))


@pytest.mark.parametrize("name,kw,train", [
    ("near_eval", dict(norm_dist_from_center=0.25), False),
    ("near_train", dict(norm_dist_from_center=0.25, add_aspect_variation=True, nonrandom_first=True), True),
    ("crop_train", dict(add_aspect_variation=True), True),
])
def test_policy_forward_matches_reference(golden, name, kw, train):
    """The batched policy (one sampler launch for all fixations) returns the reference policy's dictionary bit for bit."""
    from fovi_b200.policies import MultiRandomSaccadePolicy
    from fovi_b200.sensing import RetinalTransform
    g = golden("policy_small.npz")
    rt = RetinalTransform(resolution=64, start_res=256, fov=16, cmf_a=1.0, sampler="grid_bilinear", fixation_size=256, device="cuda")
    pol = MultiRandomSaccadePolicy(rt, n_fixations=4, **kw)
    pol.train(train)
    x = torch.from_numpy(synth_images(7, (3, 3, 256, 256))).cuda()
    np.random.seed(11)
    out = pol(x)
    assert np.array_equal(out["fixations"].cpu().numpy(), g[f"{name}_fixations"])
    assert np.array_equal(out["fixation_sizes"].numpy(), g[f"{name}_sizes"])
    assert np.array_equal(out["fix_deltas"].cpu().numpy(), g[f"{name}_deltas"])
    assert out["x_fixs"].shape == (3, 4, 3, 4010)
    assert np.array_equal(out["x_fixs"].cpu().numpy(), g[f"{name}_x_fixs"])


def test_layer_on_natively_built_tables_matches_oracle(golden):
    """table_builder='native': the layer's own tables feed both the kernel and the oracle."""
    from fovi_b200.coords import get_in_out_coords
    from fovi_b200.knn import KNNConvLayer
    ic, oc, _ = get_in_out_coords(20, 16, 1.0, 2, auto_match_cart_resources=0)
    torch.manual_seed(0)
    layer = KNNConvLayer(8, 32, 9, ic, oc, device="cuda", ref_frame_side_length=3, bias=True, table_builder="native")
    ref_layer = KNNConvLayer(8, 32, 9, ic, oc, device="cuda", ref_frame_side_length=3, bias=True, table_builder="torch")
    assert layer.knn_indices.shape == ref_layer.knn_indices.shape and layer.tap.shape == ref_layer.tap.shape
    x = torch.randn(3, 8, ic.shape[0], device="cuda")
    y = layer(x).cpu().numpy()
    V = layer.ref_coords.shape[0]
    ref = oracle.knnconv_forward(x.cpu().numpy(), layer.knn_indices_pad_token.numpy(), layer.tap.numpy(), V,
                                 layer.weight.detach().cpu().numpy(), layer.bias.detach().cpu().numpy())
    assert rel_l2(y, ref) < 1e-2


def test_front_end_host_pipeline_equals_device_path(golden):
    """run_from_host (pinned host buffers, chunked three-stream pipeline, rows '(b f)') gives the device path's numbers,
    for float32 and bf16 host images; its copy-only mode touches nothing but the copies."""
    from fovi_b200.coords import get_in_out_coords
    from fovi_b200.knn import KNNConvLayer, KNNConvStack
    from fovi_b200.pipeline import FoveatedFrontEnd
    from fovi_b200.sensing import RetinalTransform
    rt = RetinalTransform(resolution=20, start_res=64, fov=16, cmf_a=1.0, sampler="grid_bilinear", fixation_size=64, device="cuda",
                          auto_match_cart_resources=0)
    ic = rt.sampler.coords
    _, oc, _ = get_in_out_coords(20, 16, 1.0, 2, auto_match_cart_resources=0)
    torch.manual_seed(3)
    l0 = KNNConvLayer(3, 64, 9, ic, oc, device="cuda", ref_frame_side_length=3, bias=True)
    l1 = KNNConvLayer(64, 32, 9, oc, oc, device="cuda", ref_frame_side_length=3, bias=True)
    front = FoveatedFrontEnd(rt, KNNConvStack([l0, l1]))
    B, F = 11, 3
    img = torch.from_numpy(synth_images(9, (B, 3, 64, 64))).pin_memory()
    fix = torch.from_numpy((0.2 + 0.6 * np.random.RandomState(2).random_sample((B, F, 2))).astype(f32)).pin_memory()
    out = torch.zeros((B, F, len(oc), 32), dtype=torch.bfloat16).pin_memory()
    for x in (img, img.to(torch.bfloat16).pin_memory()):
        out.zero_()
        front.run_from_host(x, fix, out, chunks=4)
        torch.cuda.synchronize()
        want = front.forward(x.cuda(), fix.cuda()).view(F, B, len(oc), 32).permute(1, 0, 2, 3)
        assert torch.equal(out, want.cpu())
        keep = out.clone()
        front.run_from_host(x, fix, out, chunks=4, kernels=False)        # copies only: the slot buffers still hold the last chunks
        torch.cuda.synchronize()
        assert out.shape == keep.shape
    # the device path returns new memory on every call
    a = front.forward(img.cuda(), fix.cuda()); b = front.forward(img.cuda(), fix.cuda())
    assert a.data_ptr() != b.data_ptr() and torch.equal(a, b)
    rt.sampler.check()
