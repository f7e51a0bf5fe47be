"""Generate the golden fixtures in this directory by running the reference
implementation (nblauch/fovi, pure PyTorch) on CPU, and pin the NumPy oracle to it.

Run once, where a checkout of the reference is available:

    python tests/golden/make_golden.py --reference /path/to/fovi-checkout

Nothing at test/bench time imports the reference; the ``.npz`` files written here
travel with the repository instead.  All synthetic inputs come from
``numpy.random.RandomState`` (a frozen bit-stream), so they can be regenerated
bit-identically anywhere; weights are Kaiming-normal by construction
(``N(0,1) * sqrt(2 / fan_in)``, fan_in = Cin*V) and are copied into the reference
layers before their forward is recorded.

What is pinned while generating (the script aborts if any check fails):
  * oracle.transform_sampling_grid / grid_sample == reference sampler, bit-exact
  * oracle.knnconv_forward == reference KNNConvLayer.forward, <= 1e-5 relative
"""
import argparse
import importlib.machinery
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import fovi_oracle as oracle  # noqa: E402

f32 = np.float32


def load_reference(root):
    """Import the reference's hot-path modules without its trainer/CLI dependencies:
    seed ``sys.modules['fovi']`` with an empty package pointing at the checkout, stub two
    plotting/mesh modules the hot path never calls, and import ``fovi.arch.knn`` first."""
    pkg = types.ModuleType("fovi")
    pkg.__path__ = [os.path.join(root, "fovi")]
    pkg.__spec__ = importlib.machinery.ModuleSpec("fovi", None, is_package=True)
    sys.modules["fovi"] = pkg
    for name in ("trimesh", "skimage", "skimage.measure"):
        sys.modules.setdefault(name, types.ModuleType(name))
    sys.modules["skimage.measure"].EllipseModel = object
    sys.modules["skimage"].measure = sys.modules["skimage.measure"]
    import fovi.arch.knn as knn
    import fovi.arch.knnvit as knnvit
    import fovi.sensing.coords as coords
    import fovi.sensing.retina as retina
    import fovi.sensing.policies as policies
    load_reference.policies = policies
    return knn, retina, coords, knnvit


def synth_images(seed, shape):
    return np.random.RandomState(seed).random_sample(shape).astype(f32)


def synth_fixations(seed, B, F, lo=0.25, span=0.5):
    return (lo + span * np.random.RandomState(seed).random_sample((B, F, 2))).astype(f32)


def kaiming_weight(rs, cout, cin, V):
    return (rs.standard_normal((cout, cin * V)) * np.sqrt(2.0 / (cin * V))).astype(f32)


def coords_dict(c, prefix=""):
    d = {
        "cartesian": c.cartesian.numpy(), "polar": c.polar.numpy(), "cortical": c.cortical.numpy(),
        "cartesian_pad": c.cartesian_pad_coords.numpy(), "cortical_pad": c.cortical_pad_coords.numpy(),
        "resolution": np.int64(c.resolution), "fov": np.float64(c.fov), "cmf_a": np.float64(c.cmf_a),
    }
    return {prefix + k: v for k, v in d.items()}


def layer_tables(layer):
    """int32 [K,Nout] pad-token indices, raw indices, uint16 [Nout,K] tap table, V."""
    tap = oracle.tap_table_from_local_rf(layer.local_rf.numpy())
    return {
        "knn_idx": layer.knn_indices.numpy().astype(np.int32),
        "knn_idx_pad": layer.knn_indices_pad_token.numpy().astype(np.int32),
        "tap": tap.astype(np.uint16),
        "V": np.int64(layer.ref_coords.shape[0]),
        "n_in": np.int64(layer.in_coords.shape[0]),
    }


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


ALEXNET_SHIPPED = dict(in_res=64, in_channels=3, features_per_layer=[96, 256, 384, 384, 256], stride_per_layer=[2, 1, 1, 1, 1],
                       pool_after=[0, 1, 4], k_per_layer=[121, 25, 9, 9, 9], out_res=1, auto_match_cart_resources=1, fov=16.0, cmf_a=0.5,
                       norm_type="force_batch", ref_frame_mult=2, sample_cortex=True)


def seed_alexnet(model, seed):
    """Deterministic parameters for a KNNAlexNet (reference or fovi_b200: same module names): Kaiming-normal conv
    weights, and batch-norm affine parameters / running statistics away from their defaults."""
    for i, block in enumerate(model.layers):
        if not hasattr(block, "conv"):
            continue
        rs = np.random.RandomState(seed + i)
        cout, fan = block.conv.weight.shape
        block.conv.weight.data.copy_(torch.from_numpy((rs.standard_normal((cout, fan)) * np.sqrt(2.0 / fan)).astype(f32)))
        block.norm.weight.data.copy_(torch.from_numpy((0.5 + rs.random_sample(cout)).astype(f32)))
        block.norm.bias.data.copy_(torch.from_numpy((0.2 * rs.standard_normal(cout)).astype(f32)))
        block.norm.running_mean.copy_(torch.from_numpy((0.1 * rs.standard_normal(cout)).astype(f32)))
        block.norm.running_var.copy_(torch.from_numpy((0.5 + rs.random_sample(cout)).astype(f32)))
    if getattr(model, "n_classes", None) is not None:
        rs = np.random.RandomState(seed + 100)
        w = model.classifier.weight
        w.data.copy_(torch.from_numpy((rs.standard_normal(tuple(w.shape)) / np.sqrt(w.shape[1])).astype(f32)))
        model.classifier.bias.data.copy_(torch.from_numpy((0.1 * rs.standard_normal(w.shape[0])).astype(f32)))


def alexnet_fixture(save):
    """The shipped foveated AlexNet (config/fovi_alexnet.yaml: base_lowres, a=0.5, 64x64 resources, batch norm) run by the
    reference in evaluation mode on CPU, float32: per-block outputs of sample 0 and the logits."""
    import fovi.arch.knnalexnet as ref_alex
    torch.manual_seed(0)
    net = ref_alex.KNNAlexNet(n_classes=10, device="cpu", **ALEXNET_SHIPPED)
    seed_alexnet(net, 300)
    net.eval()
    n0 = net.layers[0].in_coords.shape[0]
    x = (np.random.RandomState(21).standard_normal((3, 3, n0))).astype(f32)
    out = {"x_seed": np.int64(21), "n_points": np.array([n0] + [L.out_coords.shape[0] for L in net.layers], np.int64)}
    h = torch.from_numpy(x)
    for i, L in enumerate(net.layers):
        h = L(h)
        out[f"layer{i}_out_b0"] = h[0].numpy()
        out[f"layer{i}_sum"] = h.double().sum((1, 2)).numpy()
    out["features"] = h.numpy()
    out["logits"] = net.classifier(h.reshape(h.shape[0], -1)).numpy()
    save("alexnet_shipped.npz", **out)
    print("alexnet point counts", out["n_points"], "logits", out["logits"][0, :4])


def backward_fixture(save, knn):
    """Gradients of the reference KNNConvLayer from its own autograd (CPU, float32) on a small layer, and the oracle's
    backward pinned to them."""
    ic, oc, _ = knn.get_in_out_coords(24, 16, 1.0, 2, style="isotropic", auto_match_cart_resources=0, device="cpu")
    torch.manual_seed(5)
    layer = knn.KNNConvLayer(16, 32, 9, ic, oc, device="cpu", ref_frame_side_length=4, bias=True)
    rs = np.random.RandomState(31)
    V = layer.ref_coords.shape[0]
    w = kaiming_weight(rs, 32, 16, V)
    b = (0.1 * rs.standard_normal(32)).astype(f32)
    x = rs.standard_normal((5, 16, len(ic))).astype(f32)
    g = rs.standard_normal((5, 32, len(oc))).astype(f32)
    with torch.enable_grad():
        layer.weight.data.copy_(torch.from_numpy(w))
        layer.bias.data.copy_(torch.from_numpy(b))
        xt = torch.from_numpy(x).requires_grad_(True)
        y = layer(xt)
        y.backward(torch.from_numpy(g))
    t = layer_tables(layer)
    dX, dW, db = oracle.knnconv_backward(x, t["knn_idx_pad"], t["tap"].astype(np.int64), int(t["V"]), w, g)
    for name, a, r in (("dX", dX, xt.grad.numpy()), ("dW", dW, layer.weight.grad.numpy()), ("dbias", db, layer.bias.grad.numpy())):
        assert rel_err(a, r) < 1e-5, (name, rel_err(a, r))
    save("backward_small.npz", y=y.detach().numpy(), dX=xt.grad.numpy(), dW=layer.weight.grad.numpy(), dbias=layer.bias.grad.numpy(),
         seed=np.int64(31), **t)
    print("backward fixture: n_in", len(ic), "n_out", len(oc), "V", V)


def depthwise_fixture(save, knn):
    """Depthwise and depthwise-separable KNN convolution (fovi/arch/knn.py:722-872).  In the checkout this was generated
    from, both layers' ``forward`` raise: ``_apply_local_rf`` returns ``[b, n, (d v)]`` and the next line rearranges it as a
    4-D ``'b d v n'`` tensor.  The fixture therefore runs the reference layer's own gather (``_pad_and_gather_knns``) and
    tap scatter (``_apply_local_rf``), views the result as ``[b, n, d, v]`` and applies the layers' own contraction
    ``einsum('bndv,dvg->bndg')``, bias and pointwise ``nn.Linear``: the reference's steps with the one shape fixed."""
    from einops import rearrange
    ic, oc, _ = knn.get_in_out_coords(24, 16, 1.0, 2, style="isotropic", auto_match_cart_resources=0, device="cpu")
    rs = np.random.RandomState(41)
    x = rs.standard_normal((4, 16, len(ic))).astype(f32)
    out = {"seed": np.int64(41)}
    torch.manual_seed(6)
    dw = knn.KNNDepthwiseConvLayer(16, 32, 9, ic, oc, device="cpu", ref_frame_side_length=4, bias=True)
    try:
        dw(torch.from_numpy(x))
        raise AssertionError("the reference's depthwise forward runs now: record its output directly")
    except AssertionError:
        raise
    except Exception as e:                                  # noqa: BLE001  (einops.EinopsError at this checkout)
        print("reference KNNDepthwiseConvLayer.forward raises:", type(e).__name__)
    V = dw.ref_coords.shape[0]
    w = (rs.standard_normal((16, V, 2)) * 0.2).astype(f32)
    b = (0.1 * rs.standard_normal(32)).astype(f32)

    def steps(layer, weight):
        f = layer._apply_local_rf(layer._pad_and_gather_knns(torch.from_numpy(x)))         # [b, n, (d v)]
        f = rearrange(f, "b n (d v) -> b n d v", d=16)
        return torch.einsum("bndv,dvg->bndg", f, torch.from_numpy(weight)).reshape(x.shape[0], f.shape[1], -1)

    y = (steps(dw, w).transpose(1, 2) + torch.from_numpy(b)[None, :, None]).numpy()
    t = layer_tables(dw)
    o = oracle.knn_depthwise_forward(x, t["knn_idx_pad"], t["tap"].astype(np.int64), w, b)
    assert rel_err(o, y) < 1e-5, rel_err(o, y)
    out.update(t)
    out["dw_out"] = y
    sep = knn.KNNDepthwiseSeparableConvLayer(16, 32, 9, ic, oc, device="cpu", ref_frame_side_length=4, bias=True)
    pw = (rs.standard_normal((32, 32)) * 0.2).astype(f32)
    pb = (0.1 * rs.standard_normal(32)).astype(f32)
    sep.p_conv.weight.data.copy_(torch.from_numpy(pw))
    sep.p_conv.bias.data.copy_(torch.from_numpy(pb))
    ys = sep.p_conv(steps(sep, w)).transpose(1, 2).numpy()
    o2 = oracle.knn_depthwise_forward(x, t["knn_idx_pad"], t["tap"].astype(np.int64), w)
    o2 = np.einsum("bcn,oc->bon", o2, pw) + pb[None, :, None]
    assert rel_err(o2, ys) < 1e-5, rel_err(o2, ys)
    out["dwsep_out"] = ys
    # gradients of both layers (autograd through the same steps) for a seeded output gradient
    def steps_t(layer, xt, wt):
        f = layer._apply_local_rf(layer._pad_and_gather_knns(xt))
        f = rearrange(f, "b n (d v) -> b n d v", d=16)
        return torch.einsum("bndv,dvg->bndg", f, wt).reshape(xt.shape[0], f.shape[1], -1)
    gy = np.random.RandomState(43).standard_normal(y.shape).astype(f32)
    out["gy"] = gy
    with torch.enable_grad():
        xt, wt, bt = (torch.from_numpy(a).clone().requires_grad_() for a in (x, w, b))
        yy = steps_t(dw, xt, wt).transpose(1, 2) + bt[None, :, None]
        (yy * torch.from_numpy(gy)).sum().backward()
        out["dw_dX"], out["dw_dW"], out["dw_db"] = xt.grad.numpy(), wt.grad.numpy(), bt.grad.numpy()
        xt, wt = (torch.from_numpy(a).clone().requires_grad_() for a in (x, w))
        sep.p_conv.weight.requires_grad_(True); sep.p_conv.bias.requires_grad_(True)
        sep.p_conv.weight.grad = None; sep.p_conv.bias.grad = None
        yy = sep.p_conv(steps_t(sep, xt, wt)).transpose(1, 2)
        (yy * torch.from_numpy(gy)).sum().backward()
        out["dwsep_dX"], out["dwsep_dW"] = xt.grad.numpy(), wt.grad.numpy()
        out["dwsep_dPW"], out["dwsep_dPb"] = sep.p_conv.weight.grad.numpy().copy(), sep.p_conv.bias.grad.numpy().copy()
    save("depthwise_small.npz", **out)
    print("depthwise fixture: n_in", len(ic), "n_out", len(oc), "V", V, "state keys", sorted(sep.state_dict().keys()), sorted(dw.state_dict().keys()))


def sampler_backward_fixture(save, retina):
    """Image gradient of the reference sensor (autograd through F.grid_sample, samplers.py:108) on CPU."""
    rt = retina.RetinalTransform(resolution=20, start_res=48, fov=16, cmf_a=1.0, style="isotropic", sampler="grid_bilinear", fixation_size=48,
                                 auto_match_cart_resources=0, device="cpu")
    rs = np.random.RandomState(61)
    B, F = 2, 3
    x = rs.random_sample((B, 3, 48, 48)).astype(f32)
    fix = (-0.1 + 1.2 * rs.random_sample((B, F, 2))).astype(f32)
    N = len(rt.sampler.coords)
    gy = rs.standard_normal((B, F, 3, N)).astype(f32)
    out = {"seed": np.int64(61), "fix": fix, "sampling_grid": rt.sampler.sampling_grid.numpy()[0, 0]}
    for mode in ("bilinear", "nearest"):
        rt.sampler.mode = mode
        with torch.enable_grad():
            xt = torch.from_numpy(x).clone().requires_grad_()
            ys = torch.stack([rt(xt, torch.from_numpy(fix[:, f])) for f in range(F)], 1)          # [B,F,C,N]
            (ys * torch.from_numpy(gy)).sum().backward()
        out[f"{mode}_y"], out[f"{mode}_dx"] = ys.detach().numpy(), xt.grad.numpy()
    save("sampler_backward_small.npz", **out)
    print("sampler backward fixture: N", N)


def norms_fixture(save, knn):
    """The per-sample norm layers (fovi/arch/norm.py) and 'gaussian' pooling (fovi/arch/knn.py:321-394), run on CPU."""
    import fovi.arch.norm as norm
    rs = np.random.RandomState(51)
    B, C, N = 3, 24, 37
    x = (rs.standard_normal((B, C, N)) * 1.5 + 0.3).astype(f32)
    out = {"seed": np.int64(51), "x_shape": np.array([B, C, N])}
    for name, cls, wshape, mode, kw in (("channel", norm.KNNChannelNorm, (C,), "channel", {}), ("coord", norm.KNNCoordNorm, (N,), "coord", {}),
                                        ("layer", norm.KNNLayerNorm, (C, N), "layer", {}), ("group", norm.KNNGroupNorm, (C,), "group", {})):
        layer = cls(N, C, device="cpu", **kw)
        w = (0.5 + rs.random_sample(wshape)).astype(f32)
        b = (0.2 * rs.standard_normal(wshape)).astype(f32)
        layer.weight.data.copy_(torch.from_numpy(w)); layer.bias.data.copy_(torch.from_numpy(b))
        y = layer(torch.from_numpy(x)).numpy()
        groups = layer.num_groups if name == "group" else 1
        o = oracle.knn_norm(x, mode, w, b, eps=layer.eps, groups=groups)
        assert np.abs(o - y).max() < 2e-6, (name, np.abs(o - y).max())
        out[f"{name}_w"], out[f"{name}_b"], out[f"{name}_out"], out[f"{name}_groups"] = w, b, y, np.int64(groups)
        assert sorted(layer.state_dict().keys()) == ["bias", "weight"]
    assert norm.find_valid_num_groups(24, 32) == 6 and norm.find_valid_num_groups(96, 32) == 24 and norm.find_valid_num_groups(7, 32) == 1
    # gaussian pooling on a small sensor pair
    ic, oc, _ = knn.get_in_out_coords(24, 16, 1.0, 2, style="isotropic", auto_match_cart_resources=0, device="cpu")
    pool = knn.KNNPoolingLayer(9, ic, oc, mode="gaussian", device="cpu", gauss_sigma=0.6)
    xp = (rs.standard_normal((2, 5, len(ic)))).astype(f32)
    xp[0, 1, 7] = np.nan                                            # a NaN input is dropped like a pad neighbour
    yp = pool(torch.from_numpy(xp)).numpy()
    idxp = pool.knn_indices_pad_token.numpy().astype(np.int32)
    gw = pool.gaussian_weights.numpy()
    o = oracle.knn_pool_weighted(xp, idxp, gw)
    assert np.allclose(o, yp, rtol=1e-5, atol=1e-6, equal_nan=True), np.nanmax(np.abs(o - yp))
    out.update(pool_x=xp, pool_out=yp, pool_knn_idx_pad=idxp, pool_knn_idx=pool.knn_indices.numpy().astype(np.int32),
               pool_weights=gw, pool_distances=pool.knn_distances.numpy(), pool_n_in=np.int64(len(ic)), pool_sigma=np.float64(0.6))
    save("norms_small.npz", **out)
    print("norms fixture: groups", int(out["group_groups"]), "pool n_in", len(ic), "n_out", len(oc))


def pool_backward_fixture(save, knn):
    """Gradients of the reference's KNNPoolingLayer (fovi/arch/knn.py:345-394) with respect to its input, from its own
    autograd on CPU in float32, for the four pooling modes on a small strided sensor pair (pad neighbours at the rim)."""
    rs = np.random.RandomState(71)
    ic, oc, _ = knn.get_in_out_coords(24, 16, 1.0, 2, style="isotropic", auto_match_cart_resources=0, device="cpu")
    x = rs.standard_normal((2, 5, len(ic))).astype(f32)
    out = {"seed": np.int64(71), "x": x, "n_in": np.int64(len(ic))}
    with torch.enable_grad():
        for mode in ("max", "avg", "sum", "gaussian"):
            pool = knn.KNNPoolingLayer(9, ic, oc, mode=mode, device="cpu", gauss_sigma=0.6)
            xt = torch.from_numpy(x).requires_grad_(True)
            y = pool(xt)
            gy = torch.from_numpy(rs.standard_normal(tuple(y.shape)).astype(f32))
            y.backward(gy)
            out[f"{mode}_gy"], out[f"{mode}_dx"], out[f"{mode}_y"] = gy.numpy(), xt.grad.numpy(), y.detach().numpy()
            if mode == "gaussian":
                out["weights"] = pool.gaussian_weights.numpy()
        out["knn_idx_pad"] = pool.knn_indices_pad_token.numpy().astype(np.int32)
        out["knn_idx"] = pool.knn_indices.numpy().astype(np.int32)
        out["distances"] = pool.knn_distances.numpy()
    n_pad = int((out["knn_idx_pad"] == len(ic)).sum())
    save("pool_backward_small.npz", **out)
    print("pool backward fixture: n_in", len(ic), "n_out", len(oc), "pad entries", n_pad)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--only", default=None, choices=[None, "alexnet", "backward", "depthwise", "norms", "sampler_backward", "pool_backward"], help="regenerate one fixture group only")
    args = ap.parse_args()
    knn, retina, coords, knnvit = load_reference(args.reference)
    torch.set_grad_enabled(False)
    save = lambda name, **kw: np.savez_compressed(os.path.join(HERE, name), **kw)  # noqa: E731
    if args.only == "alexnet":
        return alexnet_fixture(save)
    if args.only == "backward":
        return backward_fixture(save, knn)
    if args.only == "depthwise":
        return depthwise_fixture(save, knn)
    if args.only == "norms":
        return norms_fixture(save, knn)
    if args.only == "sampler_backward":
        return sampler_backward_fixture(save, retina)
    if args.only == "pool_backward":
        return pool_backward_fixture(save, knn)

    # ------------------------------------------------------------ sensors (geometry fixtures)
    sensors = {}
    for tag, a, start in (("a0p5", 0.5, 256), ("a1", 1.0, 256), ("a2p78", 2.78, 224), ("a2p785765", 2.785765, 224), ("a60p94", 60.94, 256)):
        rt = retina.RetinalTransform(resolution=64, start_res=start, fov=16, cmf_a=a, style="isotropic",
                                     sampler="grid_bilinear", fixation_size=start, auto_match_cart_resources=1, device="cpu")
        sensors[tag] = rt
        c = rt.sampler.coords
        save(f"sensor_{tag}.npz", sampling_grid=rt.sampler.sampling_grid.numpy()[0, 0], **coords_dict(c))
        print("sensor", tag, "resolution", rt.resolution, "N", len(c))

    # ------------------------------------------------------------ config 1: sensor + one KNNConv, fp32
    rt = sensors["a2p78"]
    x = synth_images(0, (8, 3, 224, 224))
    y_ref = rt(torch.from_numpy(x), None).numpy()
    grid = rt.sampler.sampling_grid.numpy()[0, 0]
    y_or = oracle.retinal_sample(x, grid, None, np.full((8, 2), 224, f32))
    assert np.array_equal(y_or, y_ref), "sampler oracle is not bit-exact (config 1)"
    c = rt.sampler.coords
    layer = knn.KNNConvLayer(3, 64, 49, c, c, device="cpu", ref_frame_side_length=7, bias=False)
    rs = np.random.RandomState(1)
    w = kaiming_weight(rs, 64, 3, 49)
    layer.weight.data.copy_(torch.from_numpy(w))
    out_ref = layer(torch.from_numpy(y_ref)).numpy()
    t = layer_tables(layer)
    out_or = oracle.knnconv_forward(y_ref, t["knn_idx_pad"], t["tap"].astype(np.int64), int(t["V"]), w)
    e = rel_err(out_or, out_ref)
    assert e < 1e-5, e
    e2 = rel_err(oracle.knnconv_forward_closed_form(y_ref, t["knn_idx_pad"], t["tap"].astype(np.int64), int(t["V"]), w), out_ref)
    assert e2 < 1e-5, e2
    print("config1 conv oracle rel err", e, e2)
    save("config1.npz", sampled=y_ref, conv_out_b0=out_ref[0], conv_out_sum=out_ref.astype(np.float64).sum((1, 2)),
         conv_out_sqsum=(out_ref.astype(np.float64) ** 2).sum((1, 2)), **t)

    # ------------------------------------------------------------ config 2 (small batch): sampler modes
    B, F = 2, 3
    x = synth_images(0, (B, 3, 256, 256))
    fix = synth_fixations(0, B, F)
    fix_any = synth_fixations(3, B, F, lo=0.0, span=1.0)      # anywhere in the image: many out-of-image taps
    sizes = np.array([[[256, 256], [192, 160], [300, 280]]] * B, f32)   # per-fixation (h, w)
    out = {"fix": fix, "fix_any": fix_any, "sizes": sizes}
    for tag in ("a1", "a2p78", "a60p94"):
        rt = sensors[tag]
        grid = rt.sampler.sampling_grid.numpy()[0, 0]
        fs = rt.fixation_size                                 # default fixation size of this sensor (224 or 256)
        out[f"{tag}_default_size"] = np.int64(fs)
        for mode in ("bilinear", "nearest"):
            rt.sampler.mode = mode
            for fname, fx in (("near", fix), ("any", fix_any)):
                ys, ysz, yb = [], [], []
                for f in range(F):
                    ys.append(rt(torch.from_numpy(x), torch.from_numpy(fx[:, f])).numpy())
                    ysz.append(rt(torch.from_numpy(x), torch.from_numpy(fx[:, f]), fixation_size=torch.from_numpy(sizes[:, f])).numpy())
                    g = coords.transform_sampling_grid(rt.sampler.sampling_grid, torch.from_numpy(fx[:, f]), torch.from_numpy(np.full((B, 2), fs, np.int64)), (256, 256))
                    yb.append(torch.nn.functional.grid_sample(torch.from_numpy(x), g, mode=mode, padding_mode="border", align_corners=False).squeeze(2).numpy())
                ys, ysz, yb = np.stack(ys, 1), np.stack(ysz, 1), np.stack(yb, 1)
                o = oracle.retinal_sample(x, grid, fx, np.full((B, F, 2), fs, f32), mode, "zeros")
                assert np.array_equal(o, ys), (tag, mode, fname, "zeros", np.abs(o - ys).max())
                o = oracle.retinal_sample(x, grid, fx, sizes, mode, "zeros")
                assert np.array_equal(o, ysz), (tag, mode, fname, "sizes", np.abs(o - ysz).max())
                o = oracle.retinal_sample(x, grid, fx, np.full((B, F, 2), fs, f32), mode, "border")
                assert np.array_equal(o, yb), (tag, mode, fname, "border", np.abs(o - yb).max())
                out[f"{tag}_{mode}_{fname}_zeros"] = ys
                if fname == "near":          # all variants are checked above; a subset is stored to keep the fixture small
                    out[f"{tag}_{mode}_{fname}_sizes"] = ysz
                else:
                    out[f"{tag}_{mode}_{fname}_border"] = yb
            rt.sampler.mode = "bilinear"
        print("config2 sampler oracle bit-exact for", tag)
    save("config2_small.npz", **out)

    # ------------------------------------------------------------ config 3: AlexNet-shaped KNNConv stack
    fov, a = 16, 1.0
    chans, strides, ks = [3, 64, 192, 384, 256, 256], [2, 2, 1, 1, 1], [121, 25, 9, 9, 9]
    in_res, cart_res = coords.auto_match_num_coords(fov, a, 64, "isotropic", 1, "cpu", quiet=True)
    rs = np.random.RandomState(1)
    layers, tables, in_coords = [], {}, None
    for i in range(5):
        ic, oc, out_cart = knn.get_in_out_coords(in_res, fov, a, strides[i], style="isotropic", auto_match_cart_resources=1, in_cart_res=cart_res, device="cpu")
        side = int(np.ceil(2 * np.sqrt(ks[i])))
        L = knn.KNNConvLayer(chans[i], chans[i + 1], ks[i], ic, oc, device="cpu", ref_frame_side_length=side, bias=True)
        w = kaiming_weight(rs, chans[i + 1], chans[i], side * side)
        L.weight.data.copy_(torch.from_numpy(w))
        L.bias.data.zero_()
        layers.append((L, w))
        for k_, v_ in layer_tables(L).items():
            tables[f"l{i}_{k_}"] = v_
        tables.update(coords_dict(ic, f"l{i}_in_"))
        tables[f"l{i}_out_resolution"] = np.int64(oc.resolution)
        print(f"config3 layer {i}: Nin {len(ic)} Nout {len(oc)} K {L._k} V {side*side} pad {float(L.knn_indices_pad_mask.float().mean()):.4f}")
        in_res, cart_res = oc.resolution, out_cart
    tables.update(coords_dict(oc, "l5_in_"))
    xb = synth_images(0, (2, 3, int(tables["l0_n_in"])))
    h = torch.from_numpy(xb)
    acts = {}
    ho = xb
    for i, (L, w) in enumerate(layers):
        h = L(h)
        ho = oracle.knnconv_forward(ho, tables[f"l{i}_knn_idx_pad"], tables[f"l{i}_tap"].astype(np.int64), int(tables[f"l{i}_V"]), w, np.zeros(chans[i + 1], f32))
        if i < 4:
            h = torch.relu(h)
            ho = np.maximum(ho, 0)
        acts[f"act{i}"] = h.numpy()
        e = rel_err(ho, h.numpy())
        assert e < 1e-5, (i, e)
    print("config3 stack oracle ok")
    save("config3_tables.npz", **tables)
    save("config3_acts_b2.npz", **acts)

    # ------------------------------------------------------------ config 4: foveated patch embedding 3 -> 384
    for tag, patch in (("p8", 8), ("p4", 4)):
        pe = knnvit.KNNPartitioningPatchEmbedding(3, 384, in_res=64, fov=16, cmf_a=2.78, in_cart_res=64, cart_patch_size=patch,
                                                  ref_frame_side_length=16, max_coord_val="auto", sample_cortex=True, bias=True,
                                                  transposed=True, device="cpu")
        t = layer_tables(pe)
        V = int(t["V"])
        w = kaiming_weight(np.random.RandomState(1), 384, 3, V)
        bvec = (0.1 * np.random.RandomState(2).standard_normal(384)).astype(f32)
        pe.weight.data.copy_(torch.from_numpy(w)); pe.bias.data.copy_(torch.from_numpy(bvec))
        xb = synth_images(0, (2, 3, int(t["n_in"])))
        o_ref = pe(torch.from_numpy(xb)).numpy()
        o = oracle.knnconv_forward(xb, t["knn_idx_pad"], t["tap"].astype(np.int64), V, w, bvec)
        e = rel_err(o, o_ref)
        assert e < 1e-5, e
        print(f"config4 patch-embed {tag}: Nin {int(t['n_in'])} tokens {o_ref.shape[-1]} K {pe._k} V {V} err {e:.2e}")
        save(f"config4_patch_embed_{tag}.npz", out_b2=o_ref, in_cartesian=pe.in_coords.cartesian.numpy(), out_cartesian=pe.out_coords.cartesian.numpy(),
             out_cortical=pe.out_coords.cortical.numpy(), **t)

    # ------------------------------------------------------------ fixation policies (seeded NumPy global state)
    pol = {}
    rt = sensors["a1"]
    rt.sampler.mode = "bilinear"
    xb = synth_images(7, (3, 3, 256, 256))
    for name, kw, train in (("near_eval", dict(norm_dist_from_center=0.25), False),
                            ("near_train", dict(norm_dist_from_center=0.25, add_aspect_variation=True, nonrandom_first=True), True),
                            ("crop_train", dict(add_aspect_variation=True), True)):
        p_ref = load_reference.policies.MultiRandomSaccadePolicy(rt, n_fixations=4, **kw)
        p_ref.train(train)
        np.random.seed(11)
        out = p_ref(torch.from_numpy(xb))
        pol[f"{name}_fixations"] = out["fixations"].numpy()
        pol[f"{name}_sizes"] = out["fixation_sizes"].numpy()
        pol[f"{name}_x_fixs"] = out["x_fixs"].numpy()
        pol[f"{name}_deltas"] = out["fix_deltas"].numpy()
        pol[f"{name}_next_random"] = np.float64(np.random.uniform())          # the stream position after the call
    save("policy_small.npz", **pol)

    # ------------------------------------------------------------ max pooling (next-row fixture)
    c = sensors["a0p5"].sampler.coords
    ic, oc, _ = knn.get_in_out_coords(c.resolution, 16, 0.5, 2, style="isotropic", auto_match_cart_resources=1, in_cart_res=64, device="cpu", in_coords=c)
    pool = knn.KNNPoolingLayer(9, ic, oc, mode="max", device="cpu")
    xb = synth_images(5, (2, 4, len(ic))) - f32(0.5)
    p_ref = pool(torch.from_numpy(xb)).numpy()
    idxp = pool.knn_indices_pad_token.numpy().astype(np.int32)
    assert np.array_equal(oracle.knn_pool_max(xb, idxp), p_ref)
    extra = {}
    for mode in ("avg", "sum"):
        pm = knn.KNNPoolingLayer(9, ic, oc, mode=mode, device="cpu")
        extra[f"out_{mode}"] = pm(torch.from_numpy(xb)).numpy()
        o = getattr(oracle, f"knn_pool_{mode}")(xb, idxp)
        assert np.allclose(o, extra[f"out_{mode}"], rtol=1e-6, atol=1e-7), mode
    save("pool_a0p5.npz", knn_idx_pad=idxp, knn_idx=pool.knn_indices.numpy().astype(np.int32), out=p_ref, n_in=np.int64(len(ic)),
         n_out=np.int64(len(oc)), **extra)
    print("point counts a=0.5 chain:", len(ic), len(oc))

    alexnet_fixture(save)
    backward_fixture(save, knn)
    depthwise_fixture(save, knn)
    norms_fixture(save, knn)
    sampler_backward_fixture(save, retina)
    pool_backward_fixture(save, knn)


if __name__ == "__main__":
    main()
