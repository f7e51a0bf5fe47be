"""GPU: KNNConv kernels (exact float32 path and tcgen05 bf16 path), called through the C ABI,
against the oracle and the golden fixtures recorded from the reference."""
import numpy as np
import pytest
import torch

from conftest import synth_images, kaiming_weight
from oracle import fovi_oracle as oracle

pytestmark = pytest.mark.gpu
f32 = np.float32
BF16_TOL = 1e-2      # relative L2 of the bf16 tensor-core path vs the float32 reference
F32_TOL = 1e-5       # max-abs / max-abs of the float32 path vs the float32 reference


@pytest.fixture(scope="module")
def ops():
    from fovi_b200 import ops
    return ops


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def rel_max(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def bf16_round(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(torch.bfloat16).to(torch.float32).numpy()


def run_tc(ops, plan, x_bcn, w, bias=None, relu=False, out_dtype=torch.float32):
    wt = plan.pack_weights(dev(w))
    xp = ops.pack_points(dev(x_bcn), plan)
    y = plan.forward(xp, wt, None if bias is None else dev(bias), relu=relu, out_dtype=out_dtype, batch=x_bcn.shape[0])
    plan.check()
    return y.to(torch.float32).permute(0, 2, 1).cpu().numpy()


def test_config1_f32_path_matches_reference(ops, golden):
    g = golden("config1.npz")
    V = int(g["V"])
    w = kaiming_weight(np.random.RandomState(1), 64, 3, V)
    plan = ops.KnnConvPlan(g["knn_idx_pad"], g["tap"], int(g["n_in"]), V, 3, 64)
    assert plan.nnz == int((g["knn_idx_pad"] != int(g["n_in"])).sum())
    wt = plan.pack_weights(dev(w), dtype=torch.float32)
    y = plan.forward_f32(dev(g["sampled"]), wt).cpu().numpy()
    assert y.shape == (8, 64, 3975)
    assert rel_max(y[0], g["conv_out_b0"]) < F32_TOL
    np.testing.assert_allclose(y.astype(np.float64).sum((1, 2)), g["conv_out_sum"], rtol=1e-5)
    np.testing.assert_allclose((y.astype(np.float64) ** 2).sum((1, 2)), g["conv_out_sqsum"], rtol=1e-5)
    # points-major in/out gives the same numbers
    y2 = plan.forward_f32(dev(g["sampled"].transpose(0, 2, 1)), wt, x_layout=ops.ACT_BNC, y_layout=ops.ACT_BNC).cpu().numpy()
    assert np.array_equal(y2.transpose(0, 2, 1), y)


def test_config1_tensor_core_path(ops, golden):
    g = golden("config1.npz")
    V = int(g["V"])
    w = kaiming_weight(np.random.RandomState(1), 64, 3, V)
    plan = ops.KnnConvPlan(g["knn_idx_pad"], g["tap"], int(g["n_in"]), V, 3, 64)
    assert plan.cin_packed == 8 and plan.x_layout == ops.X_PAIRS
    y = run_tc(ops, plan, g["sampled"], w)
    assert rel_l2(y[0], g["conv_out_b0"]) < BF16_TOL
    # against the oracle on bf16-rounded operands the only difference is fp32 summation order
    ref = oracle.knnconv_forward_closed_form(bf16_round(g["sampled"][:2]), g["knn_idx_pad"], g["tap"].astype(np.int64), V, bf16_round(w))
    assert rel_max(y[:2], ref) < 1e-4


def test_config3_stack_tensor_core(ops, golden):
    """AlexNet-shaped stack 3->64->192->384->256->256 with ReLU between layers, bf16 activations."""
    t, acts = golden("config3_tables.npz"), golden("config3_acts_b2.npz")
    chans = [3, 64, 192, 384, 256, 256]
    rs = np.random.RandomState(1)
    x = synth_images(0, (2, 3, 4010))
    h = None
    for i in range(5):
        V = int(t[f"l{i}_V"])
        w = kaiming_weight(rs, chans[i + 1], chans[i], V)
        plan = ops.KnnConvPlan(t[f"l{i}_knn_idx_pad"], t[f"l{i}_tap"], int(t[f"l{i}_n_in"]), V, chans[i], chans[i + 1])
        if h is None:
            h = ops.pack_points(dev(x), plan)
        wt = plan.pack_weights(dev(w))
        h = plan.forward(h, wt, torch.zeros(chans[i + 1], device="cuda"), relu=i < 4, out_dtype=torch.bfloat16, batch=2)
        plan.check()
        got = h.to(torch.float32).permute(0, 2, 1).cpu().numpy()
        e = rel_l2(got, acts[f"act{i}"])
        assert e < BF16_TOL, (i, e)


@pytest.mark.parametrize("tag", ["p8", "p4"])
def test_config4_patch_embed(ops, golden, tag):
    g = golden(f"config4_patch_embed_{tag}.npz")
    V = int(g["V"])
    w = kaiming_weight(np.random.RandomState(1), 384, 3, V)
    b = (0.1 * np.random.RandomState(2).standard_normal(384)).astype(f32)
    x = synth_images(0, (2, 3, int(g["n_in"])))
    plan = ops.KnnConvPlan(g["knn_idx_pad"], g["tap"], int(g["n_in"]), V, 3, 384)
    y = run_tc(ops, plan, x, w, b)
    assert rel_l2(y, g["out_b2"]) < BF16_TOL
    wt = plan.pack_weights(dev(w), dtype=torch.float32)
    y32 = plan.forward_f32(dev(x), wt, dev(b)).cpu().numpy()
    assert rel_max(y32, g["out_b2"]) < F32_TOL


@pytest.mark.parametrize("B,Cin,Nin,Nout,K,V,Cout", [
    (1, 3, 40, 17, 5, 9, 16),        # one image, tiny tables, smallest c_out tile (pair layout; repeated neighbours)
    (131, 1, 37, 9, 12, 7, 32),      # one channel, odd point count, ragged second batch tile (pair layout)
    (3, 4, 64, 10, 40, 50, 64),      # four channels, more pair slots than one stage (pair layout)
    (130, 8, 33, 9, 4, 4, 32),       # batch spills into a second, ragged batch tile
    (5, 64, 50, 21, 9, 36, 64),      # 64-channel swizzled operand path
    (3, 128, 30, 11, 7, 16, 384),    # two channel chunks, two c_out tiles of 192
    (2, 24, 30, 11, 7, 3, 48),       # 24 channels: three 8-channel boxes per neighbour, colliding taps (V < K)
    (257, 192, 12, 5, 3, 5, 256),    # three batch tiles, widest accumulator
    (5, 96, 40, 13, 9, 16, 64),      # 96 channels: the second 64-channel box of a neighbour is half zero-filled
    (200, 96, 40, 13, 9, 16, 64),    # the same on CTA pairs
    (140, 72, 25, 9, 5, 9, 32),      # 72 channels on CTA pairs
])
def test_random_small_cases_vs_oracle(ops, B, Cin, Nin, Nout, K, V, Cout):
    rs = np.random.RandomState(B * 1000 + Cin)
    x = rs.standard_normal((B, Cin, Nin)).astype(f32)
    idx = rs.randint(0, Nin + 1, (K, Nout)).astype(np.int32)      # includes pad token Nin
    idx[:, 0] = Nin                                                # a point with no neighbours at all
    tap = rs.randint(0, V, (Nout, K)).astype(np.uint16)
    w = (rs.standard_normal((Cout, Cin * V)) / np.sqrt(Cin * K)).astype(f32)
    b = rs.standard_normal(Cout).astype(f32)
    plan = ops.KnnConvPlan(idx, tap, Nin, V, Cin, Cout)
    ref = oracle.knnconv_forward_closed_form(bf16_round(x), idx, tap.astype(np.int64), V, bf16_round(w), b, relu=True)
    y = run_tc(ops, plan, x, w, b, relu=True)
    assert np.abs(y - ref).max() < 2e-3 * max(1.0, np.abs(ref).max()), np.abs(y - ref).max()
    np.testing.assert_allclose(y[:, :, 0], np.broadcast_to(np.maximum(b, 0), (B, Cout)), rtol=1e-6, atol=1e-6)
    ref32 = oracle.knnconv_forward_closed_form(x, idx, tap.astype(np.int64), V, w, b, relu=True)
    wt32 = plan.pack_weights(dev(w), dtype=torch.float32)
    y32 = plan.forward_f32(dev(x), wt32, dev(b), relu=True).cpu().numpy()
    assert rel_max(y32, ref32) < F32_TOL
    # bf16 output of the tensor-core path
    y16 = run_tc(ops, plan, x, w, b, relu=True, out_dtype=torch.bfloat16)
    assert np.abs(y16 - ref).max() < 1e-2 * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("B,Cin,Nin,Nout,K,V,Cout", [
    (600, 64, 30, 90, 5, 9, 192),     # three 256-row tiles, the last one ragged; more work items than CTA pairs
    (520, 64, 30, 11, 5, 9, 64),      # fewer work items than CTA pairs
    (300, 128, 30, 50, 7, 16, 576),   # three c_out tiles of 192, two channel chunks
    (1024, 64, 40, 80, 6, 9, 384),    # two c_out tiles, four batch tiles
    (512, 64, 30, 74, 3, 4, 128),     # exactly two work items per CTA pair of a 148-SM part
    (512, 32, 30, 60, 3, 4, 128),     # 32 channels: half a 64-channel box
])
def test_pair_kernel_larger_batches(ops, B, Cin, Nin, Nout, K, V, Cout):
    """CTA-pair kernel at several hundred rows: several batch tiles and c_out tiles per output point, ragged last tile,
    against the closed form of fovi/arch/knn.py:484-557."""
    rs = np.random.RandomState(B + Cout)
    x = rs.standard_normal((B, Cin, Nin)).astype(f32)
    idx = rs.randint(0, Nin + 1, (K, Nout)).astype(np.int32)
    idx[:, 0] = Nin                                                # a point with no neighbours at all
    tap = rs.randint(0, V, (Nout, K)).astype(np.uint16)
    w = (rs.standard_normal((Cout, Cin * V)) / np.sqrt(Cin * K)).astype(f32)
    b = rs.standard_normal(Cout).astype(f32)
    plan = ops.KnnConvPlan(idx, tap, Nin, V, Cin, Cout)
    ref = oracle.knnconv_forward_closed_form(bf16_round(x), idx, tap.astype(np.int64), V, bf16_round(w), b, relu=True)
    for od, tol in ((torch.float32, 2e-3), (torch.bfloat16, 1e-2)):
        y = run_tc(ops, plan, x, w, b, relu=True, out_dtype=od)
        assert np.abs(y - ref).max() < tol * max(1.0, np.abs(ref).max()), (od, np.abs(y - ref).max())
    np.testing.assert_allclose(run_tc(ops, plan, x, w, b, relu=True)[:, :, 0], np.broadcast_to(np.maximum(b, 0), (B, Cout)), rtol=1e-6, atol=1e-6)


@pytest.mark.parametrize("B,Cin,Nin,Nout,K,V,Cout", [
    (40, 64, 30, 23, 5, 9, 64),       # one batch tile: single-CTA kernel
    (300, 128, 30, 23, 7, 16, 192),   # CTA pairs, ragged second pair tile
])
def test_scatter_add_output(ops, B, Cin, Nin, Nout, K, V, Cout):
    """fovi_knnconv_forward_scatter_add: output point n is added into row out_map[n] of a float32 result that already
    holds values; checked against the closed form summed the same way."""
    rs = np.random.RandomState(B)
    x = rs.standard_normal((B, Cin, Nin)).astype(f32)
    idx = rs.randint(0, Nin + 1, (K, Nout)).astype(np.int32)
    idx[:, 0] = Nin
    tap = rs.randint(0, V, (Nout, K)).astype(np.uint16)
    w = (rs.standard_normal((Cout, Cin * V)) / np.sqrt(Cin * K)).astype(f32)
    rows = 5
    out_map = rs.randint(0, rows, Nout).astype(np.int32)
    init = rs.standard_normal((B, rows, Cout)).astype(f32)
    plan = ops.KnnConvPlan(idx, tap, Nin, V, Cin, Cout)
    ref = oracle.knnconv_forward_closed_form(bf16_round(x), idx, tap.astype(np.int64), V, bf16_round(w), None)   # [B, Cout, Nout]
    want = init.copy()
    np.add.at(want, (slice(None), out_map), ref.transpose(0, 2, 1))
    out = dev(init.copy())
    plan.forward_scatter_add(ops.pack_points(dev(x), plan), plan.pack_weights(dev(w)), dev(out_map), out)
    plan.check()
    got = out.cpu().numpy()
    assert np.abs(got - want).max() < 2e-3 * max(1.0, np.abs(want).max()), np.abs(got - want).max()


@pytest.mark.parametrize("Cin,Cout", [(3, 32), (64, 64)])
def test_non_finite_input_reaches_only_its_neighbourhoods(ops, Cin, Cout):
    """A NaN at one input point: outputs whose neighbourhoods contain it are NaN, as in the reference (the gather of
    knn.py:484-503 followed by the linear map); outputs whose neighbourhoods contain neither the point nor, on the pair
    layout of a <= 4-channel layer, its pair partner are bit-identical to the clean run; no other output may change on the
    channels-last layout."""
    rs = np.random.RandomState(11)
    B, Nin, Nout, K, V = 6, 40, 19, 5, 9
    x = rs.standard_normal((B, Cin, Nin)).astype(f32)
    idx = np.stack([rs.choice(Nin, K, replace=False) for _ in range(Nout)], 1).astype(np.int32)
    tap = rs.randint(0, V, (Nout, K)).astype(np.uint16)
    w = (rs.standard_normal((Cout, Cin * V)) / np.sqrt(Cin * K)).astype(f32)
    plan = ops.KnnConvPlan(idx, tap, Nin, V, Cin, Cout)
    clean = run_tc(ops, plan, x, w)
    m = 7
    bad = x.copy()
    bad[2, 0, m] = np.nan
    y = run_tc(ops, plan, bad, w)
    has_m = (idx == m).any(0)
    has_partner = (idx == (m ^ 1)).any(0)
    assert np.isnan(y[2][:, has_m]).all()
    if plan.x_layout == ops.X_PAIRS:
        touched = has_m | has_partner
        G = max(1, int(plan.group))          # consecutive output points that share an accumulator share their operand blocks
        for g0 in range(0, Nout, G):
            touched[g0:g0 + G] = touched[g0:g0 + G].any()
        untouched = ~touched
    else:
        untouched = ~has_m
    assert np.array_equal(y[2][:, untouched], clean[2][:, untouched])
    other = [b for b in range(B) if b != 2]
    assert np.array_equal(y[other], clean[other])


def test_linearity_and_determinism_full_batch(ops, golden):
    """Size-independent properties at a full batch tile count: f(x1 + x2) == f(x1) + f(x2) without
    bias, and two runs give the same bits."""
    t = golden("config3_tables.npz")
    V = int(t["l2_V"])
    w = kaiming_weight(np.random.RandomState(3), 384, 192, V)
    plan = ops.KnnConvPlan(t["l2_knn_idx_pad"], t["l2_tap"], 225, V, 192, 384)
    wt = plan.pack_weights(dev(w))
    g = torch.Generator(device="cuda").manual_seed(0)
    # integers/8 are exact in bf16 and so are their pairwise sums
    x1 = (torch.randint(-8, 9, (256, 225, 192), device="cuda", generator=g) / 8).to(torch.bfloat16)
    x2 = (torch.randint(-8, 9, (256, 225, 192), device="cuda", generator=g) / 8).to(torch.bfloat16)
    y1 = plan.forward(x1, wt, out_dtype=torch.float32); y2 = plan.forward(x2, wt, out_dtype=torch.float32)
    y12 = plan.forward(x1 + x2, wt, out_dtype=torch.float32); y12b = plan.forward(x1 + x2, wt, out_dtype=torch.float32)
    plan.check()
    assert torch.equal(y12, y12b)
    assert float((y12 - (y1 + y2)).abs().max()) < 1e-3 * float(y12.abs().max())


def test_empty_batch(ops, golden):
    g = golden("config4_patch_embed_p8.npz")
    plan = ops.KnnConvPlan(g["knn_idx_pad"], g["tap"], int(g["n_in"]), int(g["V"]), 3, 384)
    wt = plan.pack_weights(torch.zeros((384, 3 * int(g["V"])), device="cuda"))
    y = plan.forward(torch.empty((0, plan.n_pairs, 128, 8), dtype=torch.bfloat16, device="cuda"), wt, batch=0)
    assert y.shape == (0, plan.n_out, 384)


def test_shapes_outside_the_tensor_core_path(ops):
    """c_out that is not a multiple of 16: the tensor-core entry point refuses it before any launch, the exact kernel and the
    module (which then uses the exact kernel) handle it."""
    from fovi_b200._lib import FoviError
    rs = np.random.RandomState(5)
    B, Cin, Nin, Nout, K, V, Cout = 2, 3, 20, 7, 5, 9, 10
    x = rs.standard_normal((B, Cin, Nin)).astype(f32)
    idx = rs.randint(0, Nin + 1, (K, Nout)).astype(np.int32); tap = rs.randint(0, V, (Nout, K)).astype(np.uint16)
    w = rs.standard_normal((Cout, Cin * V)).astype(f32)
    plan = ops.KnnConvPlan(idx, tap, Nin, V, Cin, Cout)
    assert not plan.tc_supported
    with pytest.raises(FoviError, match="unsupported"):
        plan.pack_weights(dev(w))
    y = plan.forward_f32(dev(x), plan.pack_weights(dev(w), dtype=torch.float32)).cpu().numpy()
    assert rel_max(y, oracle.knnconv_forward_closed_form(x, idx, tap.astype(np.int64), V, w)) < F32_TOL


def test_grouped_first_layer_equals_ungrouped(ops, golden):
    """c_in <= 4: consecutive output points sharing an accumulator (the default when a group size divides n_out) give the
    ungrouped kernel's result up to the order of float32 accumulation."""
    g = golden("config1.npz")
    V, n_in = int(g["V"]), int(g["n_in"])                             # n_out = 3975 = 3 * 5^2 * 53
    x = dev(g["sampled"])
    for c_out, groups in ((64, {None: 3, 1: 1, 5: 1}), (48, {None: 3, 1: 1, 5: 5})):      # 5 * 64 channels exceed one accumulator
        w = kaiming_weight(np.random.RandomState(1), c_out, 3, V)
        bias = np.linspace(-1, 1, c_out).astype(f32)
        outs = {}
        for group, expect in groups.items():
            plan = ops.KnnConvPlan(g["knn_idx_pad"], g["tap"], n_in, V, 3, c_out, group=group)
            assert plan.group == expect
            xp = ops.pack_points(x, plan)
            outs[group] = plan.forward(xp, plan.pack_weights(dev(w)), dev(bias), relu=True, out_dtype=torch.float32, batch=8).cpu().numpy()
            plan.check()
        assert rel_l2(outs[None], outs[1]) < 1e-5 and rel_l2(outs[5], outs[1]) < 1e-5
        if c_out == 64:
            ref = np.maximum(g["conv_out_b0"] + bias[:, None], 0)
            assert rel_l2(outs[None][0].T, ref) < BF16_TOL


def test_random_shape_sweep(ops):
    """Twenty-four seeded random layers across the operand modes (1-4 channels, 5-8, 16-63, 64 and up with and without a
    multiple of 64), c_out tiles, batch sizes around the 128/256-row tile edges, with and without bias / ReLU."""
    rs = np.random.RandomState(123)
    for it in range(24):
        cin = int(rs.choice([1, 2, 3, 4, 5, 8, 16, 24, 40, 64, 72, 96, 128, 200]))
        cout = int(rs.choice([16, 32, 48, 64, 96, 128, 192, 256, 320, 384]))
        B = int(rs.choice([1, 2, 7, 127, 128, 129, 200, 255, 256, 257, 300]))
        Nin = int(rs.randint(5, 80)); Nout = int(rs.choice([1, 2, 3, 6, 9, 12, 20, 33])); K = int(rs.randint(1, min(Nin, 30) + 1))
        V = int(rs.randint(1, 40))
        x = rs.standard_normal((B, cin, Nin)).astype(f32)
        idx = np.stack([rs.choice(Nin + 1, K, replace=False) for _ in range(Nout)], 1).astype(np.int32)
        tap = rs.randint(0, V, (Nout, K)).astype(np.uint16)
        w = (rs.standard_normal((cout, cin * V)) / np.sqrt(cin * K)).astype(f32)
        b = rs.standard_normal(cout).astype(f32) if rs.rand() < 0.7 else None
        relu = bool(rs.rand() < 0.5)
        plan = ops.KnnConvPlan(idx, tap, Nin, V, cin, cout)
        assert plan.tc_supported
        ref = oracle.knnconv_forward_closed_form(bf16_round(x), idx, tap.astype(np.int64), V, bf16_round(w), b, relu=relu)
        for od, tol in ((torch.float32, 2e-3), (torch.bfloat16, 1e-2)):
            y = run_tc(ops, plan, x, w, b, relu=relu, out_dtype=od)
            err = np.abs(y - ref).max()
            assert err < tol * max(1.0, np.abs(ref).max()), (it, cin, cout, B, Nin, Nout, K, V, plan.group, od, err)
