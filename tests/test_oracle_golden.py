"""CPU: the NumPy oracle reproduces the outputs recorded from the reference (tests/golden)."""
import numpy as np
import pytest

from conftest import synth_images, kaiming_weight
from oracle import fovi_oracle as oracle

f32 = np.float32


def rel_err(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def test_config1_sampler_bit_exact(golden):
    g, s = golden("config1.npz"), golden("sensor_a2p78.npz")
    x = synth_images(0, (8, 3, 224, 224))
    y = oracle.retinal_sample(x, s["sampling_grid"], None, np.full((8, 2), 224, f32))
    assert y.shape == (8, 3, 3975)
    assert np.array_equal(y, g["sampled"])


def test_config1_knnconv(golden):
    g = golden("config1.npz")
    w = kaiming_weight(np.random.RandomState(1), 64, 3, 49)
    out = oracle.knnconv_forward(g["sampled"], g["knn_idx_pad"], g["tap"].astype(np.int64), int(g["V"]), w)
    assert rel_err(out[0], g["conv_out_b0"]) < 1e-5
    np.testing.assert_allclose(out.astype(np.float64).sum((1, 2)), g["conv_out_sum"], rtol=1e-6)
    np.testing.assert_allclose((out.astype(np.float64) ** 2).sum((1, 2)), g["conv_out_sqsum"], rtol=1e-6)
    out2 = oracle.knnconv_forward_closed_form(g["sampled"][:2], g["knn_idx_pad"], g["tap"].astype(np.int64), int(g["V"]), w)
    assert rel_err(out2[0], g["conv_out_b0"]) < 1e-5


@pytest.mark.parametrize("tag", ["a1", "a2p78", "a60p94"])
@pytest.mark.parametrize("mode", ["bilinear", "nearest"])
def test_config2_sampler_modes_bit_exact(golden, tag, mode):
    g, s = golden("config2_small.npz"), golden(f"sensor_{tag}.npz")
    x = synth_images(0, (2, 3, 256, 256))
    fs = float(g[f"{tag}_default_size"])
    full = np.full((2, 3, 2), fs, f32)
    grid = s["sampling_grid"]
    assert np.array_equal(oracle.retinal_sample(x, grid, g["fix"], full, mode, "zeros"), g[f"{tag}_{mode}_near_zeros"])
    assert np.array_equal(oracle.retinal_sample(x, grid, g["fix"], g["sizes"], mode, "zeros"), g[f"{tag}_{mode}_near_sizes"])
    assert np.array_equal(oracle.retinal_sample(x, grid, g["fix_any"], full, mode, "zeros"), g[f"{tag}_{mode}_any_zeros"])
    assert np.array_equal(oracle.retinal_sample(x, grid, g["fix_any"], full, mode, "border"), g[f"{tag}_{mode}_any_border"])


def test_known_point_counts(golden):
    """Point counts printed by the reference's notebooks (step2_knnconv cells 10-18, step4 cell 9)."""
    assert golden("sensor_a0p5.npz")["cartesian"].shape[0] == 4085
    assert int(golden("sensor_a0p5.npz")["resolution"]) == 53
    assert int(golden("pool_a0p5.npz")["n_out"]) == 964
    assert golden("sensor_a2p785765.npz")["cartesian"].shape[0] == 3976
    t = golden("config3_tables.npz")
    assert [int(t[f"l{i}_n_in"]) for i in range(5)] == [4010, 1023, 225, 225, 225]
    assert [int(t[f"l{i}_V"]) for i in range(5)] == [484, 100, 36, 36, 36]


def test_config3_stack(golden):
    t, acts = golden("config3_tables.npz"), golden("config3_acts_b2.npz")
    chans = [3, 64, 192, 384, 256, 256]
    rs = np.random.RandomState(1)
    h = synth_images(0, (2, 3, 4010))
    for i in range(5):
        V = int(t[f"l{i}_V"])
        w = kaiming_weight(rs, chans[i + 1], chans[i], V)
        h = oracle.knnconv_forward(h, t[f"l{i}_knn_idx_pad"], t[f"l{i}_tap"].astype(np.int64), V, w, np.zeros(chans[i + 1], f32))
        if i < 4:
            h = np.maximum(h, 0)
        assert rel_err(h, acts[f"act{i}"]) < 1e-5, i


@pytest.mark.parametrize("tag", ["p8", "p4"])
def test_config4_patch_embed(golden, tag):
    g = golden(f"config4_patch_embed_{tag}.npz")
    V = int(g["V"])
    w = kaiming_weight(np.random.RandomState(1), 384, 3, V)
    b = (0.1 * np.random.RandomState(2).standard_normal(384)).astype(f32)
    x = synth_images(0, (2, 3, int(g["n_in"])))
    out = oracle.knnconv_forward(x, g["knn_idx_pad"], g["tap"].astype(np.int64), V, w, b)
    assert rel_err(out, g["out_b2"]) < 1e-5


def test_pool_max(golden):
    g = golden("pool_a0p5.npz")
    x = synth_images(5, (2, 4, int(g["n_in"]))) - f32(0.5)
    assert np.array_equal(oracle.knn_pool_max(x, g["knn_idx_pad"]), g["out"])


def test_closed_form_handles_pad_and_collisions():
    rs = np.random.RandomState(7)
    B, Cin, Nin, Nout, K, V, Cout = 3, 5, 11, 7, 6, 4, 8   # V < K forces colliding taps
    x = rs.standard_normal((B, Cin, Nin)).astype(f32)
    idx = rs.randint(0, Nin + 1, (K, Nout))               # includes pad token Nin
    idx[:, 0] = Nin                                        # a point whose neighbours are all pads
    tap = rs.randint(0, V, (Nout, K))
    w = rs.standard_normal((Cout, Cin * V)).astype(f32)
    b = rs.standard_normal(Cout).astype(f32)
    a = oracle.knnconv_forward(x, idx, tap, V, w, b)
    c = oracle.knnconv_forward_closed_form(x, idx, tap, V, w, b)
    np.testing.assert_allclose(a, c, rtol=1e-5, atol=1e-5)
    np.testing.assert_allclose(a[:, :, 0], np.broadcast_to(b, (B, Cout)), rtol=1e-6)


def test_c_oracle_against_golden_and_numpy(golden):
    """The C restatement: sampler bit-exact against the reference's recorded outputs, KNNConv within float
    summation-order error of them, and equal to the NumPy oracle on a small random case with pads/collisions."""
    from oracle import c_oracle
    g, s = golden("config1.npz"), golden("sensor_a2p78.npz")
    x = synth_images(0, (8, 3, 224, 224))
    y = c_oracle.retinal_sample(x, s["sampling_grid"], np.full((8, 1, 2), 0.5, f32), np.full((8, 1, 2), 224, f32))
    assert np.array_equal(y[:, 0], g["sampled"])
    g2, s1 = golden("config2_small.npz"), golden("sensor_a1.npz")
    x2 = synth_images(0, (2, 3, 256, 256))
    full = np.full((2, 3, 2), 256, f32)
    for mode in ("bilinear", "nearest"):
        assert np.array_equal(c_oracle.retinal_sample(x2, s1["sampling_grid"], g2["fix_any"], full, mode, "zeros"), g2[f"a1_{mode}_any_zeros"])
        assert np.array_equal(c_oracle.retinal_sample(x2, s1["sampling_grid"], g2["fix_any"], full, mode, "border"), g2[f"a1_{mode}_any_border"])
        assert np.array_equal(c_oracle.retinal_sample(x2, s1["sampling_grid"], g2["fix"], g2["sizes"], mode, "zeros"), g2[f"a1_{mode}_near_sizes"])
    w = kaiming_weight(np.random.RandomState(1), 64, 3, 49)
    out = c_oracle.knnconv_forward_closed_form(g["sampled"], g["knn_idx_pad"], g["tap"].astype(np.int64), 49, w)
    assert rel_err(out[0], g["conv_out_b0"]) < 1e-4
    rs = np.random.RandomState(7)
    xs = rs.standard_normal((3, 5, 11)).astype(f32)
    idx = rs.randint(0, 12, (6, 7)).astype(np.int32); tap = rs.randint(0, 4, (7, 6))
    ws = rs.standard_normal((8, 20)).astype(f32); b = rs.standard_normal(8).astype(f32)
    np.testing.assert_allclose(c_oracle.knnconv_forward_closed_form(xs, idx, tap, 4, ws, b, relu=True),
                               oracle.knnconv_forward_closed_form(xs, idx, tap, 4, ws, b, relu=True), rtol=1e-4, atol=1e-5)


def test_pool_avg_sum(golden):
    g = golden("pool_a0p5.npz")
    x = synth_images(5, (2, 4, int(g["n_in"]))) - f32(0.5)
    np.testing.assert_allclose(oracle.knn_pool_avg(x, g["knn_idx_pad"]), g["out_avg"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(oracle.knn_pool_sum(x, g["knn_idx_pad"]), g["out_sum"], rtol=1e-6, atol=1e-7)


def test_oracle_backward_matches_reference_autograd(golden):
    g = golden("backward_small.npz")
    V, n_in = int(g["V"]), int(g["n_in"])
    rs = np.random.RandomState(int(g["seed"]))
    from conftest import kaiming_weight
    w = kaiming_weight(rs, 32, 16, V)
    rs.standard_normal(32)                                   # the bias draw of the generator
    x = rs.standard_normal((5, 16, n_in)).astype(np.float32)
    gy = rs.standard_normal((5, 32, g["knn_idx"].shape[1])).astype(np.float32)
    dX, dW, db = oracle.knnconv_backward(x, g["knn_idx_pad"], g["tap"].astype(np.int64), V, w, gy)
    for a, r in ((dX, g["dX"]), (dW, g["dW"]), (db, g["dbias"])):
        assert np.abs(a - r).max() <= 1e-5 * np.abs(r).max()


def test_oracle_depthwise_matches_reference_steps(golden):
    g = golden("depthwise_small.npz")
    V = int(g["V"])
    rs = np.random.RandomState(int(g["seed"]))
    x = rs.standard_normal((4, 16, int(g["n_in"]))).astype(np.float32)
    w = (rs.standard_normal((16, V, 2)) * 0.2).astype(np.float32)
    b = (0.1 * rs.standard_normal(32)).astype(np.float32)
    o = oracle.knn_depthwise_forward(x, g["knn_idx_pad"], g["tap"].astype(np.int64), w, b)
    assert np.abs(o - g["dw_out"]).max() <= 1e-5 * np.abs(g["dw_out"]).max()


def test_norms_and_gaussian_pooling_oracle(golden):
    g = golden("norms_small.npz")
    B, C, N = (int(v) for v in g["x_shape"])
    x = (np.random.RandomState(int(g["seed"])).standard_normal((B, C, N)) * 1.5 + 0.3).astype(np.float32)
    for name in ("channel", "coord", "layer", "group"):
        o = oracle.knn_norm(x, name, g[f"{name}_w"], g[f"{name}_b"], groups=int(g[f"{name}_groups"]))
        assert np.abs(o - g[f"{name}_out"]).max() < 2e-6, name
    o = oracle.knn_pool_weighted(g["pool_x"], g["pool_knn_idx_pad"], g["pool_weights"])
    assert np.allclose(o, g["pool_out"], rtol=1e-5, atol=1e-6, equal_nan=True)


@pytest.mark.parametrize("mode", ["max", "avg", "sum", "gaussian"])
def test_pool_backward_oracle_matches_reference_autograd(golden, mode):
    """oracle.knn_pool_backward against the gradients the reference's own autograd produced (fovi/arch/knn.py:345-394)."""
    g = golden("pool_backward_small.npz")
    dx = oracle.knn_pool_backward(g["x"], g["knn_idx_pad"], g[f"{mode}_gy"], mode, g["weights"] if mode == "gaussian" else None)
    assert np.abs(dx - g[f"{mode}_dx"]).max() < 1e-5
