"""CPU: the host-side geometry and table construction reproduce the reference's recorded coordinates
and tables bit for bit; module argument handling; sharding helpers on 2 gloo ranks."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT
from fovi_b200 import tables
from fovi_b200.coords import SamplingCoords, auto_match_num_coords, find_desired_res, get_in_out_coords
from fovi_b200.dist import all_gather_rows, shard_range


@pytest.mark.parametrize("tag,a", [("a0p5", 0.5), ("a1", 1.0), ("a2p78", 2.78), ("a2p785765", 2.785765), ("a60p94", 60.94)])
def test_sensor_coordinates_bit_exact(golden, tag, a):
    g = golden(f"sensor_{tag}.npz")
    res, n = find_desired_res(16, a, 64 ** 2, "isotropic", force_less_than=True)
    assert res == int(g["resolution"]) and n == g["cartesian"].shape[0]
    c = SamplingCoords(16, a, res)
    for key, attr in (("cartesian", "cartesian"), ("polar", "polar"), ("cortical", "cortical"),
                      ("cartesian_pad", "cartesian_pad_coords"), ("cortical_pad", "cortical_pad_coords")):
        assert np.array_equal(getattr(c, attr).numpy(), g[key]), key
    grid = torch.stack([c.cartesian[:, 0], -c.cartesian[:, 1]], 1).numpy()
    assert np.array_equal(grid, g["sampling_grid"])


@pytest.mark.parametrize("tag,a", [("a0p5", 0.5), ("a1", 1.0), ("a2p78", 2.78), ("a2p785765", 2.785765), ("a60p94", 60.94)])
def test_native_sensor_geometry_matches_recorded_sensors(golden, tag, a):
    """builder='native' (the library's host routines for fovi/sensing/coords.py:204-370, manifold.py:32-48): the same ring
    count and point counts as the reference's recorded sensors, coordinates within a few float32 ulps, same result twice."""
    g = golden(f"sensor_{tag}.npz")
    from fovi_b200 import coords
    res, n = None, None
    os.environ["FOVI_B200_GEOMETRY"] = "native"
    try:
        assert coords.default_builder() == "native"
        res, n = find_desired_res(16, a, 64 ** 2, "isotropic", force_less_than=True)
        c = SamplingCoords(16, a, res)
    finally:
        del os.environ["FOVI_B200_GEOMETRY"]
    assert c.builder == "native" and res == int(g["resolution"]) and n == g["cartesian"].shape[0]
    for key, attr, tol in (("cartesian", "cartesian", 3e-7), ("polar", "polar", 3e-7), ("cortical", "cortical", 4e-6),
                           ("cartesian_pad", "cartesian_pad_coords", 5e-7), ("cortical_pad", "cortical_pad_coords", 6e-6)):
        got = getattr(c, attr).numpy()
        assert got.shape == g[key].shape and got.dtype == g[key].dtype, key
        assert np.abs(got.astype(np.float64) - g[key]).max() <= tol, (key, np.abs(got.astype(np.float64) - g[key]).max())
    c2 = SamplingCoords(16, a, res, builder="native")
    assert np.array_equal(c2.cortical.numpy(), c.cortical.numpy()) and np.array_equal(c2.cartesian_pad_coords.numpy(), c.cartesian_pad_coords.numpy())
    # the layer chain built from it keeps the builder and the reference's point counts
    nxt, rings, _ = c.get_strided_coords(2, auto_match_cart_resources=1, in_cart_res=64)
    ref_next, ref_rings, _ = SamplingCoords(16, a, res, builder="torch").get_strided_coords(2, auto_match_cart_resources=1, in_cart_res=64)
    assert nxt.builder == "native" and rings == ref_rings and len(nxt) == len(ref_next)


def test_native_geometry_argument_checks():
    from fovi_b200._lib import lib
    assert lib.fovi_sensor_ring_layout(16.0, 1.0, 0, None, None) < 0 and lib.fovi_sensor_ring_layout(16.0, -1.0, 8, None, None) < 0
    assert lib.fovi_sensor_ring_layout(16.0, 1.0, 1, None, None) == 1
    assert lib.fovi_sensor_pad_points(16.0, 1.0, 1, 1.0, 0.5, 0, None, None) < 0


def test_config3_layer_chain_tables_bit_exact(golden):
    t = golden("config3_tables.npz")
    strides, ks = [2, 2, 1, 1, 1], [121, 25, 9, 9, 9]
    in_res, cart_res = auto_match_num_coords(16, 1.0, 64, "isotropic", 1)
    for i in range(5):
        ic, oc, out_cart = get_in_out_coords(in_res, 16, 1.0, strides[i], auto_match_cart_resources=1, in_cart_res=cart_res)
        assert len(ic) == int(t[f"l{i}_n_in"]) and oc.resolution == int(t[f"l{i}_out_resolution"])
        idx, dist, pts, cart = tables.knn_table(ic, oc, ks[i])
        ref, side = tables.reference_frame(ks[i], int(np.ceil(2 * np.sqrt(ks[i]))))
        tap, _ = tables.tap_table(idx, pts, cart, oc, ref)
        assert ref.shape[0] == int(t[f"l{i}_V"])
        # neighbour order inside a column is part of the recorded table; compare as recorded and as sets
        assert np.array_equal(np.sort(idx.numpy(), 0), np.sort(t[f"l{i}_knn_idx"], 0))
        assert np.array_equal(idx.numpy(), t[f"l{i}_knn_idx"])
        assert np.array_equal(tables.pad_token_table(idx, len(ic)).numpy(), t[f"l{i}_knn_idx_pad"])
        assert np.array_equal(tap.numpy(), t[f"l{i}_tap"])
        in_res, cart_res = oc.resolution, out_cart


def test_config1_tables_bit_exact(golden):
    g = golden("config1.npz")
    c = SamplingCoords(16, 2.78, 44)
    idx, _, pts, cart = tables.knn_table(c, c, 49)
    ref, side = tables.reference_frame(49, 7)
    tap, _ = tables.tap_table(idx, pts, cart, c, ref)
    assert side == 7 and np.array_equal(idx.numpy(), g["knn_idx"]) and np.array_equal(tap.numpy(), g["tap"])


def test_strided_and_pool_point_counts(golden):
    """fovi-AlexNet's printed chain for a=0.5: 4085 -> 964 -> 230 (notebooks/step2_knnconv)."""
    c = SamplingCoords(16, 0.5, 53)
    c2, rings2, cart2 = c.get_strided_coords(2, auto_match_cart_resources=1, in_cart_res=64)
    c4, rings4, cart4 = c2.get_strided_coords(2, auto_match_cart_resources=1, in_cart_res=cart2)
    assert (len(c), len(c2), len(c4)) == (4085, 964, 230) and (rings2, rings4) == (26, 13)
    assert repr(c2) == "SamplingCoords(length=964, fov=16, cmf_a=0.5, resolution=26, style=isotropic)"


def test_fixation_argument_forms():
    from fovi_b200.sensing import _as_bf2
    B = 3
    t, multi = _as_bf2((0.5, 0.25), B, "cpu", "fix_loc")
    assert t.shape == (B, 1, 2) and not multi and float(t[2, 0, 1]) == 0.25
    t, multi = _as_bf2(torch.rand(B, 2), B, "cpu", "fix_loc")
    assert t.shape == (B, 1, 2) and not multi
    t, multi = _as_bf2(torch.rand(B, 4, 2), B, "cpu", "fix_loc")
    assert t.shape == (B, 4, 2) and multi
    t, _ = _as_bf2(np.array([10, 20, 30]), B, "cpu", "fixation_size")      # one size per image -> (h, w) = (s, s)
    assert t[1, 0].tolist() == [20.0, 20.0]
    with pytest.raises(ValueError):
        _as_bf2(torch.rand(B + 1, 2), B, "cpu", "fix_loc")


def test_shard_range_covers_everything():
    for n in (0, 1, 7, 256, 1023):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def _gloo_worker(rank, world, port, n_rows):
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = torch.arange(n_rows * 3, dtype=torch.float32).reshape(n_rows, 3)
    lo, hi = shard_range(n_rows, rank, world)
    # every rank computes its shard independently (stand-in for the per-rank kernels), then gathers
    mine = full[lo:hi] * 2
    for total in (None, n_rows):
        got = all_gather_rows(mine, total_rows=total)
        assert torch.equal(got, full * 2), (rank, total)
    dist.destroy_process_group()


@pytest.mark.parametrize("n_rows", [8, 7])
def test_all_gather_rows_two_gloo_ranks(n_rows):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_gloo_worker, args=(2, port, n_rows), nprocs=2, join=True)


@pytest.mark.parametrize("name,kw,train", [
    ("near_eval", dict(norm_dist_from_center=0.25), False),
    ("near_train", dict(norm_dist_from_center=0.25, add_aspect_variation=True, nonrandom_first=True), True),
    ("crop_train", dict(add_aspect_variation=True), True),
])
def test_policy_draws_reference_fixations(golden, name, kw, train):
    """Seeded NumPy state -> the same fixation centres and window sizes as the reference policy, and the random stream
    ends at the same position."""
    import types
    from fovi_b200.policies import MultiRandomSaccadePolicy
    g = golden("policy_small.npz")
    rt = types.SimpleNamespace(fixation_size=256, dtype=torch.float32, device="cpu")
    pol = MultiRandomSaccadePolicy(rt, n_fixations=4, **kw)
    pol.train(train)
    np.random.seed(11)
    fix, size = pol.draw((256, 256), 3, 4)
    nxt = np.random.uniform()
    if kw.get("nonrandom_first"):
        fix[:, 0] = 0.5
    assert np.array_equal(fix, g[f"{name}_fixations"])
    assert np.array_equal(size, g[f"{name}_sizes"])
    assert nxt == float(g[f"{name}_next_random"])


def test_group_tables_are_the_union_of_the_members_lists(golden):
    """Grouped first-layer plans: G consecutive output points share one neighbour list (the union) and keep their own taps."""
    from fovi_b200.ops import group_tables
    t = golden("config3_tables.npz")
    c1 = golden("config1.npz")
    for idx, tap, n_in, G in ((t["l0_knn_idx_pad"], t["l0_tap"], int(t["l0_n_in"]), 3), (c1["knn_idx_pad"], c1["tap"], int(c1["n_in"]), 5)):
        K, n_out = idx.shape
        uidx, utap, mtap = group_tables(idx, tap, n_in, G)
        kq, ng = uidx.shape
        assert ng == n_out // G and kq % 8 == 0 and utap.shape == (ng, kq) and mtap.shape == (ng, kq, G)
        assert np.array_equal(utap[0], np.arange(kq))
        for g in (0, ng // 2, ng - 1):
            for j in range(G):
                n = g * G + j
                want = {int(m): int(tap[n, k]) for k, m in enumerate(idx[:, n]) if m != n_in}
                got = {int(uidx[k, g]): int(mtap[g, k, j]) for k in range(kq) if uidx[k, g] != n_in and mtap[g, k, j] != 0xFFFF}
                assert want == got
            members = set(int(m) for m in uidx[:, g] if m != n_in)
            assert len(members) == int((uidx[:, g] != n_in).sum())                      # no point twice
    idx, tap, n_in = t["l0_knn_idx_pad"], t["l0_tap"], int(t["l0_n_in"])
    assert group_tables(idx, tap, n_in, 11) is None                                       # union longer than the kernel's lists
    dup = idx.copy()
    dup[1, 0] = dup[0, 0]
    assert group_tables(dup, tap, n_in, 3) is None                                        # a member lists a point twice
