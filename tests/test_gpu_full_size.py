"""GPU: the benchmark configurations at their full sizes.  The CPU oracle used here is the C restatement
(bit-exact for the sampler), fast enough to check every output of the sampler sweep and a sample of the
rows of the KNNConv configurations; the rest is covered by size-independent properties (determinism,
row independence = shard equivalence)."""
import numpy as np
import pytest
import torch

from conftest import kaiming_weight
from oracle import c_oracle

pytestmark = pytest.mark.gpu
f32 = np.float32


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


@pytest.mark.parametrize("tag", ["a1", "a2p78", "a60p94"])
def test_config2_sampler_sweep_full_size(golden, tag):
    """512 images of 3x256x256, 4 fixations each at centres uniform in the central 50 %, bilinear; zeros padding (the
    reference's) and border clamp; float32 checked bit for bit on all 512*4*3*N outputs, bf16 storage on all of them too."""
    from fovi_b200 import ops
    grid = golden(f"sensor_{tag}.npz")["sampling_grid"]
    rs = np.random.RandomState(0)
    B, F = 512, 4
    x = rs.random_sample((B, 3, 256, 256)).astype(f32)
    fix = (0.25 + 0.5 * rs.random_sample((B, F, 2))).astype(f32)
    hw = np.full((B, F, 2), 256, f32)
    plan = ops.SamplerPlan(grid)
    xd, fd, hd = torch.from_numpy(x).cuda(), torch.from_numpy(fix).cuda(), torch.from_numpy(hw).cuda()
    for pad_name, pad in (("zeros", ops.PAD_ZEROS), ("border", ops.PAD_BORDER)):
        ref = c_oracle.retinal_sample(x, grid, fix, hw, "bilinear", pad_name)
        y = ops.sample(plan, xd, fd, hd, pad=pad)
        assert y.shape == (B, F, 3, grid.shape[0])
        assert np.array_equal(y.cpu().numpy(), ref), pad_name
    # bf16 images: float32 arithmetic on the bf16 values, bf16 result
    xb = torch.from_numpy(x).to(torch.bfloat16)
    ref16 = torch.from_numpy(c_oracle.retinal_sample(xb.float().numpy(), grid, fix, hw)).to(torch.bfloat16)
    y16 = ops.sample(plan, xb.cuda(), fd, hd)
    assert torch.equal(y16.cpu(), ref16)
    # shard equivalence: any slice of the batch gives the same rows
    ys = ops.sample(plan, xd[100:164], fd[100:164], hd[100:164])
    assert torch.equal(ys, ops.sample(plan, xd, fd, hd)[100:164])


def test_config3_stack_full_batch(golden):
    """Batch 256 through the five-layer stack (bf16 activations).  Every layer is checked on 6 rows against the C oracle
    fed with the bf16 values the GPU layer actually consumed; the end-to-end output of those rows against the float32
    chain within the stated 1e-2 relative L2; batch 256 against the same rows run alone (row independence)."""
    from fovi_b200 import ops
    t = golden("config3_tables.npz")
    chans = [3, 64, 192, 384, 256, 256]
    rs = np.random.RandomState(1)
    B = 256
    x = np.random.RandomState(0).random_sample((B, 3, 4010)).astype(f32)
    rows = [0, 1, 127, 128, 200, 255]
    plans, wts, ws = [], [], []
    for i in range(5):
        V = int(t[f"l{i}_V"])
        w = kaiming_weight(rs, chans[i + 1], chans[i], V)
        p = ops.KnnConvPlan(t[f"l{i}_knn_idx_pad"], t[f"l{i}_tap"], int(t[f"l{i}_n_in"]), V, chans[i], chans[i + 1])
        plans.append(p); ws.append(w); wts.append(p.pack_weights(torch.from_numpy(w).cuda()))

    def run(xin):
        h = ops.pack_points(torch.from_numpy(xin).cuda(), plans[0])
        acts = []
        for i in range(5):
            h = plans[i].forward(h, wts[i], torch.zeros(chans[i + 1], device="cuda"), relu=i < 4, batch=xin.shape[0])
            plans[i].check()
            acts.append(h)
        return acts
    acts = run(x)
    h32 = x[rows]                                                     # float32 chain of the reference formulation
    prev = torch.from_numpy(x[rows]).to(torch.bfloat16).float().numpy()
    for i in range(5):
        idx, tap, V = t[f"l{i}_knn_idx_pad"], t[f"l{i}_tap"].astype(np.int64), int(t[f"l{i}_V"])
        wb = torch.from_numpy(ws[i]).to(torch.bfloat16).float().numpy()
        want = c_oracle.knnconv_forward_closed_form(prev, idx, tap, V, wb, np.zeros(chans[i + 1], f32), relu=i < 4)
        got = acts[i][rows].float().permute(0, 2, 1).cpu().numpy()
        assert np.abs(got - want).max() <= 1e-2 * max(1.0, np.abs(want).max()), i          # bf16 output rounding only
        prev = got
        h32 = c_oracle.knnconv_forward_closed_form(h32, idx, tap, V, ws[i], np.zeros(chans[i + 1], f32), relu=i < 4)
    assert rel_l2(prev, h32) < 1e-2
    alone = run(x[rows])[-1]
    assert torch.equal(alone, acts[-1][rows])
    assert torch.equal(run(x)[-1], acts[-1])                          # run-to-run determinism


def test_config5_patch_embedding_wide(golden):
    """ViT-H-sized foveated patch embedding 3 -> 1280 (five c_out tiles) on 1024 images x 2 fixations of sensor output."""
    from fovi_b200 import ops
    g = golden("config4_patch_embed_p8.npz")
    V, n_in = int(g["V"]), int(g["n_in"])
    w = kaiming_weight(np.random.RandomState(1), 1280, 3, V)
    b = (0.1 * np.random.RandomState(2).standard_normal(1280)).astype(f32)
    plan = ops.KnnConvPlan(g["knn_idx_pad"], g["tap"], n_in, V, 3, 1280)
    wt = plan.pack_weights(torch.from_numpy(w).cuda())
    rows = 2048
    x = np.random.RandomState(0).random_sample((rows, 3, n_in)).astype(f32)
    y = plan.forward(ops.pack_points(torch.from_numpy(x).cuda(), plan), wt, torch.from_numpy(b).cuda(), out_dtype=torch.float32, batch=rows)
    plan.check()
    pick = [0, 127, 128, 1000, 2047]
    want = c_oracle.knnconv_forward_closed_form(x[pick], g["knn_idx_pad"], g["tap"].astype(np.int64), V, w, b)
    assert rel_l2(y[pick].permute(0, 2, 1).cpu().numpy(), want) < 1e-2
