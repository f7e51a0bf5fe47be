#!/usr/bin/env python
"""Benchmark of the foveated hot path on B200: sensor sampling of F fixations per image followed by
the fovi-AlexNet-shaped KNNConv stack.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extras]

A step = one pass of the hot path over one batch: `--batch` images of 3x256x256 (float32, uniform
[0,1), synthetic) x `--fixations` fixations -> sensor (a=1, ~4010 points, bilinear, zeros padding)
-> KNNConv 3->64->192->384->256->256 with ReLU between layers (bf16 operands, fp32 accumulation).
`value` is image x fixations per second with the images resident in HBM; `e2e` is the same metric
through the public module API with pinned HOST images in and the final activations copied back to the
host inside the timed region (`e2e_bf16_in` / `e2e_u8_in`: the same with bf16 / uint8 host images;
`e2e_copy_floor_ms`: the copies alone).  With N > 1 every rank runs its own batch (weak scaling, no collective on the path); times
are the max over ranks; the one collective the path has, the all-gather of final outputs, is timed
separately after the loop.  `extras` (one GPU) holds the other workloads of the task: the sampler sweep,
the exact float32 layer, the patch embeddings, a training step, the shipped AlexNet backbone, and the
reference's own formulation in PyTorch eager on the same GPU.
"""
import argparse
import hashlib
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CHANS = [3, 64, 192, 384, 256, 256]
# dram__bytes_read.sum + dram__bytes_write.sum per launch from one ncu capture of this workload (256 images x 4 fixations,
# captured directly: three metrics, one pass); sampler, then the five KNNConv launches.  `sources` is the hash of the kernel
# sources the capture was taken on: when the sources change the figure is reported as null until the capture is redone.
NCU_DRAM_TRAFFIC_MB = {"workload": (256, 4), "sources": "755e5d3a984b21c1", "sampler": 208.1, "conv": [220.2, 196.7, 225.7, 284.3, 207.0]}
METRIC = "images x fixations/s through sensor+KNNConv"
UNIT = "img*fix/s"


FOV, CMF_A, STRIDES, KS = 16, 1.0, [2, 2, 1, 1, 1], [121, 25, 9, 9, 9]


def kernel_sources_hash():
    h = hashlib.sha256()
    d = os.path.join(ROOT, "fovi_b200", "csrc")
    for f in sorted(os.listdir(d)):
        if f.endswith((".cu", ".cuh")):
            h.update(open(os.path.join(d, f), "rb").read())
    return h.hexdigest()[:16]


def layer_geometry():
    """Point sets and (K, reference-frame side) of the five layers, built by the package's host geometry
    exactly as fovi's KNNAlexNet chains them (auto-matched to a 64x64 cartesian budget)."""
    from fovi_b200.coords import auto_match_num_coords, get_in_out_coords
    in_res, cart_res = auto_match_num_coords(FOV, CMF_A, 64, "isotropic", 1)
    out = []
    for i in range(5):
        ic, oc, out_cart = get_in_out_coords(in_res, FOV, CMF_A, STRIDES[i], auto_match_cart_resources=1, in_cart_res=cart_res)
        out.append((ic, oc, KS[i], int(np.ceil(2 * np.sqrt(KS[i])))))
        in_res, cart_res = oc.resolution, out_cart
    return out


def make_weights(geo):
    rs = np.random.RandomState(1)
    return [(rs.standard_normal((CHANS[i + 1], CHANS[i] * side * side)) * np.sqrt(2.0 / (CHANS[i] * side * side))).astype(np.float32)
            for i, (_, _, _, side) in enumerate(geo)]


def sampler_algorithmic_bytes(grid_xy, fix_rc, H, W, size, C, in_bytes, out_bytes, mode="bilinear", border=False):
    """Algorithmic bytes of the sampler per image x fixation: C * (U * in_bytes + N * out_bytes), U = distinct
    in-image source pixels under the footprints (2x2 bilinear, 1x1 nearest; computed here in float64: the count does not
    depend on the last bit).  fix_rc [M,2] normalised (row, col); square fixation windows of `size` pixels.
    Returns (bytes, mean U)."""
    total_u = 0
    for r, c in fix_rc:
        ix = grid_xy[:, 0] * (size / 2) + c * W - 0.5
        iy = grid_xy[:, 1] * (size / 2) + r * H - 0.5
        if border:
            ix, iy = np.clip(ix, 0, W - 1), np.clip(iy, 0, H - 1)
        if mode == "bilinear":
            x0, y0 = np.floor(ix).astype(np.int64), np.floor(iy).astype(np.int64)
            xx = np.concatenate([x0, x0 + 1, x0, x0 + 1]); yy = np.concatenate([y0, y0, y0 + 1, y0 + 1])
        else:
            xx, yy = np.rint(ix).astype(np.int64), np.rint(iy).astype(np.int64)
        ok = (xx >= 0) & (xx < W) & (yy >= 0) & (yy < H)
        total_u += np.unique(yy[ok] * W + xx[ok]).size
    mean_u = total_u / len(fix_rc)
    return C * (mean_u * in_bytes + grid_xy.shape[0] * out_bytes), mean_u


def workload_name(args):
    return (f"sensor(a=1,N=4010,bilinear,zeros) x {args.fixations} fixations on {args.batch}x3x256x256 fp32 images "
            f"+ KNNConv stack 3-64-192-384-256-256 (K=121,25,9,9,9; bf16, fp32 accumulate)")


class ClockSampler:
    """Polls NVML (read-only queries) every ~5 ms in a thread during the timed region: SM clock,
    power, and the clock-event (throttle) reasons."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index, self.sm, self.pw, self.mask, self.max_sm = index, [], [], 0, None
        self._stop = threading.Event()
        self._thread = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(nvml_index(self.index))
            self.max_sm = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:
            return

        def poll():
            while not self._stop.is_set():
                try:
                    self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    self.pw.append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
                    self.mask |= int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h))
                except Exception:
                    pass
                time.sleep(0.005)
        self._thread = threading.Thread(target=poll, daemon=True)
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"]}
        self._thread.join()
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.max_sm,
                "power_w_max": max(self.pw) if self.pw else None, "samples": len(self.sm),
                "reasons": sorted(v for k, v in self.REASONS.items() if self.mask & k)}


def nvml_index(local):
    """NVML enumerates physical devices; map through CUDA_VISIBLE_DEVICES when it lists indices."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
    if vis and all(v.strip().isdigit() for v in vis.split(",")):
        return int(vis.split(",")[local])
    return local


def bind_near_gpu(local):
    """Restrict this process to the CPU cores NVML reports as local to the GPU (a read-only topology query), so that the
    pinned host buffers allocated afterwards sit in that socket's memory.  Returns the number of cores, or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(nvml_index(local))
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64)
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


class CpuPath:
    """The oracle — a port of the reference's CPU path for this workload (C with POSIX threads when it builds,
    else NumPy) — with tables and weights set up once; `run(n_images)` does one pass on a bounded sample."""

    def __init__(self, n_fix):
        from fovi_b200 import tables
        from oracle import fovi_oracle
        self.np_oracle = fovi_oracle
        try:
            from oracle import c_oracle
            c_oracle.load()
            self.c, self.kind, self.cores = c_oracle, "C/pthreads", c_oracle.threads()
        except Exception:
            self.c, self.kind, self.cores = None, "NumPy", os.cpu_count()
        geo = layer_geometry()
        self.ws = make_weights(geo)
        self.tabs = []
        for ic, oc, k, side in geo:
            idx, _, pts, cart = tables.knn_table(ic, oc, k)
            ref, _ = tables.reference_frame(k, side)
            tap, _ = tables.tap_table(idx, pts, cart, oc, ref)
            self.tabs.append((tables.pad_token_table(idx, len(ic)).numpy().astype(np.int32), tap.numpy().astype(np.int64), side * side))
        c0 = geo[0][0].cartesian
        self.grid = np.stack([c0[:, 0].numpy(), -c0[:, 1].numpy()], 1)
        self.n_fix = n_fix

    def run(self, n_images, seed=0):
        rs = np.random.RandomState(seed)
        x = rs.random_sample((n_images, 3, 256, 256)).astype(np.float32)
        fix = (0.25 + 0.5 * rs.random_sample((n_images, self.n_fix, 2))).astype(np.float32)
        hw = np.full((n_images, self.n_fix, 2), 256, np.float32)
        t0 = time.perf_counter()
        impl = self.c if self.c is not None else self.np_oracle
        y = impl.retinal_sample(x, self.grid, fix, hw)                                              # [B,F,3,N]
        h = np.ascontiguousarray(y.transpose(1, 0, 2, 3).reshape(n_images * self.n_fix, 3, -1))     # (f b) c n
        for i in range(5):
            idx, tap, V = self.tabs[i]
            zero = np.zeros(CHANS[i + 1], np.float32)
            if self.c is not None:
                h = self.c.knnconv_forward_closed_form(h, idx, tap, V, self.ws[i], zero, relu=i < 4)
            else:
                h = self.np_oracle.knnconv_forward(h, idx, tap, V, self.ws[i], zero)
                h = np.maximum(h, 0) if i < 4 else h
        return time.perf_counter() - t0

    def sample_text(self, n_images):
        return (f"{n_images} images x {self.n_fix} fixations per pass (same sensor, tables and weights), float32, "
                f"{self.kind} port of the reference path on {self.cores} threads")


def cpu_baseline(n_fix, budget_s=10.0):
    """Times the CPU port for about `budget_s` seconds.  Returns the cpu_baseline object of the JSON line."""
    path = CpuPath(n_fix)
    n_images = 8
    path.run(n_images)                                   # warm-up (page faults, thread start)
    t0 = time.perf_counter(); times = []
    while len(times) < 3 or time.perf_counter() - t0 < budget_s:
        times.append(path.run(n_images))
    v = n_images * n_fix / float(np.median(times))
    return {"value": v, "unit": UNIT, "cores": path.cores, "kind": "port", "sample": path.sample_text(n_images)}


def run_reference(args):
    """`--impl reference`: the reference's own implementation is Python + PyTorch and cannot travel to the GPU
    box, and it has nothing to compile (no oracle/_ref), so this arm times the oracle port of its CPU path on all
    host threads.  A step = one pass over a bounded sample of the workload."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    path = CpuPath(args.fixations)
    n_images = 8
    for _ in range(max(args.warmup, 1)):
        path.run(n_images)
    times = [path.run(n_images, seed=s) for s in range(args.steps)]
    per_step = float(np.sum(times)) / args.steps
    v = n_images * args.fixations / per_step
    sample = path.sample_text(n_images)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": workload_name(args), "sample": sample},
        "cpu_baseline": {"value": v, "unit": UNIT, "cores": path.cores, "kind": "port", "sample": sample},
        "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------------------------------------------ extras (one GPU)
def _time_us(torch, fn, flush, n=20, warm=3):
    """Median / p10 / p90 in microseconds of `fn` with the L2 flushed before every call."""
    for _ in range(warm):
        fn()
    ts = []
    for _ in range(n):
        flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b) * 1e3)
    return float(np.median(ts)), float(np.percentile(ts, 10)), float(np.percentile(ts, 90))


def extra_sampler_sweep(torch, dev, flush, hbm_gbs):
    """Config 2: 512 images 3x256x256 x 4 near-centre fixations, sensors a = 1 / 2.78 / 60.94, float32 and bf16 images
    (output in the input's dtype, the reference's [B,F,C,N] layout), zeros and border padding, bilinear."""
    from fovi_b200.sensing import RetinalTransform
    B, F = 512, 4
    rs = np.random.RandomState(0)
    x32 = torch.from_numpy(rs.random_sample((B, 3, 256, 256)).astype(np.float32)).to(dev)
    x16 = x32.to(torch.bfloat16)
    fix_np = (0.25 + 0.5 * rs.random_sample((B, F, 2))).astype(np.float32)
    fix = torch.from_numpy(fix_np).to(dev)
    rows = []
    for a in (1.0, 2.78, 60.94):
        for pad in ("zeros", "border"):
            rt = RetinalTransform(resolution=64, start_res=256, fov=FOV, cmf_a=a, sampler="grid_bilinear", fixation_size=256, device=dev,
                                  padding_mode=pad)
            grid = rt.sampler.sampling_grid[0, 0].cpu().numpy().astype(np.float64)
            for name, x, nb in (("f32", x32, 4), ("bf16", x16, 2)):
                rt.dtype = x.dtype
                med, p10, p90 = _time_us(torch, lambda: rt(x, fix), flush, n=10)
                by, _ = sampler_algorithmic_bytes(grid, fix_np.reshape(-1, 2)[:64].astype(np.float64), 256, 256, 256, 3, nb, nb, border=pad == "border")
                gbs = by * B * F / (med * 1e-6) / 1e9
                rows.append({"a": a, "n_points": int(grid.shape[0]), "dtype": name, "padding": pad, "us": med, "p10": p10, "p90": p90,
                             "gbs": gbs, "frac_of_hbm": gbs / hbm_gbs})
            rt.sampler.check()
    return {"images": B, "fixations": F, "layout": "[B,F,C,N] in the image dtype", "rows": rows}


def extra_config1(torch, dev, flush):
    """Config 1: the exact float32 kernel, batch 8 of 3x224x224, sensor a=2.78 (N=3975), KNNConv 3->64, K=49, 7x7 frame."""
    from fovi_b200.knn import KNNConvLayer
    from fovi_b200.sensing import RetinalTransform
    rt = RetinalTransform(resolution=64, start_res=224, fov=FOV, cmf_a=2.78, sampler="grid_bilinear", fixation_size=224, device=dev)
    c = rt.sampler.coords
    layer = KNNConvLayer(3, 64, 49, c, c, device=dev, ref_frame_side_length=7, bias=False, precision="fp32")
    x = torch.from_numpy(np.random.RandomState(0).random_sample((8, 3, 224, 224)).astype(np.float32)).to(dev)
    with torch.no_grad():
        med_s, _, _ = _time_us(torch, lambda: rt(x, None), flush, n=10)
        xs = rt(x, None)
        med_c, _, _ = _time_us(torch, lambda: layer(xs), flush, n=10)
    flops = 8 * layer.plan.flops_per_image()
    return {"sampler_us": med_s, "knnconv_f32_us": med_c, "knnconv_gflops": flops / (med_c * 1e-6) / 1e9, "images_per_s": 8 / ((med_s + med_c) * 1e-6)}


def extra_patch_embeddings(torch, dev, flush, hbm_gbs, big):
    """Configs 4 and 5: sampler (a=2.78, res 64) + foveated patch embedding 3->D onto ~64 tokens (cart_patch_size 8, the
    reference's build) and ~278 tokens (cart_patch_size 4, closest to the 256 the task names); bandwidth-bound, so reported in
    GB/s of algorithmic bytes (image footprint in, tokens out)."""
    from fovi_b200.knn import KNNPartitioningPatchEmbedding
    from fovi_b200.sensing import RetinalTransform
    out = []
    cases = [("config4", 256, 4, 224, 384, 8), ("config4_p4", 256, 4, 224, 384, 4)]
    if big:
        cases.append(("config5", 1024, 8, 256, 1280, 8))
    for name, B, F, S, D, patch in cases:
        rt = RetinalTransform(resolution=64, start_res=S, fov=FOV, cmf_a=2.78, sampler="grid_bilinear", fixation_size=S, device=dev)
        pe = KNNPartitioningPatchEmbedding(3, D, in_res=64, fov=FOV, cmf_a=2.78, in_cart_res=64, cart_patch_size=patch, ref_frame_side_length=16,
                                           max_coord_val="auto", sample_cortex=True, bias=True, transposed=True, device=dev)
        rs = np.random.RandomState(0)
        x = torch.from_numpy(rs.random_sample((B, 3, S, S)).astype(np.float32)).to(dev).to(torch.bfloat16)
        fix_np = ((0.25 + 0.5 * rs.random_sample((B, F, 2))) if name != "config5" else rs.random_sample((B, F, 2))).astype(np.float32)
        fix = torch.from_numpy(fix_np).to(dev)
        rows = B * F
        y = torch.empty((rows, pe.plan.n_out, D), dtype=torch.bfloat16, device=dev)

        def step():
            xp, _ = rt.forward_points(x, fix, conv_plan=pe.plan)
            pe.forward_points(xp, batch=rows, out=y)
        with torch.no_grad():
            med, p10, p90 = _time_us(torch, step, flush, n=10)
            xp, _ = rt.forward_points(x, fix, conv_plan=pe.plan)
            med_pe, _, _ = _time_us(torch, lambda: pe.forward_points(xp, batch=rows, out=y), flush, n=10)
        pe.plan.check()
        grid = rt.sampler.sampling_grid[0, 0].cpu().numpy().astype(np.float64)
        by_in, _ = sampler_algorithmic_bytes(grid, fix_np.reshape(-1, 2)[:64].astype(np.float64), S, S, S, 3, 2, 0)
        by = by_in + pe.plan.n_out * D * 2
        gbs = by * rows / (med * 1e-6) / 1e9
        out.append({"name": name, "images": B, "fixations": F, "tokens": int(pe.plan.n_out), "K": int(pe._k), "D": D, "us": med, "p10": p10, "p90": p90,
                    "patch_embed_us": med_pe, "imgfix_per_s": rows / (med * 1e-6), "gbs": gbs, "frac_of_hbm": gbs / hbm_gbs,
                    "patch_embed_tflops": rows * pe.plan.flops_per_image() / (med_pe * 1e-6) / 1e12})
        del x, y, pe, rt
        torch.cuda.empty_cache()
    return out


def extra_training_step(torch, dev, stack, n0, rows):
    """Forward + backward of the config-3 stack at `rows` image x fixations in bf16 (as under the reference's autocast
    training): the stack's output receives a given upstream gradient, every layer computes its weight, bias and input
    gradients (the first layer: weight and bias)."""
    x = torch.rand(rows, 3, n0, device=dev).to(torch.bfloat16)
    for p in stack.parameters():
        p.requires_grad_(True)
    gy = None

    def step():
        nonlocal gy
        for p in stack.parameters():
            p.grad = None
        y = stack(x)
        if gy is None:
            gy = torch.randn(y.shape[0], y.shape[2], y.shape[1], device=dev).to(y.dtype).permute(0, 2, 1)   # y's layout
        y.backward(gy)
    ts = []
    for i in range(6):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); step(); b.record()
        torch.cuda.synchronize()
        if i >= 2:
            ts.append(a.elapsed_time(b))
    for p in stack.parameters():
        p.requires_grad_(False)
        p.grad = None
    return {"rows": rows, "ms": float(np.median(ts))}


def extra_alexnet(torch, dev, flush, rows):
    """The shipped foveated AlexNet backbone (a=0.5, 96/256/384/384/256 channels, pools after blocks 0, 1, 4), random weights,
    evaluation-mode batch norm folded, on `rows` sensor outputs."""
    from fovi_b200 import ops
    from fovi_b200.alexnet import KNNAlexNet
    net = KNNAlexNet(n_classes=None, device=dev, in_res=64, in_channels=3, features_per_layer=[96, 256, 384, 384, 256], stride_per_layer=[2, 1, 1, 1, 1],
                     pool_after=[0, 1, 4], k_per_layer=[121, 25, 9, 9, 9], out_res=1, auto_match_cart_resources=1, fov=16.0, cmf_a=0.5,
                     norm_type="force_batch", ref_frame_mult=2, sample_cortex=True).eval()
    n0 = net.layers[0].in_coords.shape[0]
    xp = ops.pack_points(torch.rand(rows, 3, n0, device=dev), net.layers[0].conv.plan)
    with torch.no_grad():
        med, p10, p90 = _time_us(torch, lambda: net.forward_points(xp, rows), flush, n=10)
    return {"rows": rows, "us": med, "p10": p10, "p90": p90, "imgfix_per_s": rows / (med * 1e-6)}


def extra_library_baseline(torch, dev, geo, ws, flush, images=64, n_fix=4):
    """The reference's own formulation restated in PyTorch ops and run eagerly on this GPU, bf16 like its AMP configs:
    per fixation the grid transform and F.grid_sample (fovi/sensing/samplers.py:91-112, coords.py:590-642), then per layer
    zero-pad + gather of the K neighbours, the one-hot reference-frame einsum and F.linear (fovi/arch/knn.py:484-557),
    ReLU between layers.  Same sensor, tables and weights as the benchmark; a batch that fits the one-hot intermediates."""
    import torch.nn.functional as TF
    from fovi_b200 import tables
    rs = np.random.RandomState(5)
    x = torch.from_numpy(rs.random_sample((images, 3, 256, 256)).astype(np.float32)).to(dev)
    fix = torch.from_numpy((0.25 + 0.5 * rs.random_sample((images, n_fix, 2))).astype(np.float32)).to(dev)
    c0 = geo[0][0].cartesian
    grid0 = torch.stack([c0[:, 0], -c0[:, 1]], 1).to(dev).float()[None, None]               # (1,1,N,2) = (x, -y)
    layers = []
    for i, (ic, oc, k, side) in enumerate(geo):
        idx, _, pts, cart = tables.knn_table(ic, oc, k)
        ref, _ = tables.reference_frame(k, side)
        tap, _ = tables.tap_table(idx, pts, cart, oc, ref)
        pad_tok = tables.pad_token_table(idx, len(ic)).to(dev)                                # [K, n_out], pad == n_in
        rf = torch.zeros(tap.shape[0], tap.shape[1], side * side)
        rf.scatter_(2, tap.long().unsqueeze(2), 1)
        layers.append((pad_tok, rf.to(dev).to(torch.bfloat16), torch.from_numpy(ws[i]).to(dev).to(torch.bfloat16), k))

    def forward():
        B = x.shape[0]
        outs = []
        for f in range(n_fix):
            g = grid0.repeat(B, 1, 1, 1).clone()
            g[..., 0] = (g[..., 0] * (256 / 2) + fix[:, f, 1].view(B, 1, 1) * 256) * 2 / 256 - 1
            g[..., 1] = (g[..., 1] * (256 / 2) + fix[:, f, 0].view(B, 1, 1) * 256) * 2 / 256 - 1
            outs.append(TF.grid_sample(x, g, mode="bilinear", align_corners=False)[:, :, 0])   # [B,3,N]
        h = torch.stack(outs, 0).reshape(n_fix * B, 3, -1).to(torch.bfloat16)                  # (f b) c n
        for i, (pad_tok, rf, w, k) in enumerate(layers):
            b, d, n_in = h.shape
            hp = torch.cat([h, torch.zeros(b, d, 1, device=dev, dtype=h.dtype)], 2)
            kf = torch.gather(hp, 2, pad_tok.reshape(1, 1, -1).expand(b, d, -1)).reshape(b, d, k, -1)
            kf = kf.permute(0, 1, 3, 2).reshape(b * d, kf.shape[3], k)                         # (b d) n k
            kf = torch.einsum("ank,nkv->anv", kf, rf)
            kf = kf.reshape(b, d, kf.shape[1], kf.shape[2]).permute(0, 2, 1, 3).reshape(b, kf.shape[1], -1)   # b n (d v)
            h = TF.linear(kf, w).transpose(1, 2)
            if i < len(layers) - 1:
                h = torch.relu(h)
        return h
    with torch.no_grad():
        forward(); forward()
        torch.cuda.synchronize()
        ts = []
        for _ in range(5):
            flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(); forward(); b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
    ms = float(np.median(ts))
    del layers
    torch.cuda.empty_cache()
    return {"kind": "PyTorch eager on this GPU, the reference's formulation (grid_sample + gather + one-hot einsum + linear), bf16",
            "images": images, "fixations": n_fix, "ms": ms, "value": images * n_fix / (ms * 1e-3), "unit": UNIT}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--batch", type=int, default=256, help="images per GPU per step")
    ap.add_argument("--fixations", type=int, default=4)
    ap.add_argument("--chunks", type=int, default=8, help="chunks of the host->device->host pipeline (e2e)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the additional workloads (they run on one GPU only)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
    cores_bound = bind_near_gpu(local)          # before any pinned allocation

    import torch
    import torch.distributed as dist
    from fovi_b200 import ops
    from fovi_b200.dist import all_gather_rows
    from fovi_b200.knn import KNNConvLayer, KNNConvStack
    from fovi_b200.pipeline import FoveatedFrontEnd
    from fovi_b200.sensing import RetinalTransform

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    warmup = max(args.warmup, 3)

    # ---- the model of the workload, through the public module API
    geo = layer_geometry()
    ws = make_weights(geo)
    retina = RetinalTransform(resolution=64, start_res=256, fov=FOV, cmf_a=CMF_A, sampler="grid_bilinear", fixation_size=256, device=dev)
    layers = []
    for i, (ic, oc, k, side) in enumerate(geo):
        L = KNNConvLayer(CHANS[i], CHANS[i + 1], k, ic, oc, device=dev, ref_frame_side_length=side, bias=True)
        L.weight.data.copy_(torch.from_numpy(ws[i]))
        layers.append(L)
    stack = KNNConvStack(layers)
    front = FoveatedFrontEnd(retina, stack)
    plans = [L.plan for L in layers]

    B, F = args.batch, args.fixations
    M = B * F
    rs = np.random.RandomState(1000 + rank)
    x_host = torch.from_numpy(rs.random_sample((B, 3, 256, 256)).astype(np.float32)).pin_memory()
    x_host16 = x_host.to(torch.bfloat16).pin_memory()
    x_host8 = (x_host * 255).round().to(torch.uint8).pin_memory()      # what a data loader holds before its float conversion
    fix_host = torch.from_numpy((0.25 + 0.5 * rs.random_sample((B, F, 2))).astype(np.float32)).pin_memory()
    x_dev, fix_dev = x_host.to(dev), fix_host.to(dev)
    out_host = torch.empty((B, F, plans[-1].n_out, CHANS[-1]), dtype=torch.bfloat16).pin_memory()
    out_dev = torch.empty((M, plans[-1].n_out, CHANS[-1]), dtype=torch.bfloat16, device=dev)
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB L2

    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    kernel_events = []

    def device_step(record):
        if record is None:
            return front.forward(x_dev, fix_dev, out=out_dev)
        marks = [ev() for _ in range(7)]
        marks[0].record()
        y = front.forward(x_dev, fix_dev, between=lambda i: marks[i + 1].record(), out=out_dev)
        record.append(marks)
        return y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, n_warm, record=None):
        """Returns (total ms of `steps` steps: max over ranks, launches, this rank's per-step ms)."""
        for _ in range(n_warm):
            flush.zero_(); fn(None)
        barrier()
        l0 = ops.launch_count()
        pairs = []
        for _ in range(steps):
            flush.zero_()                       # L2 flush between timed iterations (outside the timed events)
            a, b = ev(), ev()
            a.record(); fn(record); b.record()  # no host sync inside the loop: the host stays ahead of the GPU
            pairs.append((a, b))
        launches = ops.launch_count() - l0
        barrier()
        per = [a.elapsed_time(b) for a, b in pairs]
        tt = torch.tensor([sum(per)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item()), launches, per

    def spread(per):
        return {"median": float(np.median(per)), "p10": float(np.percentile(per, 10)), "p90": float(np.percentile(per, 90))}

    clocks = ClockSampler(local)
    clocks.start()
    # `value`: the step with nothing between its launches (an event between two kernels would stop the next kernel's
    # prologue from overlapping the tail of the previous one); then a second pass with an event after every launch for
    # the per-kernel durations the roofline figures use.
    ms_total, launches, per_step = timed(lambda _r: device_step(None), args.steps, warmup)
    timed(device_step, min(args.steps, 20), 1, kernel_events)
    clk = clocks.stop()
    ms_e2e, _, per_e2e = timed(lambda _r: front.run_from_host(x_host, fix_host, out_host, chunks=args.chunks), args.steps, 3)
    for p in plans:
        p.check()
    retina.sampler.check()
    # the pipelined host path and the device path compute the same thing
    y_dev = front.forward(x_dev, fix_dev).view(F, B, plans[-1].n_out, CHANS[-1])
    torch.cuda.synchronize()
    e2e_matches = bool(torch.equal(y_dev.permute(1, 0, 2, 3).cpu(), out_host))
    ms_floor, _, _ = timed(lambda _r: front.run_from_host(x_host, fix_host, out_host, chunks=args.chunks, kernels=False), min(args.steps, 20), 2)
    ms_e2e16, _, per_e2e16 = timed(lambda _r: front.run_from_host(x_host16, fix_host, out_host, chunks=args.chunks), args.steps, 3)
    y16 = front.forward(x_host16.to(dev), fix_dev).view(F, B, plans[-1].n_out, CHANS[-1])
    torch.cuda.synchronize()
    e2e16_matches = bool(torch.equal(y16.permute(1, 0, 2, 3).cpu(), out_host))
    ms_floor16, _, _ = timed(lambda _r: front.run_from_host(x_host16, fix_host, out_host, chunks=args.chunks, kernels=False), min(args.steps, 20), 2)
    del y16
    ms_e2e8, _, per_e2e8 = timed(lambda _r: front.run_from_host(x_host8, fix_host, out_host, chunks=args.chunks), args.steps, 3)
    y8 = front.forward(x_host8.to(dev), fix_dev).view(F, B, plans[-1].n_out, CHANS[-1])
    torch.cuda.synchronize()
    e2e8_matches = bool(torch.equal(y8.permute(1, 0, 2, 3).cpu(), out_host))
    del y8

    # ---- the one collective of the path (N > 1): all-gather of the final outputs, and of a [rows, 1280] bf16 block shaped
    # like the CLS embeddings of the ViT-H configuration; verified, timed apart from `value`
    gather = None
    strong = None
    if world > 1:
        y_local = front.forward(x_dev, fix_dev, out=out_dev)
        cls = torch.from_numpy(np.random.RandomState(7000 + rank).standard_normal((1024 * 8 // world, 1280)).astype(np.float32)).to(dev).to(torch.bfloat16)
        res = {}
        for name, t in (("final_outputs", y_local), ("cls_1280", cls)):
            all_gather_rows(t, total_rows=t.shape[0] * world)          # warm-up
            barrier()
            a, b = ev(), ev()
            a.record(); g = all_gather_rows(t, total_rows=t.shape[0] * world); b.record()
            barrier()
            tt = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            rows_r = t.shape[0]
            ok = bool(torch.equal(g[rank * rows_r:(rank + 1) * rows_r], t))
            if name == "cls_1280":      # every rank's block can be regenerated from its seed
                for r in range(world):
                    want = torch.from_numpy(np.random.RandomState(7000 + r).standard_normal((rows_r, 1280)).astype(np.float32)).to(dev).to(torch.bfloat16)
                    ok = ok and bool(torch.equal(g[r * rows_r:(r + 1) * rows_r], want))
            else:                       # checksums of every rank's own block against the gathered copy
                sums = torch.zeros(world, dtype=torch.float64, device=dev)
                sums[rank] = t.double().sum()
                dist.all_reduce(sums)
                got = torch.stack([g[r * rows_r:(r + 1) * rows_r].double().sum() for r in range(world)])
                ok = ok and bool(torch.equal(sums, got))
            okt = torch.tensor([1 if ok else 0], device=dev)
            dist.all_reduce(okt, op=dist.ReduceOp.MIN)
            nbytes = t.numel() * t.element_size() * world
            ms = float(tt.item())
            res[name] = {"ms": ms, "bytes_gathered_per_rank": nbytes, "bus_gbs": nbytes * (world - 1) / world / (ms * 1e-3) / 1e9, "verified": bool(okt.item())}
            del g
        gather = res
        # strong scaling: one global batch of 256 images x 4 fixations cut into `world` shards
        Bs = max(1, 256 // world)
        xs, fs = x_dev[:Bs].contiguous(), fix_dev[:Bs].contiguous()
        outs = torch.empty((Bs * F, plans[-1].n_out, CHANS[-1]), dtype=torch.bfloat16, device=dev)
        ms_s, _, _ = timed(lambda _r: front.forward(xs, fs, out=outs), min(args.steps, 20), 3)
        strong = {"global_images": Bs * world, "rows_per_gpu": Bs * F, "ms_per_step": ms_s / min(args.steps, 20),
                  "value": Bs * world * F * min(args.steps, 20) / (ms_s * 1e-3), "unit": UNIT,
                  "note": "at 128 rows or fewer per GPU the 64-channel layers leave the CTA-pair kernel (one 128-row batch tile per item)"}

    # per-kernel times from the events recorded inside the timed steps
    per = np.zeros(6)
    for marks in kernel_events:
        for i in range(6):
            per[i] += marks[i].elapsed_time(marks[i + 1])
    per /= max(len(kernel_events), 1)                      # ms per launch: [sampler, conv0..conv4]
    flops = [M * p.flops_per_image() for p in plans]
    peaks = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "src": "fallback"}
    pk = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(pk):
        d = json.load(open(pk))
        # the conv launches are 0.1-0.4 ms bursts inside a ~1 ms step: if the sampled SM clock stayed at its
        # maximum the burst figure is the denominator, otherwise the sustained one
        burst = clk["sm_mhz"] is not None and clk["sm_max_mhz"] and clk["sm_mhz"] >= 0.95 * clk["sm_max_mhz"]
        peaks = {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"] if burst else d["bf16_tflops_sustained"],
                 "src": "measured (burst)" if burst else "measured (sustained)"}
    conv_ms = per[1:].sum()
    conv_tflops = sum(flops) / (conv_ms * 1e-3) / 1e12
    layer_rows = [{"layer": i, "ms": float(per[i + 1]), "tflops": flops[i] / (per[i + 1] * 1e-3) / 1e12} for i in range(5)]
    # the dominant kernel: the CTA-pair tensor-core kernel that runs the four 64-channel layers (about 3/4 of the step)
    pair_layers = [i for i in range(5) if CHANS[i] % 64 == 0 and M > 128]
    dom_ms = float(sum(per[i + 1] for i in pair_layers)) or conv_ms
    dom_flops = float(sum(flops[i] for i in pair_layers)) or float(sum(flops))
    dom_tflops = dom_flops / (dom_ms * 1e-3) / 1e12
    n_dom = max(len(pair_layers), 1)

    extras = None
    if world == 1 and not args.no_extras:
        extras = {}
        n0 = geo[0][0].shape[0]
        for name, fn in (
            ("sampler_sweep", lambda: extra_sampler_sweep(torch, dev, flush, peaks["hbm_gbs"])),
            ("config1_fp32", lambda: extra_config1(torch, dev, flush)),
            ("patch_embeddings", lambda: extra_patch_embeddings(torch, dev, flush, peaks["hbm_gbs"], big=True)),
            ("training_step", lambda: extra_training_step(torch, dev, stack, n0, M)),
            ("alexnet_backbone", lambda: extra_alexnet(torch, dev, flush, M)),
            ("library_baseline", lambda: extra_library_baseline(torch, dev, geo, ws, flush)),
        ):
            try:
                extras[name] = fn()
            except Exception as e:          # an extra that cannot run here must not take the headline down with it
                extras[name] = {"error": f"{type(e).__name__}: {e}"[:300]}
            torch.cuda.empty_cache()

    if rank == 0:
        fx = fix_host.numpy().reshape(-1, 2)[:64]
        grid = retina.sampler.sampling_grid[0, 0].cpu().numpy().astype(np.float64)
        samp_bytes_per, mean_u = sampler_algorithmic_bytes(grid, fx.astype(np.float64), 256, 256, 256, 3, 4, 2)
        sampler_gbs = samp_bytes_per * M / (per[0] * 1e-3) / 1e9
        value = world * M * args.steps / (ms_total * 1e-3)
        e2e = world * M * args.steps / (ms_e2e * 1e-3)
        e2e16 = world * M * args.steps / (ms_e2e16 * 1e-3)
        e2e8 = world * M * args.steps / (ms_e2e8 * 1e-3)
        fresh = NCU_DRAM_TRAFFIC_MB["sources"] == kernel_sources_hash() and (B, F) == NCU_DRAM_TRAFFIC_MB["workload"] and NCU_DRAM_TRAFFIC_MB["conv"]
        floor_steps = min(args.steps, 20)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_total / args.steps, "ms_per_step_spread": spread(per_step), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_name(args), "images_per_gpu": B, "fixations": F, "l2": "flushed between steps (192 MB write)",
                       "cpu_cores_bound_near_gpu": cores_bound},
            "roofline": {"bound": "tensor", "kernel": f"fovi_knnconv_tc_pair_kernel ({n_dom} launches per step: layers {pair_layers})",
                         "achieved": dom_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": dom_tflops / peaks["bf16_tflops"],
                         "traffic": (sum(NCU_DRAM_TRAFFIC_MB["conv"][i] for i in pair_layers) / n_dom * 1e6) if fresh and pair_layers else None,
                         "traffic_note": "DRAM bytes per launch, mean over this kernel's launches (ncu dram read+write; null when the kernel sources "
                                         "or the workload differ from the ones the capture was taken on)",
                         "peak_source": peaks["src"], "flops_per_launch_avg": dom_flops / n_dom, "ms_per_launch_avg": dom_ms / n_dom},
            "roofline_all_knnconv": {"kernel": "all five KNNConv launches (first layer: fovi_knnconv_tc_kernel<PAIRS>)", "achieved": conv_tflops,
                                     "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": conv_tflops / peaks["bf16_tflops"], "ms": float(conv_ms)},
            "layers": layer_rows,
            "sampler": {"kernel": "fovi_sample_strip_kernel", "ms": float(per[0]), "algorithmic_bytes_per_imgfix": samp_bytes_per, "mean_unique_pixels": mean_u,
                        "gbs": sampler_gbs, "frac_of_hbm": sampler_gbs / peaks["hbm_gbs"],
                        "traffic": NCU_DRAM_TRAFFIC_MB["sampler"] * 1e6 if fresh and NCU_DRAM_TRAFFIC_MB["sampler"] else None},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 4 + fix_host.numel() * 4, "d2h_bytes_per_step": out_host.numel() * 2,
                    "ms_per_step": ms_e2e / args.steps, "ms_per_step_spread": spread(per_e2e), "chunks": args.chunks, "matches_device_path": e2e_matches,
                    "input": "float32 host images"},
            "e2e_bf16_in": {"value": e2e16, "unit": UNIT, "h2d_bytes_per_step": x_host16.numel() * 2 + fix_host.numel() * 4,
                            "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": ms_e2e16 / args.steps, "ms_per_step_spread": spread(per_e2e16),
                            "matches_device_path": e2e16_matches, "input": "bfloat16 host images"},
            "e2e_u8_in": {"value": e2e8, "unit": UNIT, "h2d_bytes_per_step": x_host8.numel() + fix_host.numel() * 4, "d2h_bytes_per_step": out_host.numel() * 2,
                          "ms_per_step": ms_e2e8 / args.steps, "ms_per_step_spread": spread(per_e2e8), "matches_device_path": e2e8_matches,
                          "input": "uint8 host images (sampled as the float32 values 0..255 they hold)"},
            "e2e_copy_floor_ms": {"float32_in": ms_floor / floor_steps, "bf16_in": ms_floor16 / floor_steps,
                                  "note": "the same chunks, streams and dependencies with the kernels left out: what the host<->device copies cost "
                                          "on this machine; per-rank GB/s = (h2d + d2h bytes) / this",
                                  "gbs_per_rank_float32_in": (x_host.numel() * 4 + out_host.numel() * 2) / (ms_floor / floor_steps * 1e-3) / 1e9},
            "gpu_launches": int(launches), "clocks": clk,
        }
        if gather is not None:
            line["allgather"] = gather
        if strong is not None:
            line["strong"] = strong
        if extras is not None:
            line["extras"] = extras
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(F)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
