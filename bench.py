#!/usr/bin/env python
"""Benchmark of the foveated hot path on B200: sensor sampling of F fixations per image followed by
the fovi-AlexNet-shaped KNNConv stack.  Prints ONE JSON line (rank 0).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step = one pass of the hot path over one batch: `--batch` images of 3x256x256 (float32, uniform
[0,1), synthetic) x `--fixations` fixations -> sensor (a=1, ~4010 points, bilinear, zeros padding)
-> KNNConv 3->64->192->384->256->256 with ReLU between layers (bf16 operands, fp32 accumulation).
`value` is image x fixations per second with the images resident in HBM; `e2e` is the same metric
through the public module API with pinned HOST images in and the final activations copied back to the
host inside the timed region.  With N > 1 every rank runs its own batch (weak scaling, no collective
on the path); times are the max over ranks.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CHANS = [3, 64, 192, 384, 256, 256]
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from one ncu capture of this workload at its default size
# (256 images x 4 fixations; profiles/dram_traffic_bench_default.md): sampler, then the five KNNConv launches.
NCU_DRAM_TRAFFIC_MB = {"sampler": 239.5, "conv": [220.6, 197.2, 226.0, 286.3, 206.8]}
METRIC = "images x fixations/s through sensor+KNNConv"
UNIT = "img*fix/s"


FOV, CMF_A, STRIDES, KS = 16, 1.0, [2, 2, 1, 1, 1], [121, 25, 9, 9, 9]


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


def sampler_algorithmic_bytes(grid_xy, fix_rc, H, W, size, C, in_bytes, out_bytes):
    """Algorithmic bytes of the bilinear sampler per image x fixation: C * (U * in_bytes + N * out_bytes), U = distinct
    in-image source pixels under the 2x2 footprints (computed here in float64; the count does not depend on the last bit).
    fix_rc [M,2] normalised (row, col); square fixation windows of `size` pixels.  Returns (bytes, mean U)."""
    total_u = 0
    for r, c in fix_rc:
        ix = grid_xy[:, 0] * (size / 2) + c * W - 0.5
        iy = grid_xy[:, 1] * (size / 2) + r * H - 0.5
        x0, y0 = np.floor(ix).astype(np.int64), np.floor(iy).astype(np.int64)
        xx = np.concatenate([x0, x0 + 1, x0, x0 + 1]); yy = np.concatenate([y0, y0, y0 + 1, y0 + 1])
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
            # NVML enumerates physical devices; map through CUDA_VISIBLE_DEVICES when it lists indices
            vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            idx = self.index
            if vis and all(v.strip().isdigit() for v in vis.split(",")):
                idx = int(vis.split(",")[self.index])
            h = pynvml.nvmlDeviceGetHandleByIndex(idx)
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
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist
    from fovi_b200 import ops
    from fovi_b200.knn import KNNConvLayer, KNNConvStack
    from fovi_b200.pipeline import FoveatedFrontEnd
    from fovi_b200.sensing import RetinalTransform

    rank = int(os.environ.get("RANK", "0")); world = int(os.environ.get("WORLD_SIZE", "1")); local = int(os.environ.get("LOCAL_RANK", "0"))
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
    front = FoveatedFrontEnd(retina, KNNConvStack(layers))
    plans = [L.plan for L in layers]

    B, F = args.batch, args.fixations
    M = B * F
    rs = np.random.RandomState(1000 + rank)
    x_host = torch.from_numpy(rs.random_sample((B, 3, 256, 256)).astype(np.float32)).pin_memory()
    fix_host = torch.from_numpy((0.25 + 0.5 * rs.random_sample((B, F, 2))).astype(np.float32)).pin_memory()
    x_dev, fix_dev = x_host.to(dev), fix_host.to(dev)
    out_host = torch.empty((F, B, plans[-1].n_out, CHANS[-1]), dtype=torch.bfloat16).pin_memory()
    flush = torch.empty(192 * 1024 * 1024, dtype=torch.uint8, device=dev)   # > 126 MB L2

    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    kernel_events = []

    def device_step(record):
        if record is None:
            return front.forward(x_dev, fix_dev)
        marks = [ev() for _ in range(7)]
        marks[0].record()
        y = front.forward(x_dev, fix_dev, between=lambda i: marks[i + 1].record())
        record.append(marks)
        return y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, n_warm, record=None):
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
        t = sum(a.elapsed_time(b) for a, b in pairs)
        tt = torch.tensor([t], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item()), launches

    clocks = ClockSampler(local)
    clocks.start()
    # `value`: the step with nothing between its launches (an event between two kernels would stop the next kernel's
    # prologue from overlapping the tail of the previous one); then a second pass with an event after every launch for
    # the per-kernel durations the roofline figures use.
    ms_total, launches = timed(lambda _r: device_step(None), args.steps, warmup)
    timed(device_step, min(args.steps, 20), 1, kernel_events)
    clk = clocks.stop()
    ms_e2e, _ = timed(lambda _r: front.run_from_host(x_host, fix_host, out_host, chunks=args.chunks), args.steps, 3)
    for p in plans:
        p.check()
    # the pipelined host path and the device path compute the same thing
    y_dev = front.forward(x_dev, fix_dev).view(F, B, plans[-1].n_out, CHANS[-1])
    torch.cuda.synchronize()
    e2e_matches = bool(torch.equal(y_dev.cpu(), out_host))

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
        # the conv launches are 0.1-0.4 ms bursts inside a ~1.3 ms step: if the sampled SM clock stayed at its
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

    if rank == 0:
        fx = fix_host.numpy().reshape(-1, 2)[:64]
        grid = retina.sampler.sampling_grid[0, 0].cpu().numpy().astype(np.float64)
        samp_bytes_per, mean_u = sampler_algorithmic_bytes(grid, fx.astype(np.float64), 256, 256, 256, 3, 4, 2)
        sampler_gbs = samp_bytes_per * M / (per[0] * 1e-3) / 1e9
        value = world * M * args.steps / (ms_total * 1e-3)
        e2e = world * M * args.steps / (ms_e2e * 1e-3)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": ms_total / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": {"workload": workload_name(args), "images_per_gpu": B, "fixations": F, "l2": "flushed between steps (192 MB write)"},
            "roofline": {"bound": "tensor", "kernel": f"fovi_knnconv_tc_pair_kernel ({n_dom} launches per step: layers {pair_layers})",
                         "achieved": dom_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": dom_tflops / peaks["bf16_tflops"],
                         "traffic": (sum(NCU_DRAM_TRAFFIC_MB["conv"][i] for i in pair_layers) / n_dom * 1e6) if (B, F) == (256, 4) and pair_layers else None,
                         "traffic_note": "DRAM bytes per launch, mean over this kernel's launches (ncu dram read+write)", "peak_source": peaks["src"],
                         "flops_per_launch_avg": dom_flops / n_dom, "ms_per_launch_avg": dom_ms / n_dom},
            "roofline_all_knnconv": {"kernel": "all five KNNConv launches (first layer: fovi_knnconv_tc_kernel<PAIRS>)", "achieved": conv_tflops,
                                     "peak": peaks["bf16_tflops"], "unit": "TFLOP/s", "frac": conv_tflops / peaks["bf16_tflops"], "ms": float(conv_ms)},
            "layers": layer_rows,
            "sampler": {"ms": float(per[0]), "algorithmic_bytes_per_imgfix": samp_bytes_per, "mean_unique_pixels": mean_u, "gbs": sampler_gbs,
                        "frac_of_hbm": sampler_gbs / peaks["hbm_gbs"]},
            "e2e": {"value": e2e, "unit": UNIT, "h2d_bytes_per_step": x_host.numel() * 4 + fix_host.numel() * 4, "d2h_bytes_per_step": out_host.numel() * 2,
                    "ms_per_step": ms_e2e / args.steps, "chunks": args.chunks, "matches_device_path": e2e_matches},
            "gpu_launches": int(launches), "clocks": clk,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(F)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
