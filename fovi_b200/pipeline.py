"""The hot path end to end: images -> sensor (all fixations) -> KNNConv stack, as one object.

``FoveatedFrontEnd(retina, stack)`` is the call a user makes for this path:

* ``forward(images, fix_loc)`` — device tensors in, device tensor out.
* ``run_from_host(images_pinned, fix_pinned, out_pinned)`` — host buffers in and out.  The batch is cut
  into chunks of images that flow through three streams (host->device copy, kernels, device->host copy)
  with double-buffered device memory, so PCIe transfers of neighbouring chunks overlap the kernels.

Rows of ``forward``'s result are ordered '(f b)' (fixation-major), the order in which the reference flattens
fixations before its network (fovi/fovinet.py:281); ``run_from_host`` writes ``[B, F, n_out, C_out]`` (the
fixations of an image together), so that a chunk of images is one contiguous block of the host buffer.
"""
import torch

from . import ops

__all__ = ["FoveatedFrontEnd"]


class FoveatedFrontEnd:
    def __init__(self, retina, stack, out_dtype=torch.bfloat16):
        self.retina, self.stack, self.out_dtype = retina, stack, out_dtype
        self.device = torch.device(retina.device)
        self._slots = {}
        self._streams = None

    @property
    def first_plan(self):
        return self.stack.layers[0].plan

    def _slot(self, key, B, F, img_shape, img_dtype):
        """Device buffers for one in-flight chunk: image, fixations, sensor output, every layer's output."""
        k = (key, B, F, tuple(img_shape), img_dtype)
        if k not in self._slots:
            dev, rows = self.device, B * F
            p0 = self.first_plan
            n_pts = len(self.retina.sampler.coords)
            if p0.x_layout == 1:
                s_out = torch.zeros(((rows + 127) // 128, (n_pts + 1) // 2, 128, 8), dtype=torch.bfloat16, device=dev)
            else:
                s_out = torch.empty((F, B, n_pts, p0.cin_packed), dtype=torch.bfloat16, device=dev)
            n = len(self.stack.layers)
            acts = [torch.empty((rows, L.plan.n_out, L.out_channels), dtype=self.out_dtype if i == n - 1 else torch.bfloat16, device=dev)
                    for i, L in enumerate(self.stack.layers)]
            self._slots[k] = dict(img=torch.empty((B,) + tuple(img_shape), dtype=img_dtype, device=dev),
                                  fix=torch.empty((B, F, 2), dtype=torch.float32, device=dev), s_out=s_out, acts=acts)
        return self._slots[k]

    def _run(self, img, fix, slot, fixation_size=None, between=None, out=None, row_order="fb"):
        """Sensor + stack on device tensors into the slot's buffers (`out`: destination of the last layer instead of
        the slot's).  `between(i)` is called after launch i (0 = sensor, 1.. = layers): the benchmark records events there."""
        B, F = fix.shape[0], fix.shape[1]
        rows = B * F
        n = len(self.stack.layers)
        L0 = self.stack.layers[0]
        first = 0
        if between is None and L0.plan.tc_supported:
            # sensor and first layer through the fused entry point: the sensor output is handed over in L2
            sampler = self.retina.sampler
            fix_rc, fix_hw = self.retina.fixation_tensors(img, fix, fixation_size)
            dst = out if (out is not None and n == 1) else slot["acts"][0]
            h, _ = ops.sample_knnconv_fused(sampler._plan, L0.plan, img, fix_rc, fix_hw, L0.packed_weight(), L0.bias, relu=(n > 1) or self.stack.final_relu,
                                            mode=ops.BILINEAR if sampler.mode == "bilinear" else ops.NEAREST,
                                            pad=ops.PAD_ZEROS if sampler.padding_mode == "zeros" else ops.PAD_BORDER,
                                            out_dtype=dst.dtype, intermediate=slot["s_out"], out=dst, row_order=row_order)
            first = 1
        else:
            h, _ = self.retina.forward_points(img, fix, fixation_size, conv_plan=self.first_plan, out=slot["s_out"], row_order=row_order)
            if between:
                between(0)
        for i, L in enumerate(self.stack.layers):
            if i < first:
                continue
            dst = out if (out is not None and i == n - 1) else slot["acts"][i]
            h = L.forward_points(h, batch=rows, relu=(i < n - 1) or self.stack.final_relu, out_dtype=dst.dtype, out=dst)
            if between:
                between(i + 1)
        return h

    @torch.no_grad()
    def forward(self, images, fix_loc, fixation_size=None, between=None, out=None):
        """images [B,C,H,W] and fix_loc [B,F,2] on the device -> [F*B, n_out, C_out] (channels last).  The result is
        newly allocated on every call (intermediate buffers are reused) unless the caller passes its own `out`."""
        B, F = images.shape[0], fix_loc.shape[1]
        slot = self._slot("dev", B, F, images.shape[1:], images.dtype)
        if out is None:
            last = self.stack.layers[-1]
            out = torch.empty((B * F, last.plan.n_out, last.out_channels), dtype=self.out_dtype, device=self.device)
        return self._run(images, fix_loc, slot, fixation_size, between, out=out)

    @torch.no_grad()
    def run_from_host(self, images, fix_loc, out, chunks=8, fixation_size=None, kernels=True):
        """images [B,C,H,W] (float32 or bfloat16), fix_loc [B,F,2] float32, out [B,F,n_out,C_out]: PINNED host tensors.
        Returns after the last byte of `out` has been written.  Per chunk of images: one host->device copy of the images
        (and one of the fixations), the kernels, one device->host copy of the chunk's result.
        `kernels=False` runs the copies alone (same chunks, same streams, same dependencies): the transfer floor of
        this pipeline on the machine at hand."""
        B, F = images.shape[0], fix_loc.shape[1]
        assert out.shape[0] == B and out.shape[1] == F, "out is [B, F, n_out, C_out]"
        chunks = max(1, min(chunks, B))
        bounds = [(c * B) // chunks for c in range(chunks + 1)]
        if self._streams is None:
            self._streams = [torch.cuda.Stream(self.device) for _ in range(3)]
        s_in, s_run, s_out = self._streams
        cur = torch.cuda.current_stream(self.device)
        for s in self._streams:
            s.wait_stream(cur)
        ev_in, ev_run, ev_out = {}, {}, {}
        for c in range(chunks):
            lo, hi = bounds[c], bounds[c + 1]
            slot = self._slot(c % 2, hi - lo, F, images.shape[1:], images.dtype)
            with torch.cuda.stream(s_in):
                if c >= 2:
                    s_in.wait_event(ev_run[c - 2])          # the kernels of chunk c-2 have consumed this slot's inputs
                slot["img"].copy_(images[lo:hi], non_blocking=True)
                slot["fix"].copy_(fix_loc[lo:hi], non_blocking=True)
                ev_in[c] = s_in.record_event()
            with torch.cuda.stream(s_run):
                s_run.wait_event(ev_in[c])
                if c >= 2:
                    s_run.wait_event(ev_out[c - 2])         # this slot's output has left for the host
                if kernels:
                    y = self._run(slot["img"], slot["fix"], slot, fixation_size, row_order="bf")
                else:
                    y = slot["acts"][-1]
                ev_run[c] = s_run.record_event()
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_run[c])
                out[lo:hi].copy_(y.view(hi - lo, F, y.shape[1], y.shape[2]), non_blocking=True)   # rows (b f): one block
                ev_out[c] = s_out.record_event()
        for s in self._streams:
            cur.wait_stream(s)
        return out
