"""Sensor front end: drop-in counterparts of the reference's ``GridSampler``
(fovi/sensing/samplers.py:51-130) and ``RetinalTransform`` (fovi/sensing/retina.py:14-292) on the
CUDA sampler.  Same constructors, same attribute names, same ``forward`` signatures; in addition
``fix_loc`` may be ``[B,F,2]`` so that all fixations of every image are sampled in one launch
(the reference loops over fixations in Python, fovi/sensing/policies.py:266-277).

Fixation arguments given as CUDA tensors stay on the device: nothing here synchronises with the host
(the reference round-trips ``fix_loc`` through NumPy on every call, retina.py:226-235).
"""
import numpy as np
import torch
import torch.nn as nn

from . import ops
from .coords import SamplingCoords, find_desired_res

__all__ = ["GridSampler", "RetinalTransform"]

_MODES = {"nearest": ops.NEAREST, "bilinear": ops.BILINEAR}
_PADS = {"zeros": ops.PAD_ZEROS, "border": ops.PAD_BORDER}


_CONST_CACHE = {}


def _as_bf2(v, B, device, what):
    """Fixation argument -> float32 tensor [B,F,2] on `device` plus whether a fixation axis was given.
    A tensor that already is float32 [B,F,2] on the device is passed through untouched; Python numbers and
    tuples (the usual default arguments) are uploaded once and cached, so steady-state calls issue no
    host->device copy and no extra kernel."""
    if isinstance(v, torch.Tensor):
        if v.dim() == 3 and v.dtype == torch.float32 and v.device == torch.device(device) and v.is_contiguous() and v.shape[0] == B and v.shape[2] == 2:
            return v.detach(), True
        t = v.detach().to(device=device, dtype=torch.float32)
    else:
        arr = np.asarray(v, dtype=np.float32)
        if arr.size <= 2:
            key = (arr.tobytes(), arr.shape, B, str(device))
            if key not in _CONST_CACHE:
                if len(_CONST_CACHE) > 64:
                    _CONST_CACHE.clear()
                pair = np.broadcast_to(arr.reshape(-1), (2,)) if arr.size == 2 else np.full(2, arr.reshape(-1)[0], np.float32)
                _CONST_CACHE[key] = torch.as_tensor(np.ascontiguousarray(np.broadcast_to(pair, (B, 1, 2))), device=device)
            return _CONST_CACHE[key], False
        t = torch.as_tensor(arr, device=device)
    multi = False
    if t.dim() == 0:
        t = t.reshape(1, 1, 1).expand(B, 1, 2)
    elif t.dim() == 1:
        if t.shape[0] == 2:
            t = t.reshape(1, 1, 2).expand(B, 1, 2)
        elif t.shape[0] == B:                      # one scalar per image: same value for both axes
            t = t.reshape(B, 1, 1).expand(B, 1, 2)
        else:
            raise ValueError(f"{what} shape: {tuple(t.shape)}")
    elif t.dim() == 2:
        if t.shape != (B, 2):
            raise ValueError(f"{what} shape {tuple(t.shape)} does not match batch size {B}")
        t = t.reshape(B, 1, 2)
    elif t.dim() == 3:
        if t.shape[0] != B or t.shape[2] != 2:
            raise ValueError(f"{what} shape {tuple(t.shape)}: expected [{B},F,2]")
        multi = True
    else:
        raise ValueError(f"{what} shape: {tuple(t.shape)}")
    return t.contiguous(), multi


class _SampleFunction(torch.autograd.Function):
    """sampler(img) with the image gradient of the reference (autograd through F.grid_sample, samplers.py:108); the
    fixations carry no gradient."""

    @staticmethod
    def forward(ctx, img, fix_rc, fix_hw, sampler):
        ctx.sampler, ctx.shape, ctx.in_dtype = sampler, tuple(img.shape), img.dtype
        ctx.save_for_backward(fix_rc, fix_hw)
        with torch.no_grad():
            return sampler.sample(img, fix_rc, fix_hw)

    @staticmethod
    def backward(ctx, gy):
        fix_rc, fix_hw = ctx.saved_tensors
        s = ctx.sampler
        g = ops.sample_backward(s._plan, gy, ctx.shape, fix_rc, fix_hw, mode=_MODES[s.mode], pad=_PADS[s.padding_mode])
        return g.to(ctx.in_dtype), None, None, None


class GridSampler(nn.Module):
    """Nearest / bilinear sampling of an image at the sensor's points around a fixation.

    Constructor and attributes as the reference class (samplers.py:59-89): ``coords``,
    ``sampling_grid`` ``(1,1,N,2)`` holding (x, -y) of the cartesian coordinates, ``out_sampling_grid``,
    ``polar_radius``.  ``padding_mode`` ('zeros' as in the reference, or 'border') is an addition.
    """

    def __init__(self, fov, cmf_a, resolution, device="cuda", dtype=torch.float, mode="nearest", style="isotropic", coords=None,
                 padding_mode="zeros"):
        super().__init__()
        if mode not in _MODES or padding_mode not in _PADS:
            raise ValueError(f"mode {mode!r} / padding_mode {padding_mode!r} not supported")
        self.fov, self.cmf_a, self.resolution = fov, cmf_a, resolution
        self.device, self.dtype, self.mode, self.style, self.padding_mode = device, dtype, mode, style, padding_mode
        self.coords = SamplingCoords(fov, cmf_a, resolution, device=device, style=style, dtype=dtype) if coords is None else coords
        cart = self.coords.cartesian
        self.sampling_grid = torch.stack([cart[:, 0], -cart[:, 1]], 1).unsqueeze(0).unsqueeze(0)   # (x, -y): grid_sample's (x, y)
        self.out_sampling_grid = self.sampling_grid
        self.polar_radius = self.coords.polar[:, 0]
        self._plan = ops.SamplerPlan(self.sampling_grid[0, 0].detach().float().cpu().numpy(), device=torch.device(device))

    def sample(self, img, fix_rc, fix_hw, out_dtype=None, layout=ops.OUT_BFCN, channel_stride=None, out=None):
        """All fixations in one launch.  fix_rc / fix_hw: float32 CUDA [B,F,2]; see ops.sample for layouts."""
        return ops.sample(self._plan, img, fix_rc, fix_hw, mode=_MODES[self.mode], pad=_PADS[self.padding_mode],
                          out_dtype=out_dtype, layout=layout, channel_stride=channel_stride, out=out)

    def forward(self, img, fix_loc=None, fixation_size=None, return_coords=False):
        """img [B,C,H,W]; fix_loc normalised (row, col) as [B,2] (or [B,F,2]); fixation_size pixels (h, w).
        Returns [B,C,N] (or [B,F,C,N]) — samplers.py:91-112."""
        B, _, H, W = img.shape
        fix_rc, multi = _as_bf2((0.5, 0.5) if fix_loc is None else fix_loc, B, img.device, "fix_loc")
        fix_hw, _ = _as_bf2((H, W) if fixation_size is None else fixation_size, B, img.device, "fixation_size")
        if fix_hw.shape[1] != fix_rc.shape[1]:
            fix_hw = fix_hw.expand(B, fix_rc.shape[1], 2).contiguous()
        if torch.is_grad_enabled() and img.requires_grad:
            out = _SampleFunction.apply(img, fix_rc, fix_hw, self)
        else:
            out = self.sample(img, fix_rc, fix_hw)
        out = out if multi else out[:, 0]
        if return_coords:
            raise NotImplementedError("return_coords: the normalised grid is not materialised by the CUDA sampler")
        return out

    def check(self):
        """Synchronise the current stream and raise if a launch of this sampler gave up on its bounded wait."""
        self._plan.check()

    def all_coords(self, device=None):
        return self.coords.cartesian.to(self.device if device is None else device)

    def __repr__(self):
        return f"GridSampler(fov={self.fov}, cmf_a={self.cmf_a}, style={self.style}, resolution={self.resolution}, mode={self.mode}, n={len(self.coords)})"


class RetinalTransform(nn.Module):
    """Foveated sensor: constructor and forward of the reference module (retina.py:31-156) for the grid
    samplers ('grid_nn', 'grid_bilinear').  Colour decay (``sigma``), train-time ``pre/post_transforms`` and
    the pooling samplers are outside the hot path and not built: asking for them raises."""

    def __init__(self, resolution, start_res=256, fov=16, cmf_a=0.5, style="isotropic", sampler="grid_nn", fixation_size=None,
                 device="cuda", dtype=torch.float, auto_match_cart_resources=True, pre_transforms=None, post_transforms=None,
                 sigma=None, no_color_val=False, padding_mode="zeros", **kwargs):
        super().__init__()
        if sigma is not None or no_color_val or pre_transforms is not None or post_transforms is not None:
            raise NotImplementedError("colour decay, grayscale evaluation and train-time transforms are not part of the CUDA hot path")
        if sampler not in ("grid_nn", "grid_bilinear"):
            raise ValueError(f"Invalid sampler for the CUDA path: {sampler}")
        self.sigma, self.cmf_a, self.fov = sigma, cmf_a, fov
        self.fixation_size = start_res if fixation_size is None else fixation_size
        self.start_res, self.device, self.dtype = start_res, device, dtype
        if auto_match_cart_resources != 0:
            resolution, _ = find_desired_res(fov, cmf_a, resolution ** 2, style=style, force_less_than=True)
        self.resolution = self.out_size = resolution
        self.mode = f"pointcloud_{style}"
        self.reshape_as_grid = False
        self.no_color_val = no_color_val
        self.foveal_color = None
        self.pre_transforms = self.post_transforms = None
        self.sampler = GridSampler(fov, cmf_a, resolution, device=device, mode="nearest" if sampler == "grid_nn" else "bilinear",
                                   style=style, padding_mode=padding_mode)
        self.scatter_sizes = self.sampler.coords.get_scatter_sizes().cpu().numpy()
        self._hw_cache = {}

    def _defaults(self, fix_loc, fixation_size):
        if fix_loc is None:
            fix_loc = (0.5, 0.5)
        elif isinstance(fix_loc, (int, float)):
            fix_loc = (fix_loc, fix_loc)
        if fixation_size is None or (isinstance(fixation_size, str) and fixation_size == "none"):
            fixation_size = self.fixation_size
        if isinstance(fixation_size, (int, float)):
            fixation_size = (fixation_size, fixation_size)
        return fix_loc, fixation_size

    def forward(self, x, fix_loc, fixation_size=None, **kwargs):
        """x [B,C,H,W] -> [B,C,N] in ``self.dtype`` (retina.py:118-156); with fix_loc [B,F,2] -> [B,F,C,N].  Differentiable
        with respect to the images (the gradient kernel scatters onto the footprints with the forward's weights)."""
        fix_loc, fixation_size = self._defaults(fix_loc, fixation_size)
        return self.sampler(x, fix_loc=fix_loc, fixation_size=fixation_size).to(self.dtype)

    @torch.no_grad()
    def forward_points(self, x, fix_loc, fixation_size=None, conv_plan=None, out=None, row_order="fb"):
        """All fixations sampled straight into the layout the first KNNConv consumes: the pair layout when `conv_plan`
        asks for it, else channels-last [rows, N, cin_packed] bf16.  Rows are ordered '(f b)' as fovi/fovinet.py:281
        flattens them (row_order "fb"), or '(b f)' (row_order "bf": the fixations of an image next to each other, which is
        what a pipeline cutting the batch into chunks of images wants).  Returns (tensor, rows)."""
        if row_order not in ("fb", "bf"):
            raise ValueError("row_order must be 'fb' or 'bf'")
        B = x.shape[0]
        fix_rc, fix_hw = self.fixation_tensors(x, fix_loc, fixation_size)
        F = fix_rc.shape[1]
        fb = row_order == "fb"
        if conv_plan is not None and conv_plan.x_layout == ops.X_PAIRS:
            y = self.sampler.sample(x, fix_rc, fix_hw, layout=ops.OUT_FB_PAIRS if fb else ops.OUT_BF_PAIRS, out=out)
        else:
            cp = 8 if conv_plan is None else conv_plan.cin_packed
            y = self.sampler.sample(x, fix_rc, fix_hw, out_dtype=torch.bfloat16, layout=ops.OUT_FBNC if fb else ops.OUT_BFNC, channel_stride=cp, out=out)
            y = y.reshape(F * B, y.shape[2], cp)
        return y, F * B

    def fixation_tensors(self, x, fix_loc, fixation_size=None):
        """(centres, sizes) as the kernels take them: float32 [B,F,2] on x's device, defaults filled in."""
        B = x.shape[0]
        fix_loc, fixation_size = self._defaults(fix_loc, fixation_size)
        fix_rc, _ = _as_bf2(fix_loc, B, x.device, "fix_loc")
        fix_hw, _ = _as_bf2(fixation_size, B, x.device, "fixation_size")
        if fix_hw.shape[1] != fix_rc.shape[1]:
            fix_hw = self._expanded(fix_hw, B, fix_rc.shape[1])
        return fix_rc, fix_hw

    def _expanded(self, fix_hw, B, F):
        """[B,1,2] -> contiguous [B,F,2]; the result for a cached constant is cached too."""
        key = (fix_hw.data_ptr(), B, F)
        hit = self._hw_cache.get(key)
        if hit is None or hit[0] is not fix_hw:
            if len(self._hw_cache) > 16:
                self._hw_cache.clear()
            hit = (fix_hw, fix_hw.expand(B, F, 2).contiguous())
            self._hw_cache[key] = hit
        return hit[1]

    def get_warp_params(self):
        return self.fov, self.cmf_a, self.resolution, self.fixation_size
