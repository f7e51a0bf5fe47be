"""Fixation policies: where to look.  Counterparts of the reference's ``MultiRandomSaccadePolicy`` and
``NoSaccadePolicy`` (fovi/sensing/policies.py:13-340) that draw the same fixations from NumPy's global
random state (same calls in the same order, so a seeded run reproduces the reference's fixations exactly)
and then sample ALL fixations of the batch with one launch of the CUDA sensor instead of one
``RetinalTransform`` call per fixation (policies.py:266-277).

forward returns the reference's dictionary: ``x_fixs [B,F,C,N]``, ``fixations [B,F,2]``,
``fixation_sizes [B,F,2]``, ``fix_deltas [B,F,2]``.
"""
import numpy as np
import torch
import torch.nn as nn

__all__ = ["MultiRandomSaccadePolicy", "NoSaccadePolicy", "FIXATION_POLICY_REGISTRY"]


def _span(v):
    return hasattr(v, "__len__")


def _draw_near_centre(height, width, scale, ratio, reach):
    """One fixation within `reach` (normalised) of the image centre, window area/aspect drawn from `scale` / `ratio`
    when those are ranges (policies.py:90-129).  Draw order: area, aspect, row, column."""
    area = height * width
    target = area * (np.random.uniform(scale[0], scale[1]) if _span(scale) else scale)
    aspect = np.exp(np.random.uniform(*np.log(ratio))) if _span(ratio) else ratio
    w = int(round(np.sqrt(target * aspect)))
    h = int(round(np.sqrt(target / aspect)))
    lo, hi = 0.5 - reach, 0.5 + reach
    return [np.random.uniform(lo, hi), np.random.uniform(lo, hi)], [h, w]


def _draw_crop(height, width, scale, ratio):
    """One RandomResizedCrop-style window anywhere in the image, returned as (normalised centre, size); up to ten
    attempts, then the largest centred window with an allowed aspect (policies.py:36-88)."""
    area = height * width
    for _ in range(10):
        target = area * (np.random.uniform(scale[0], scale[1]) if _span(scale) else scale)
        aspect = np.exp(np.random.uniform(*np.log(ratio))) if _span(ratio) else ratio
        w = int(np.round(np.sqrt(target * aspect)))
        h = int(np.round(np.sqrt(target / aspect)))
        if 0 < w <= width and 0 < h <= height:
            i = int(np.random.uniform(0, height - h + 1))
            j = int(np.random.uniform(0, width - w + 1))
            return [(i + h / 2) / height, (j + w / 2) / width], [h, w]
    lo, hi = (min(ratio), max(ratio)) if _span(ratio) else (ratio, ratio)
    in_ratio = float(width) / float(height)
    if in_ratio < lo:
        w, h = width, int(round(width / lo))
    elif in_ratio > hi:
        h, w = height, int(round(height * hi))
    else:
        w, h = width, height
    i, j = (height - h) // 2, (width - w) // 2
    return [(i + h / 2) / height, (j + w / 2) / width], [h, w]


class MultiRandomSaccadePolicy(nn.Module):
    """Several random fixations per image (constructor as policies.py:185-220)."""

    def __init__(self, retinal_transform, n_fixations=2, crop_area_range=[0.08, 1], add_aspect_variation=False, nonrandom_val=False,
                 val_crop_size=1, nonrandom_first=False, norm_dist_from_center=None):
        super().__init__()
        self.retinal_transform, self.n_fixations = retinal_transform, n_fixations
        self.fixation_size, self.dtype, self.device = retinal_transform.fixation_size, retinal_transform.dtype, retinal_transform.device
        self.crop_area_range = crop_area_range
        self.crop_aspect_range = [3 / 4, 4 / 3] if add_aspect_variation else 1
        self.val_crop_size, self.nonrandom_val, self.nonrandom_first = val_crop_size, nonrandom_val, nonrandom_first
        self.norm_dist_from_center = norm_dist_from_center
        self.multi_policy = True

    def draw(self, img_size, batch, n_fixations, area_range=None):
        """Fixation centres float32 [B,F,2] and window sizes int64 [B,F,2] (h, w), consuming ``np.random`` exactly as the
        reference does: fixation index outermost, image innermost (policies.py:248-253, 131-164)."""
        if area_range is None:
            area_range = self.crop_area_range if self.training else self.val_crop_size
        ratio = self.crop_aspect_range if self.training else 1
        H, W = img_size
        fix = np.empty((batch, n_fixations, 2), np.float64)
        size = np.empty((batch, n_fixations, 2), np.int64)
        for f in range(n_fixations):
            for b in range(batch):
                if self.norm_dist_from_center is not None:
                    fix[b, f], size[b, f] = _draw_near_centre(H, W, area_range, ratio, self.norm_dist_from_center)
                else:
                    fix[b, f], size[b, f] = _draw_crop(H, W, area_range, ratio)
        return fix.astype(np.float32), size

    @torch.no_grad()
    def forward(self, x, n_fixations=None, fixations=None, fixation_size=None, area_range=None):
        F = self.n_fixations if n_fixations is None else n_fixations
        B = x.shape[0]
        fix_np, size_np = self.draw(x.shape[2:], B, F, area_range)      # always drawn: keeps the random stream in step
        if fixations is not None:
            assert len(fixations) == F
            fix = torch.stack([torch.as_tensor(f, dtype=torch.float32).reshape(-1, 2).expand(B, 2) for f in fixations], 1)
        elif self.nonrandom_val and not self.training:
            fix = torch.full((B, F, 2), 0.5)
        else:
            fix = torch.from_numpy(fix_np)
            if self.nonrandom_first:
                fix[:, 0] = 0.5
        fix = fix.to(device=x.device, dtype=torch.float32).contiguous()
        sizes = torch.from_numpy(size_np)
        x_fixs = self.retinal_transform(x, fix, fixation_size=sizes.to(x.device, torch.float32))     # [B,F,C,N], one launch
        deltas = torch.cat([torch.zeros(B, 1, 2, device=x.device), fix[:, 1:] - fix[:, :-1]], 1)
        return {"x_fixs": x_fixs, "fixations": fix.to(self.dtype), "fixation_sizes": sizes, "fix_deltas": deltas}


class NoSaccadePolicy(nn.Module):
    """A single central fixation (policies.py:297-340)."""

    def __init__(self, retinal_transform):
        super().__init__()
        self.retinal_transform, self.n_fixations, self.multi_policy = retinal_transform, 1, False
        self.fixation_size, self.dtype, self.device = retinal_transform.fixation_size, retinal_transform.dtype, retinal_transform.device

    @torch.no_grad()
    def forward(self, x, f1=None, area_range=None, n_fixations=None, fixation_size=None, fixations=None):
        assert f1 is None and area_range is None and (n_fixations is None or n_fixations == 1) and fixation_size is None and fixations is None
        x1 = self.retinal_transform(x, None).unsqueeze(1)
        B = x1.shape[0]
        return {"x_fixs": x1, "fixations": 0.5 * torch.ones((B, 1, 2)), "fixation_sizes": self.fixation_size * torch.ones((B, 1, 2)),
                "fix_deltas": torch.zeros(B, 1, 2)}


class _Registry(dict):
    """name -> builder(model) (policies.py:343-400)."""

    def register(self, name, builder_fn):
        self[name] = builder_fn

    def has(self, name):
        return name in self


FIXATION_POLICY_REGISTRY = _Registry()
