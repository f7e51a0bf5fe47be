"""Normalisation layers of KNN activations ``[B, C, N]``: counterparts of the reference's ``fovi/arch/norm.py`` with the
same class names, constructor signatures and parameter names/shapes (they subclass the same torch modules, so state
dicts line up).  Batch norm (every shipped configuration) is folded into the convolution by ``KNNAlexNetBlock``; the
per-sample norms (channel / coord / layer / group) run on the CUDA normalisation kernels, on both activation layouts,
with the following ReLU fused.  Under autograd (training) the per-sample norms are evaluated with the torch functions
the reference's own layers call (``F.layer_norm`` / ``F.group_norm`` on the same axes), which carry the gradients; batch
norm in training mode is torch's ``BatchNorm1d`` as in the reference.
"""
import numpy as np
import torch
import torch.nn as nn

from . import ops

__all__ = ["KNNChannelNorm", "KNNBatchNorm", "KNNCoordNorm", "KNNLayerNorm", "KNNGroupNorm", "find_valid_num_groups", "get_norm"]


class _KernelNorm:
    """Mixin: forward([B,C,N]) and forward_points([B,N,C]) on the CUDA kernel."""
    _mode = None

    def _groups(self):
        return 1

    def _run(self, x, layout, relu=False, out_dtype=None):
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            y = self._torch_forward(x if layout == ops.ACT_BCN else x.permute(0, 2, 1))      # [B, C, N] view
            y = torch.relu(y) if relu else y
            y = y if layout == ops.ACT_BCN else y.permute(0, 2, 1)
            return y if out_dtype is None else y.to(out_dtype)
        w = self.weight.reshape(-1) if self.weight is not None else None
        b = self.bias.reshape(-1) if self.bias is not None else None
        return ops.knn_norm(x, self._mode, w, b, eps=self.eps, groups=self._groups(), layout=layout, relu=relu, out_dtype=out_dtype)

    def _torch_forward(self, x):
        """Differentiable evaluation on [B, C, N] with the reference's torch calls (fovi/arch/norm.py:14-101)."""
        import torch.nn.functional as F
        if self._mode == "channel":
            return F.layer_norm(x.transpose(1, 2), self.normalized_shape, self.weight, self.bias, self.eps).transpose(1, 2)
        if self._mode in ("coord", "layer"):
            return F.layer_norm(x, self.normalized_shape, self.weight, self.bias, self.eps)
        return F.group_norm(x, self.num_groups, self.weight, self.bias, self.eps)

    def forward(self, x):
        return self._run(x, ops.ACT_BCN)

    def forward_points(self, x_bnc, relu=False, out_dtype=None):
        """Channels-last [B, N, C] in and out (the layout between the KNNConv kernels), optional fused ReLU."""
        return self._run(x_bnc, ops.ACT_BNC, relu, out_dtype)


class KNNChannelNorm(_KernelNorm, nn.LayerNorm):
    """LayerNorm over the channels of every (sample, point) (fovi/arch/norm.py:14-33)."""
    _mode = "channel"

    def __init__(self, num_coords, num_channels, device="cuda"):
        nn.LayerNorm.__init__(self, [num_channels], device=device)

    def __repr__(self):
        return nn.LayerNorm.__repr__(self).replace("LayerNorm", "KNNChannelNorm")


class KNNBatchNorm(nn.BatchNorm1d):
    """Batch normalisation over [B, C, N] activations (fovi/arch/norm.py:36-48)."""

    def __init__(self, num_coords, num_channels, device="cuda"):
        super().__init__(num_channels, device=device)

    def __repr__(self):
        return super().__repr__().replace("BatchNorm1d", "KNNBatchNorm")

    def folded(self):
        """Per-channel (scale, shift) of the evaluation-mode transform y = x*scale + shift, float32."""
        scale = torch.rsqrt(self.running_var.float() + self.eps)
        if self.weight is not None:
            scale = scale * self.weight.detach().float()
        shift = -self.running_mean.float() * scale
        if self.bias is not None:
            shift = shift + self.bias.detach().float()
        return scale, shift


class KNNCoordNorm(_KernelNorm, nn.LayerNorm):
    """LayerNorm over the points of every (sample, channel) (fovi/arch/norm.py:51-64)."""
    _mode = "coord"

    def __init__(self, num_coords, num_channels, device="cuda"):
        nn.LayerNorm.__init__(self, [num_coords], device=device)

    def __repr__(self):
        return nn.LayerNorm.__repr__(self).replace("LayerNorm", "KNNCoordNorm")


class KNNLayerNorm(_KernelNorm, nn.LayerNorm):
    """LayerNorm over channels and points of every sample (fovi/arch/norm.py:67-80)."""
    _mode = "layer"

    def __init__(self, num_coords, num_channels, device="cuda"):
        nn.LayerNorm.__init__(self, [num_channels, num_coords], device=device)

    def __repr__(self):
        return nn.LayerNorm.__repr__(self).replace("LayerNorm", "KNNLayerNorm")


class KNNGroupNorm(_KernelNorm, nn.GroupNorm):
    """GroupNorm over channel groups x points (fovi/arch/norm.py:83-100)."""
    _mode = "group"

    def __init__(self, num_coords, num_channels, base_groups=32, min_channels_per_group=4, device="cuda"):
        nn.GroupNorm.__init__(self, find_valid_num_groups(num_channels, base_groups, min_channels_per_group), num_channels, device=device)

    def _groups(self):
        return self.num_groups

    def __repr__(self):
        return nn.GroupNorm.__repr__(self).replace("GroupNorm", "KNNGroupNorm")


def find_valid_num_groups(num_channels, base_groups, min_channels_per_group=4):
    """Largest group count <= min(base_groups, num_channels // min_channels_per_group) that divides num_channels
    (fovi/arch/norm.py:103-123)."""
    desired = int(min(max(num_channels // min_channels_per_group, 1), base_groups))
    for g in range(desired, 0, -1):
        if num_channels % g == 0:
            return g
    return 1


def get_norm(norm_type, num_coords, num_channels, base_groups=32, min_channels_per_group=4, device="cuda"):
    """Normalisation layer by name (fovi/arch/norm.py:126-160)."""
    if norm_type in ("layer_chan", "channel"):
        return KNNChannelNorm(num_coords, num_channels, device=device)
    if norm_type in ("layer_space", "coord"):
        return KNNCoordNorm(num_coords, num_channels, device=device)
    if norm_type in ("layer_all", "layer"):
        return KNNLayerNorm(num_coords, num_channels, device=device)
    if norm_type == "group":
        return KNNGroupNorm(num_coords, num_channels, base_groups, min_channels_per_group, device=device)
    if "batch" in norm_type:
        return KNNBatchNorm(num_coords, num_channels, device=device)
    if norm_type == "none":
        return None
    raise NotImplementedError(f"norm_type {norm_type} not implemented")
