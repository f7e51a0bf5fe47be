"""The foveated AlexNet backbone on the CUDA kernels: counterparts of the reference's ``KNNAlexNetBlock`` and
``KNNAlexNet`` (fovi/arch/knnalexnet.py:13-127, 130-260) with the same constructor signatures, sub-module names
(``layers.{i}.conv / .norm / .pool``, ``classifier``) and parameter shapes, so reference checkpoints load unchanged.

A block is conv -> norm -> activation -> pool.  Without gradients (inference) batch normalisation (the norm of every
shipped configuration, fovi/arch/norm.py:36-48, evaluated with its running statistics) is folded into the convolution's
packed weights and bias and ReLU runs in the convolution's epilogue; a per-sample norm (channel / coord / layer / group)
runs as its own kernel behind the convolution with the ReLU fused into it; pooling is the gather-reduce kernel on the same
channels-last layout, so activations stay in the kernels' layout from the sensor to the classifier.  Under autograd
(training) the blocks run one by one: the convolution and the pooling with their own gradient kernels, the norm and the
activation through torch as in the reference (batch norm with batch statistics in training mode).
"""
import numpy as np
import torch
import torch.nn as nn

from . import ops
from .coords import auto_match_num_coords, get_in_out_coords
from .knn import KNNConvLayer, KNNPoolingLayer, get_knn_conv_layer
from .norm import KNNBatchNorm, _KernelNorm, get_norm

__all__ = ["KNNBatchNorm", "get_norm", "KNNAlexNetBlock", "KNNAlexNet", "FoveatedAlexNet"]   # the norms live in fovi_b200/norm.py


class KNNAlexNetBlock(nn.Module):
    """conv -> norm -> activation -> optional pool (fovi/arch/knnalexnet.py:13-127); arguments as the reference."""

    def __init__(self, in_channels, out_channels, k, fov, cmf_a, in_res, stride, style="isotropic", conv_layer="default", cart_res=None,
                 pool=True, pool_mode="max", pool_k=9, pool_stride=2, norm_type="batch", arch_flag="", activation=nn.ReLU,
                 sample_cortex=True, device="cuda", auto_match_cart_resources=0, ref_frame_mult=None):
        super().__init__()
        if isinstance(conv_layer, str):
            conv_layer = get_knn_conv_layer(conv_layer)
        self.in_coords, self.out_coords, out_cart_res = get_in_out_coords(
            in_res, fov, cmf_a, stride, style=style, auto_match_cart_resources=auto_match_cart_resources, in_cart_res=cart_res)
        side = int(np.ceil(ref_frame_mult * np.sqrt(k))) if ref_frame_mult is not None else None
        self.conv = None if conv_layer is None else conv_layer(
            in_channels=in_channels, out_channels=out_channels, k=k, in_coords=self.in_coords, out_coords=self.out_coords,
            sample_cortex=sample_cortex, arch_flag=arch_flag, device=device, ref_frame_side_length=side)
        self.norm = get_norm(norm_type, self.out_coords.shape[0], out_channels, device=device)
        self.activation = activation() if activation is not None else None
        if pool:
            _, pooled, out_cart_res = get_in_out_coords(self.in_coords.resolution, fov, cmf_a, pool_stride, style=style,
                                                        auto_match_cart_resources=auto_match_cart_resources, in_cart_res=out_cart_res)
            self.pool = KNNPoolingLayer(k=pool_k, in_coords=self.out_coords, out_coords=pooled, mode=pool_mode, device=device,
                                        sample_cortex=sample_cortex)
            self.out_coords = pooled
        else:
            self.pool = None
        self.out_res = self.out_coords.resolution
        self.out_cart_res = out_cart_res
        self._folded = None        # (key, packed weights, bias) of the convolution with the norm folded in
        self.to(device)

    # ---- the convolution's operands with the evaluation-mode batch norm folded in
    def _fold_key(self):
        ts = [self.conv.weight, self.conv.bias]
        if isinstance(self.norm, KNNBatchNorm):
            ts += [self.norm.weight, self.norm.bias, self.norm.running_mean, self.norm.running_var]
        return tuple((t._version, t.data_ptr()) for t in ts if t is not None)

    def refresh_weights(self):
        """Forget the folded operands (needed only after writes through ``.data``, which no version counter sees)."""
        self._folded = None

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self._folded = None

    def folded_operands(self):
        """(packed bf16 weights, float32 bias) such that conv(x; W', b') == norm(conv(x; W, b))."""
        key = self._fold_key()
        if self._folded is None or self._folded[0] != key:
            w = self.conv.weight.detach().float()
            b = self.conv.bias.detach().float() if self.conv.bias is not None else None
            if isinstance(self.norm, KNNBatchNorm):
                scale, shift = self.norm.folded()
                w = w * scale[:, None]
                b = shift if b is None else b * scale + shift
            self._folded = (key, self.conv.plan.pack_weights(w), b)
        return self._folded[1], self._folded[2]

    @property
    def points_path(self):
        """True when the block can run on the kernels' channels-last layout end to end."""
        return (self.conv is not None and self.conv.plan.tc_supported and getattr(self.conv, "precision", "bf16") == "bf16"
                and (self.norm is None or isinstance(self.norm, (KNNBatchNorm, _KernelNorm))))

    @torch.no_grad()
    def forward_points(self, h, rows):
        """h: the convolution's input layout (KNNConvLayer.forward_points) -> channels-last [rows, N_out, C_out] bf16."""
        if isinstance(self.norm, KNNBatchNorm) and self.norm.training:
            raise RuntimeError("KNNAlexNetBlock runs batch norm from its running statistics: call .eval() first")
        wt, b = self.folded_operands()
        relu = isinstance(self.activation, nn.ReLU)
        per_sample = isinstance(self.norm, _KernelNorm)
        h = self.conv.plan.forward(h, wt, b, relu=relu and not per_sample, out_dtype=torch.bfloat16, batch=rows)
        if per_sample:
            h = self.norm.forward_points(h, relu=relu)
        if self.activation is not None and not relu:
            h = self.activation(h)
        if self.pool is not None:
            h = self.pool.forward_points(h)
        return h

    def _wants_grad(self, x):
        return torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters()))

    def _forward_train(self, x):
        """The block under autograd: the convolution's own gradients (fovi_b200/grad.py), torch's norm and activation as in
        the reference (batch norm with batch statistics in training mode), the pooling's own gradient."""
        if self.conv is not None:
            x = self.conv(x)
        if self.norm is not None:
            x = self.norm(x)
        if self.activation is not None:
            x = self.activation(x)
        if self.pool is not None:
            x = self.pool(x)
        return x

    def forward(self, x):
        """x [B, C_in, N_in] -> [B, C_out, N_out] (fovi/arch/knnalexnet.py:109-127)."""
        if self._wants_grad(x):
            return self._forward_train(x)
        with torch.no_grad():
            return self._forward_eval(x)

    def _forward_eval(self, x):
        if self.points_path:
            h = self.forward_points(ops.pack_points(x, self.conv.plan), x.shape[0])
            return h.permute(0, 2, 1).to(x.dtype)
        if self.conv is not None:
            x = self.conv(x)
        if self.norm is not None:
            if isinstance(self.norm, KNNBatchNorm) and self.norm.training:
                raise RuntimeError("KNNAlexNetBlock runs batch norm from its running statistics: call .eval() first")
            x = self.norm(x)
        if self.activation is not None:
            x = self.activation(x)
        if self.pool is not None:
            x = self.pool(x)
        return x


class KNNAlexNet(nn.Module):
    """Stack of KNNAlexNetBlocks, an optional average pooling onto ``out_res`` and an optional linear classifier
    (fovi/arch/knnalexnet.py:130-260); arguments as the reference."""

    def __init__(self, in_res, in_channels, features_per_layer, stride_per_layer, pool_after, k_per_layer, n_classes=None, out_res=None,
                 auto_match_cart_resources=0, style="isotropic", layer_cls="default", norm_type="batch", arch_flag="", fov=16, cmf_a=0.5,
                 device="cuda", sample_cortex=True, ref_frame_mult=None):
        super().__init__()
        if isinstance(layer_cls, str):
            layer_cls = get_knn_conv_layer(layer_cls)
        in_res, cart_res = auto_match_num_coords(fov, cmf_a, in_res, style, auto_match_cart_resources, quiet=True)
        layers = []
        for i, feats in enumerate(features_per_layer):
            block = KNNAlexNetBlock(in_channels=in_channels, out_channels=feats, k=k_per_layer[i], fov=fov, cmf_a=cmf_a, in_res=in_res,
                                    stride=stride_per_layer[i], style=style, conv_layer=layer_cls, cart_res=cart_res,
                                    auto_match_cart_resources=auto_match_cart_resources, pool=i in pool_after, pool_mode="max", pool_k=9,
                                    pool_stride=2, norm_type=norm_type, arch_flag=arch_flag, sample_cortex=sample_cortex, device=device,
                                    ref_frame_mult=ref_frame_mult)
            in_channels, in_res, cart_res = feats, block.out_res, block.out_cart_res
            layers.append(block)
        if out_res is not None and out_res != -1:
            in_coords = block.out_coords
            out_coords, out_radii, _ = in_coords.get_strided_coords(1, auto_match_cart_resources=auto_match_cart_resources, in_cart_res=out_res)
            k = int(2 * np.ceil(in_res / out_radii)) ** 2      # the reference's heuristic: twice the downsampling factor, squared
            layers.append(KNNPoolingLayer(k=k, mode="avg", in_coords=in_coords, out_coords=out_coords, sample_cortex=sample_cortex, device=device))
        self.layers = nn.ModuleList(layers)
        self.n_classes = n_classes
        self.out_channels = features_per_layer[-1]
        self.out_coords = self.layers[-1].out_coords
        self.total_embed_dim = self.out_channels * self.out_coords.shape[0]
        if n_classes is not None:
            self.classifier = nn.Linear(self.total_embed_dim, n_classes, device=device)

    @property
    def points_path(self):
        return all(L.points_path for L in self.layers if isinstance(L, KNNAlexNetBlock))

    @torch.no_grad()
    def forward_points(self, h, rows):
        """h: the first convolution's input layout -> channels-last features [rows, N_out, C_out] bf16."""
        for L in self.layers:
            h = L.forward_points(h, rows) if isinstance(L, KNNAlexNetBlock) else L.forward_points(h)
        return h

    def forward(self, x):
        """x [B, C_in, N_in] -> logits [B, n_classes], or features [B, C_out, N_out] without a classifier.  Under autograd
        (training) the blocks run one by one with gradients; otherwise on the kernels' channels-last path."""
        if torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters())):
            for L in self.layers:
                x = L(x)
            if self.n_classes is not None:
                x = self.classifier(x.reshape(x.shape[0], -1))
            return x
        with torch.no_grad():
            return self._forward_eval(x)

    def _forward_eval(self, x):
        if self.points_path:
            h = self.forward_points(ops.pack_points(x, self.layers[0].conv.plan), x.shape[0])
            x = h.permute(0, 2, 1).to(x.dtype)
        else:
            for L in self.layers:
                x = L(x)
        if self.n_classes is not None:
            x = self.classifier(x.reshape(x.shape[0], -1))
        return x


class FoveatedAlexNet(nn.Module):
    """Images and fixations in, per-fixation or fixation-averaged network outputs out: the supervised forward pass of the
    reference model (fovi/fovinet.py:251-294: fixate, flatten '(f b)', run the network, un-flatten to [B, F, D]) with its
    mean over fixations (``saccades.fix_agg: mean``), without the projector head.

    The sensor writes all fixations of all images straight into the first convolution's input layout in one launch."""

    def __init__(self, retina, network):
        super().__init__()
        self.retina, self.network = retina, network

    @torch.no_grad()
    def forward(self, images, fix_loc, fixation_size=None, fix_agg=None):
        """images [B,3,H,W], fix_loc [B,F,2] (row, col in [0,1]) -> [B, F, D]; with fix_agg='mean' -> [B, D].
        D = n_classes, or C_out*N_out flattened channel-major when the network has no classifier."""
        net = self.network
        if not net.points_path:
            raise RuntimeError("FoveatedAlexNet needs a network whose blocks all run on the tensor-core path")
        B, F = images.shape[0], fix_loc.shape[1]
        xp, rows = self.retina.forward_points(images, fix_loc, fixation_size, conv_plan=net.layers[0].conv.plan)
        h = net.forward_points(xp, rows)                                  # [(f b), N_out, C_out]
        h = h.permute(0, 2, 1).reshape(rows, -1).float()
        if net.n_classes is not None:
            h = net.classifier(h)
        h = h.view(F, B, -1).permute(1, 0, 2)
        if fix_agg is None:
            return h
        if fix_agg == "mean":
            return h.mean(1)
        raise NotImplementedError(f"fix_agg {fix_agg!r}: 'mean' or None")
