"""KNNConv modules: drop-in counterparts of the reference's ``KNNConvLayer`` (fovi/arch/knn.py:401-720)
and of the patch embeddings built on it (fovi/arch/knnvit.py:17-98, 224-290) on the CUDA kernels.

Same constructor signatures, parameter names/shapes (``weight [C_out, C_in*V]`` c-major/v-minor,
``bias [C_out]``: reference checkpoints load unchanged) and table attributes.  The forward pass runs the
tensor-core kernel (bf16 operands, fp32 accumulation) or, with ``precision='fp32'``, the exact
float32 kernel.  With gradients enabled the bf16 path is differentiable (fovi_b200/grad.py: both gradient
contractions run on the same kernel).
"""

import numpy as np
import torch
import torch.nn as nn

from . import ops, tables
from .coords import SamplingCoords, get_in_out_coords  # noqa: F401  (re-exported for callers of the reference API)

__all__ = ["KNNPoolingLayer", "KNNConvLayer", "KNNDepthwiseConvLayer", "KNNDepthwiseSeparableConvLayer", "KNNPatchEmbedding", "KNNPartitioningPatchEmbedding", "KNNConvStack", "KNN_CONV_REGISTRY", "get_knn_conv_layer"]


class _PoolFunction(torch.autograd.Function):
    """KNN pooling with its input gradient (fovi_knnpool_backward): what autograd computes through the reference's gather
    and nan-aware reductions (fovi/arch/knn.py:345-394)."""

    @staticmethod
    def forward(ctx, x, plan, mode, layout):
        ctx.plan, ctx.mode, ctx.layout = plan, mode, layout
        ctx.save_for_backward(x)
        with torch.no_grad():
            return plan.forward(x, mode, layout)

    @staticmethod
    def backward(ctx, gy):
        (x,) = ctx.saved_tensors
        return ctx.plan.backward(x, gy, ctx.mode, ctx.layout).to(x.dtype), None, None, None


class KNNPoolingLayer(nn.Module):
    """Pooling over the K nearest neighbours; counterpart of the reference layer (fovi/arch/knn.py:276-397): modes 'max',
    'avg', 'sum' and 'gaussian' (distance-weighted mean).  forward(X [B,C,N_in]) -> [B,C,N_out]."""

    def __init__(self, k, in_coords, out_coords, mode="max", device="cuda", sample_cortex=True, gauss_sigma=10, batch_size=None,
                 table_builder=None):
        super().__init__()
        if mode not in ops.POOL_MODES:
            raise NotImplementedError(f"Pooling style {mode} not implemented")
        self.in_coords, self.out_coords, self.device, self.mode = in_coords, out_coords, device, mode
        self.sample_cortex, self.batch_size = sample_cortex, batch_size
        n_in = in_coords.shape[0]
        self.k = torch.minimum(torch.tensor(k), torch.tensor(n_in))
        self._k = int(self.k.item())
        self.knn_indices, self.knn_distances, _, _ = tables.knn_table(in_coords, out_coords, self._k, sample_cortex, batch_size, builder=table_builder)
        self.knn_pad_token_val = n_in
        self.knn_indices_pad_mask = self.knn_indices >= n_in
        self.knn_indices_pad_token = tables.pad_token_table(self.knn_indices, n_in)
        self._plan = ops.KnnPoolPlan(self.knn_indices_pad_token.numpy().astype(np.int32), n_in, device=torch.device(device))
        if mode == "gaussian":
            self.gauss_sigma = gauss_sigma
            self.gaussian_weights = self._compute_gaussian_weights()
            self._plan.set_weights(self.gaussian_weights.numpy())

    def _compute_gaussian_weights(self):
        """[K, n_out] weights exp(-d^2 / (2 sigma^2)) of the neighbour distances, min-max normalised per neighbourhood, summing
        to one per output point (fovi/arch/knn.py:325-343; same torch operations, so the same numbers)."""
        d = self.knn_distances
        lo, hi = d.min(0).values.unsqueeze(0), d.max(0).values.unsqueeze(0)
        k = (d - lo) / (hi - lo)
        w = torch.exp(-k ** 2 / (2 * self.gauss_sigma ** 2))
        return w / (w.sum(dim=0, keepdim=True) + 1e-8)

    def forward(self, X_l):
        """X_l [B,C,N_in] -> [B,C,N_out]; differentiable with respect to X_l."""
        if torch.is_grad_enabled() and X_l.requires_grad:
            return _PoolFunction.apply(X_l, self._plan, self.mode, ops.ACT_BCN)
        with torch.no_grad():
            return self._plan.forward(X_l, self.mode, ops.ACT_BCN)

    def forward_points(self, x_bnc):
        """Channels-last [B,N_in,C] -> [B,N_out,C] (the layout between the KNNConv kernels); differentiable."""
        if torch.is_grad_enabled() and x_bnc.requires_grad:
            return _PoolFunction.apply(x_bnc, self._plan, self.mode, ops.ACT_BNC)
        with torch.no_grad():
            return self._plan.forward(x_bnc, self.mode, ops.ACT_BNC)

    def __repr__(self):
        return f"KNNPoolingLayer(\n\tmode={self.mode}\n\tk={self.k}\n\tin_coords={self.in_coords}\n\tout_coords={self.out_coords}\n\tsample_cortex={self.sample_cortex}\n)"


class KNNConvLayer(nn.Module):
    """Convolution over the K nearest neighbours of each output point, filter taps assigned through a
    per-neighbourhood reference frame.

    Args as the reference (knn.py:423-430); ``precision`` ('bf16' | 'fp32') is an addition.
    ``tables_override`` = dict(knn_indices [K,n_out] int64, tap [n_out,K], V, ref_coords?) skips the
    table construction (used to run recorded tables).  ``table_builder`` ('torch' | 'native', default from
    ``tables.default_builder()``) selects how the tables are built (see fovi_b200/tables.py).

    Inputs of a layer with at most 4 input channels (a first layer fed by the sensor) must be finite on the bf16 path:
    there the two points of an aligned pair (2p, 2p+1) share one operand block, the non-neighbour multiplied by zero
    weights, so an Inf / NaN would also reach outputs whose neighbourhoods hold only the point's partner (and the
    neighbouring output points that share an accumulator with them).  Layers with more
    channels, and ``precision='fp32'``, confine a non-finite input to the neighbourhoods that contain it, as the reference does.
    """

    def __init__(self, in_channels, out_channels, k, in_coords, out_coords, device="cuda", arch_flag="", sample_cortex=True,
                 bias=False, ref_frame_side_length=None, batch_size=None, precision="bf16", tables_override=None, table_builder=None):
        super().__init__()
        if precision not in ("bf16", "fp32"):
            raise ValueError("precision must be 'bf16' or 'fp32'")
        self.in_channels, self.out_channels = in_channels, out_channels
        self.in_coords, self.out_coords = in_coords, out_coords
        self.device, self.arch_flag, self.sample_cortex = device, arch_flag, sample_cortex
        self.ref_frame_side_length, self.batch_size, self.precision = ref_frame_side_length, batch_size, precision
        n_in = in_coords.shape[0]
        self.k = torch.minimum(torch.tensor(k), torch.tensor(n_in))
        self._k = int(self.k.item())
        if tables_override is None:
            self.knn_indices, self.knn_distances, pts, cart = tables.knn_table(in_coords, out_coords, self._k, sample_cortex, batch_size,
                                                                               builder=table_builder)
            self.ref_coords, self.ref_grid_size = tables.reference_frame(self._k, ref_frame_side_length, arch_flag, in_coords.dtype)
            self.tap, self.knn_coords = tables.tap_table(self.knn_indices, pts, cart, out_coords, self.ref_coords, bool(sample_cortex),
                                                         builder=table_builder)
        else:
            self.knn_indices = torch.as_tensor(np.asarray(tables_override["knn_indices"]), dtype=torch.long)
            self.tap = torch.as_tensor(np.asarray(tables_override["tap"]).astype(np.int64))
            self.knn_distances = self.knn_coords = None
            V = int(tables_override["V"])
            self.ref_grid_size = int(round(V ** 0.5))
            self.ref_coords = tables_override.get("ref_coords", tables.reference_frame(self._k, self.ref_grid_size)[0] if self.ref_grid_size ** 2 == V else torch.zeros(V, 2))
        self.knn_indices_pad_mask = self.knn_indices >= n_in
        self.knn_indices_pad_token = tables.pad_token_table(self.knn_indices, n_in)
        self.knn_indices_batch_cache = self.knn_indices_pad_token
        V = self.ref_coords.shape[0]
        self.weight = nn.Parameter(torch.empty(out_channels, in_channels * V))
        if bias:
            self.bias = nn.Parameter(torch.empty(out_channels))
        else:
            self.register_parameter("bias", None)
        nn.init.kaiming_normal_(self.weight)
        if self.bias is not None:
            nn.init.zeros_(self.bias)
        dev = torch.device(device)
        self.to(dev)
        self._plan = ops.KnnConvPlan(self.knn_indices_pad_token.numpy().astype(np.int32), self.tap.numpy().astype(np.uint16),
                                     n_in, V, in_channels, out_channels, device=dev)
        self._packed = {}          # dtype -> (weight version, data_ptr, packed tensor)
        self._grad = None

    # ---- tables in the reference's own representation, built on demand (can be hundreds of MB)
    @property
    def local_rf(self):
        """One-hot [n_out, K, V] float32, as the reference stores it (knn.py:636-647)."""
        rf = torch.zeros(self.tap.shape[0], self.tap.shape[1], self.ref_coords.shape[0])
        rf.scatter_(2, self.tap.unsqueeze(2), 1)
        return rf

    @property
    def plan(self):
        return self._plan

    def refresh_weights(self):
        """Drop the kernel-layout copies of ``weight``.  In-place updates of the parameter (optimizer steps,
        ``load_state_dict``, ``with torch.no_grad(): w.copy_(...)``) are noticed through its version counter;
        writes through ``weight.data`` bypass that counter, so call this after them."""
        self._packed.clear()

    def _load_from_state_dict(self, *args, **kwargs):
        super()._load_from_state_dict(*args, **kwargs)
        self._packed.clear()

    def packed_weight(self, dtype=torch.bfloat16):
        """Kernel-layout copy of ``weight``, rebuilt when the parameter changes (see refresh_weights)."""
        w = self.weight
        key = (w._version, w.data_ptr())
        hit = self._packed.get(dtype)
        if hit is None or hit[0] != key:
            self._packed[dtype] = (key, self._plan.pack_weights(w.detach(), dtype))
        return self._packed[dtype][1]

    @torch.no_grad()
    def forward_points(self, x_points, batch=None, relu=False, out_dtype=torch.bfloat16, out=None):
        """Tensor-core path on the kernel layout: channels-last [B,n_in,cin_packed] bf16 (or the pair
        layout with `batch` rows) -> channels-last [B,n_out,C_out]."""
        return self._plan.forward(x_points, self.packed_weight(), self.bias, relu=relu, out_dtype=out_dtype, out=out, batch=batch)

    def forward(self, X_l):
        """X_l [B,C_in,N_in] -> [B,C_out,N_out] in X_l's dtype (knn.py:538-557); the result is a
        channels-last view."""
        if torch.is_grad_enabled() and (X_l.requires_grad or self.weight.requires_grad or (self.bias is not None and self.bias.requires_grad)):
            from .grad import knnconv_autograd
            return knnconv_autograd(self, X_l)      # tensor-core gradients, or the exact float32 ones for precision='fp32'
        with torch.no_grad():
            return self._forward(X_l)

    @property
    def grad_plans(self):
        """Derived plans of the backward pass (fovi_b200/grad.py), built on first use."""
        if self._grad is None:
            from .grad import KnnConvGrad
            self._grad = KnnConvGrad(self.knn_indices_pad_token.numpy(), self.tap.numpy(), self.in_coords.shape[0], self.ref_coords.shape[0],
                                     self.in_channels, self.out_channels, torch.device(self.device))
        return self._grad

    def _forward(self, X_l):
        # shapes the tensor-core kernel does not cover (c_out not a multiple of 16, > 256 neighbours) run on the exact kernel
        if self.precision == "fp32" or not self._plan.tc_supported:
            y = self._plan.forward_f32(X_l, self.packed_weight(torch.float32), self.bias)
            return y.to(X_l.dtype)
        out_dtype = torch.float32 if X_l.dtype == torch.float32 else torch.bfloat16
        xp = ops.pack_points(X_l, self._plan)
        y = self._plan.forward(xp, self.packed_weight(), self.bias, out_dtype=out_dtype, batch=X_l.shape[0])
        return y.permute(0, 2, 1).to(X_l.dtype)

    def load_conv2d_weights(self, conv2d, strict=False):
        """Load a Conv2d kernel: transpose/flip from (row, col) to (x, y), resample to the reference
        frame if sizes differ, flatten to [C_out, C_in*V] (knn.py:649-702)."""
        w = conv2d.weight.data.clone().transpose(-1, -2).flip(-1)
        g = self.ref_grid_size
        if w.shape[0] != self.out_channels or w.shape[1] != self.in_channels:
            raise ValueError("Conv2d channel counts do not match this layer")
        if w.shape[2] != g or w.shape[3] != g:
            if strict:
                raise ValueError(f"Conv2d kernel {tuple(w.shape[2:])} != reference frame {g}x{g}")
            w = nn.functional.interpolate(w, size=(g, g), mode="bilinear", align_corners=True)
        self.weight.data.copy_(w.reshape(w.shape[0], -1))
        if conv2d.bias is not None:
            if self.bias is None:
                raise ValueError("Conv2d has bias but layer does not. Recreate layer with bias=True.")
            self.bias.data.copy_(conv2d.bias.data)

    def __repr__(self):
        return (f"{self.__class__.__name__}(\n\tin_channels={self.in_channels}\n\tout_channels={self.out_channels}\n\tk={self.k}\n\t"
                f"n_ref={self.ref_coords.shape[0]}\n\tin_coords={self.in_coords}\n\tout_coords={self.out_coords}\n\tsample_cortex={self.sample_cortex}\n)")


class _DepthwiseBase(KNNConvLayer):
    """Shared part of the depthwise layers: the filter ``[C_in, V, g]`` in the kernel's ``[V, C_in*g]`` float32 layout."""

    def _packed_depthwise(self, w):
        key = (w._version, w.data_ptr())
        hit = self._packed.get("dw")
        if hit is None or hit[0] != key:
            V = self.ref_coords.shape[0]
            self._packed["dw"] = (key, w.detach().float().permute(1, 0, 2).reshape(V, self.out_channels).contiguous())
        return self._packed["dw"][1]

    @staticmethod
    def _wants_grad(*tensors):
        return torch.is_grad_enabled() and any(t is not None and t.requires_grad for t in tensors)


class _DepthwiseFunction(torch.autograd.Function):
    """Depthwise KNN convolution with its gradients (float32 atomics on the ordinary cores)."""

    @staticmethod
    def forward(ctx, x, weight, bias, layer):
        ctx.layer, ctx.has_bias = layer, bias is not None
        ctx.save_for_backward(x, weight)
        with torch.no_grad():
            return layer._plan.depthwise(x, layer._packed_depthwise(weight), bias)

    @staticmethod
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        layer = ctx.layer
        gx, gwp = layer._plan.depthwise_backward(x, layer._packed_depthwise(weight), gy, need_gx=ctx.needs_input_grad[0],
                                                 need_gw=ctx.needs_input_grad[1])
        gw = None
        if gwp is not None:             # [V, C_in * g] -> [C_in, V, g]
            V = gwp.shape[0]
            gw = gwp.view(V, layer.in_channels, -1).permute(1, 0, 2).contiguous().to(weight.dtype)
        gb = gy.sum((0, 2), dtype=torch.float32) if (ctx.has_bias and ctx.needs_input_grad[2]) else None
        return (gx.to(x.dtype) if gx is not None else None), gw, gb, None


class _Points:
    """Stand-in for a coordinate set where only the point count matters."""

    def __init__(self, n):
        self.shape, self.dtype = (n, 2), torch.float32


class KNNDepthwiseConvLayer(_DepthwiseBase):
    """Depthwise KNN convolution: every input channel is filtered on its own into g = out/in output channels
    (fovi/arch/knn.py:803-872).  Parameters as the reference: ``weight [C_in, V, g]``, ``bias [C_out]`` (a zero tensor
    when bias=False).  forward(X [B,C_in,N_in]) -> [B,C_out,N_out]; differentiable (input, filter and bias gradients)."""

    def __init__(self, in_channels, out_channels, k, in_coords, out_coords, device="cuda", arch_flag="", sample_cortex=True, bias=False,
                 batch_size=None, ref_frame_side_length=None, **kwargs):
        assert out_channels % in_channels == 0, "out_channels must be divisible by in_channels for depthwise conv"
        super().__init__(in_channels, out_channels, k, in_coords, out_coords, device, arch_flag, sample_cortex, bias, ref_frame_side_length,
                         batch_size, **kwargs)
        dev = torch.device(device)
        self.weight = nn.Parameter(torch.empty(in_channels, self.ref_coords.shape[0], out_channels // in_channels, device=dev))
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_channels, device=dev))
        else:
            self.bias = None
            self.zero_bias = torch.zeros(out_channels, device=dev)
        bound = 1 / (in_channels * self._k)
        nn.init.uniform_(self.weight, a=-bound, b=bound)

    def forward(self, X_l):
        if self._wants_grad(X_l, self.weight, self.bias):
            return _DepthwiseFunction.apply(X_l, self.weight, self.bias, self)
        with torch.no_grad():
            return self._plan.depthwise(X_l, self._packed_depthwise(self.weight), self.bias)


class KNNDepthwiseSeparableConvLayer(_DepthwiseBase):
    """Depthwise KNN convolution followed by a pointwise linear map over channels (fovi/arch/knn.py:722-800).
    Parameters as the reference: ``dw_conv [C_in, V, g]``, ``p_conv`` = Linear(C_out, C_out); the base class's dense
    ``weight`` is kept (unused, as in the reference) so that state dicts line up.  The pointwise map is a KNNConv whose
    every point has itself as only neighbour (one tap), so it runs on the same kernels: the tensor-core kernel for bf16
    activations, the exact float32 kernel otherwise."""

    def __init__(self, in_channels, out_channels, k, in_coords, out_coords, device="cuda", arch_flag="", sample_cortex=True, bias=False,
                 batch_size=None, ref_frame_side_length=None, **kwargs):
        assert out_channels % in_channels == 0, "out_channels must be divisible by in_channels for depthwise conv"
        super().__init__(in_channels, out_channels, k, in_coords, out_coords, device, arch_flag, sample_cortex, bias, ref_frame_side_length,
                         batch_size, **kwargs)
        dev = torch.device(device)
        self.dw_conv = nn.Parameter(torch.empty(in_channels, self.ref_coords.shape[0], out_channels // in_channels, device=dev))
        self.p_conv = nn.Linear(out_channels, out_channels, bias=bias, device=dev)
        bound = 1 / (in_channels * self._k)
        nn.init.uniform_(self.dw_conv, a=-bound, b=bound)
        nn.init.uniform_(self.p_conv.weight, a=-bound, b=bound)
        if self.p_conv.bias is not None:
            nn.init.zeros_(self.p_conv.bias)
        n_out = self.knn_indices.shape[1]
        self._pw_layer = None
        self._pw_plan = ops.KnnConvPlan(np.arange(n_out, dtype=np.int32)[None, :], np.zeros((n_out, 1), np.uint16), n_out, 1,
                                        out_channels, out_channels, device=dev)

    def _packed_pointwise(self, dtype):
        w = self.p_conv.weight
        key, name = (w._version, w.data_ptr()), ("pw", dtype)
        hit = self._packed.get(name)
        if hit is None or hit[0] != key:
            self._packed[name] = (key, self._pw_plan.pack_weights(w.detach(), dtype))
        return self._packed[name][1]

    def _pointwise_layer(self):
        """The pointwise map as a KNNConv layer (every point its own only neighbour, one tap) that shares ``p_conv``'s
        parameters: what the autograd path differentiates.  Kept out of the module tree so that state dicts are unchanged."""
        if self._pw_layer is None:
            n_out = self.knn_indices.shape[1]
            L = KNNConvLayer(self.out_channels, self.out_channels, 1, _Points(n_out), _Points(n_out), device=self.device, bias=False,
                             tables_override=dict(knn_indices=np.arange(n_out)[None, :], tap=np.zeros((n_out, 1), np.int64), V=1))
            self._pw_layer = [L]
        L = self._pw_layer[0]
        L._parameters["weight"], L._parameters["bias"] = self.p_conv.weight, self.p_conv.bias
        return L

    def forward(self, X_l):
        if self._wants_grad(X_l, self.dw_conv, self.p_conv.weight, self.p_conv.bias):
            from .grad import knnconv_autograd
            dw = _DepthwiseFunction.apply(X_l, self.dw_conv, None, self)                  # [B, C_out, N_out]
            return knnconv_autograd(self._pointwise_layer(), dw)
        with torch.no_grad():
            tc = X_l.dtype == torch.bfloat16 and self._pw_plan.tc_supported and self._pw_plan.x_layout == ops.X_BNC \
                and self._pw_plan.cin_packed == self.out_channels
            dw = self._plan.depthwise(X_l, self._packed_depthwise(self.dw_conv), None, y_layout=ops.ACT_BNC,
                                      out_dtype=torch.bfloat16 if tc else torch.float32)                          # [B, N_out, C_out]
            if tc:
                y = self._pw_plan.forward(dw, self._packed_pointwise(torch.bfloat16), self.p_conv.bias, out_dtype=torch.bfloat16)
                return y.permute(0, 2, 1)
            y = self._pw_plan.forward_f32(dw, self._packed_pointwise(torch.float32), self.p_conv.bias, x_layout=ops.ACT_BNC)
            return y.to(X_l.dtype)


class KNNPatchEmbedding(KNNConvLayer):
    """Foveated patch embedding: one KNNConv from the sensor points onto ~(cart_res/patch)^2 token points
    (fovi/arch/knnvit.py:17-98).  forward returns [B, tokens, D] ([B, D, tokens] if `transposed`)."""

    def __init__(self, in_channels, embed_dim, in_res, fov, cmf_a, style="isotropic", auto_match_cart_resources=True, in_cart_res=224,
                 cart_patch_size=16, patch_overlap_factor=1, device="cuda", force_patches_less_than_matched=True,
                 new_parameterization=False, transposed=False, max_coord_val=1, sample_cortex=True, ref_frame_side_length=None, **kwargs):
        stride = cart_patch_size / patch_overlap_factor if new_parameterization else cart_patch_size
        ic, oc, out_cart_res = get_in_out_coords(in_res, fov, cmf_a, stride, style=style, auto_match_cart_resources=auto_match_cart_resources,
                                                 in_cart_res=in_cart_res, device="cpu", force_out_match_less_than=force_patches_less_than_matched,
                                                 max_out_coord_val=max_coord_val)
        k = cart_patch_size ** 2 if new_parameterization else int((cart_patch_size * out_cart_res / np.sqrt(len(oc)) * patch_overlap_factor) ** 2)
        super().__init__(in_channels, embed_dim, k, ic, oc, device=device, sample_cortex=sample_cortex, ref_frame_side_length=ref_frame_side_length, **kwargs)
        self.transposed = transposed

    def forward(self, x):
        if x.dim() == 4:
            x = x.flatten(2)
        tokens = super().forward(x)
        return tokens if self.transposed else tokens.permute(0, 2, 1)


class KNNPartitioningPatchEmbedding(KNNPatchEmbedding):
    """Patch embedding whose K is the smallest neighbourhood size that lets the token neighbourhoods cover
    every input point: inputs are partitioned by nearest token, and K is the largest count of inputs lying
    closer to a token than its farthest partition member (fovi/arch/knnvit.py:224-290)."""

    def __init__(self, in_channels, embed_dim, in_res, fov, cmf_a, style="isotropic", auto_match_cart_resources=True, in_cart_res=224,
                 cart_patch_size=16, device="cuda", force_patches_less_than_matched=True, transposed=False, max_coord_val="auto",
                 sample_cortex=True, **kwargs):
        ic, oc, _ = get_in_out_coords(in_res, fov, cmf_a, cart_patch_size, style=style, auto_match_cart_resources=auto_match_cart_resources,
                                      in_cart_res=in_cart_res, device="cpu", force_out_match_less_than=force_patches_less_than_matched,
                                      max_out_coord_val=max_coord_val)
        if sample_cortex == "geodesic":
            raise NotImplementedError("geodesic neighbour ranking is not built; use sample_cortex=True")
        pts = torch.cat([ic.cortical, ic.cortical_pad_coords], 0) if sample_cortex else torch.cat([ic.cartesian, ic.cartesian_pad_coords], 0)
        dist = torch.cdist(pts, oc.cortical.clone() if sample_cortex else oc.cartesian)        # [n_in+pad, tokens]
        owner = torch.argmin(dist[: len(ic)], 1)
        k = 0
        for t in range(len(oc)):
            reach = dist[torch.argwhere(owner == t).squeeze(), t].max()
            k = max(k, int((dist[:, t] < reach).sum()))
        KNNConvLayer.__init__(self, in_channels, embed_dim, k, ic, oc, device=device, sample_cortex=sample_cortex, **kwargs)
        self.transposed = transposed


class KNNConvStack(nn.Module):
    """A chain of KNNConv layers with ReLU between them, kept in the kernels' channels-last layout from
    end to end (the conv -> activation skeleton of fovi/arch/knnalexnet.py:109-127).  Buffers between layers are
    allocated once per batch size and reused; the returned tensor is new memory on every call."""

    def __init__(self, layers, final_relu=False):
        super().__init__()
        self.layers = nn.ModuleList(layers)
        self.final_relu = final_relu
        self._acts = {}

    def _act_buffers(self, rows, device):
        """Buffers of the layers between the first and the last: allocated once per batch size and reused.  The last
        layer's output is NOT among them: it is what the caller receives, so every call gets fresh memory."""
        key = (rows, str(device))
        if key not in self._acts:
            self._acts[key] = [torch.empty((rows, L.plan.n_out, L.out_channels), dtype=torch.bfloat16, device=device)
                               for L in self.layers[:-1]]
        return self._acts[key]

    @torch.no_grad()
    def forward_points(self, x_points, rows, out_dtype=torch.bfloat16, out=None):
        """x_points: the first layer's kernel layout (see KNNConvLayer.forward_points) -> [rows, n_out, C_out].
        `out`: optional destination of the last layer (a caller that recycles its own buffer); otherwise the result
        is newly allocated, so results of earlier calls stay valid."""
        bufs = self._act_buffers(rows, x_points.device)
        h = x_points
        for i, L in enumerate(self.layers):
            last = i == len(self.layers) - 1
            dst = out if last else bufs[i]
            h = L.forward_points(h, batch=rows, relu=(not last) or self.final_relu, out_dtype=out_dtype if last else torch.bfloat16, out=dst)
        return h

    def forward(self, X):
        """X [B,C_in,N_in] -> [B,C_out,N_out] (channels-last view), dtype of X.  With gradients enabled the chain is
        differentiable and stays in the kernels' layout in both directions (fovi_b200/grad.py)."""
        if torch.is_grad_enabled() and any(p.requires_grad for p in self.parameters()):
            return self._forward_autograd(X)
        with torch.no_grad():
            return self._forward_inference(X)

    def _forward_autograd(self, X):
        from .grad import knnconv_points_autograd
        if not all(L.plan.tc_supported and L.precision == "bf16" for L in self.layers):
            raise RuntimeError("the backward pass is built for the bf16 tensor-core path")
        first = self.layers[0].plan.x_layout == ops.X_PAIRS
        if not first and self.layers[0].in_channels % 8:
            raise RuntimeError("the first layer's channels must be at most 4 or a multiple of 8")
        h = X if first else X.permute(0, 2, 1).to(torch.bfloat16)     # differentiable layout change
        n = len(self.layers)
        for i, L in enumerate(self.layers):
            h = knnconv_points_autograd(L, h, (i < n - 1) or self.final_relu)
        return h.permute(0, 2, 1).to(X.dtype)

    def _forward_inference(self, X):
        xp = ops.pack_points(X, self.layers[0].plan)
        out_dtype = torch.float32 if X.dtype == torch.float32 else torch.bfloat16
        return self.forward_points(xp, X.shape[0], out_dtype).permute(0, 2, 1)


KNN_CONV_REGISTRY = {"default": KNNConvLayer, "b200": KNNConvLayer, "dwsep": KNNDepthwiseSeparableConvLayer, "dw": KNNDepthwiseConvLayer}


def get_knn_conv_layer(name):
    """Layer class by registry name (fovi/arch/knn.py:1014-1030)."""
    if name not in KNN_CONV_REGISTRY:
        raise ValueError(f"Unknown KNN conv layer: {name}. Available: {list(KNN_CONV_REGISTRY.keys())}")
    return KNN_CONV_REGISTRY[name]
