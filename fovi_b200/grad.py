"""Backward pass of KNNConv on the forward tensor-core kernel.

Both gradient contractions of ``out[b,o,n] = sum_k sum_c Xpad[b,c,idx[k,n]] * W[o, c*V + tap[n,k]]``
(fovi/arch/knn.py:538-557; the reference gets them from autograd through its gather, one-hot matmul and linear) are
themselves table-driven gather-GEMMs, so each runs as a forward launch of ``fovi_knnconv_forward`` on a derived plan:

* input gradient — the transposed layer: "output" points are the layer's input points m, the neighbours of m are the
  output points n that list m, each with the tap it was given; channels swap roles
  (``dX[b,m,c] = sum_{(n,k): idx[k,n]=m} sum_o dY[b,n,o] * W[o, c*V + tap[n,k]]``).
* weight gradient — the contraction runs over the batch, so the batch takes the place of the channels: rows are the
  output channels o, "points" are the layer's output points n holding ``dY^T [o][n][b]``, the "taps" are the layer's input
  points m holding ``X^T [m][c][b]`` in the packed-weight layout, and there is one "output point" per filter tap v whose
  neighbour list is every (n, m) pair that uses v
  (``dW[o,c,v] = sum_{(n,k): tap[n,k]=v} sum_b dY[b,n,o] * X[b,idx[k,n],c]``).  Lists longer than the kernel's limit are
  split and the parts added into their tap's rows by the kernel's epilogue.  Layers with at most 4 input channels use one GEMM per output point instead (see
  ``_weight_grad_few``).

Operands are bf16 with float32 accumulation, as under the reference's autocast training.  Layers that run on the exact
float32 kernel (``precision='fp32'``, or shapes outside the tensor-core kernel) take the same two derived layers through
that kernel instead (``input_grad_f32`` / ``weight_grad_f32``): float32 arithmetic throughout, for parity work, not speed.
"""
import numpy as np
import torch

from . import ops

__all__ = ["KnnConvGrad", "knnconv_autograd", "knnconv_points_autograd"]

MAX_LIST = 256      # longest neighbour list the tensor-core kernel takes


def _grouped(keys, n_groups, limit=None):
    """Stable grouping of entry indices by key.  Returns (order, group id of each ordered entry, position inside its
    group, number of groups, parts).  With `limit`, groups longer than it are cut into consecutive parts; `parts` is then
    either an int P (every key has P parts, some possibly empty: part p of key g is group g*P + p) or, when that would
    leave too many empty parts, the array of each group's owner key."""
    order = np.argsort(keys, kind="stable")
    k = keys[order]
    start = np.searchsorted(k, np.arange(n_groups))
    pos = np.arange(k.size) - start[k]
    if limit is None:
        return order, k, pos, n_groups, 1
    counts = np.bincount(k, minlength=n_groups)
    need = np.maximum(1, -(-counts // limit))
    P = int(need.max()) if need.size else 1
    if n_groups * P <= 1.3 * need.sum():                    # few empty parts: uniform, the parts are summed by a reduction
        return order, k * P + pos // limit, pos % limit, n_groups * P, P
    first = np.concatenate([[0], np.cumsum(need)[:-1]])     # uneven lists: as many parts as each key needs, summed by index
    return order, first[k] + pos // limit, pos % limit, int(need.sum()), np.repeat(np.arange(n_groups), need)


class KnnConvGrad:
    """Derived plans of one KNNConv layer's backward pass (built on first use, cached)."""

    def __init__(self, knn_idx_pad, tap, n_in, V, c_in, c_out, device):
        idx = np.asarray(knn_idx_pad).astype(np.int64)          # [K, n_out], pad == n_in
        tp = np.asarray(tap).astype(np.int64)                   # [n_out, K]
        self.n_in, self.V, self.c_in, self.c_out, self.device = int(n_in), int(V), int(c_in), int(c_out), device
        self.K, self.n_out = idx.shape
        ks, ns = np.nonzero(idx != n_in)
        self._n, self._m, self._v, self._k = ns, idx[ks, ns], tp[ns, ks], ks
        self._idx, self._tap, self._few = idx, tp, None
        self._dx_plan = None
        self._dw_plans = {}
        self.c_in_pad = -(-self.c_in // 16) * 16

    # ---- dX
    def dx_plan(self):
        if self._dx_plan is None:
            if self.c_in % 16:
                raise NotImplementedError("input gradient needs in_channels to be a multiple of 16 (a first layer's input needs none)")
            order, gid, pos, _, _ = _grouped(self._m, self.n_in)
            kt = max(8, int(pos.max()) + 1 if pos.size else 8)
            if kt > MAX_LIST:
                raise NotImplementedError(f"an input point feeds {kt} outputs; the kernel takes lists up to {MAX_LIST}")
            idx_t = np.full((kt, self.n_in), self.n_out, np.int32)
            tap_t = np.zeros((self.n_in, kt), np.uint16)
            idx_t[pos, gid] = self._n[order]
            tap_t[gid, pos] = self._v[order]
            self._dx_plan = ops.KnnConvPlan(idx_t, tap_t, self.n_out, self.V, self.c_out, self.c_in, device=self.device)
            if not self._dx_plan.tc_supported:
                raise NotImplementedError("the transposed layer is outside the tensor-core kernel's shapes")
        return self._dx_plan

    def input_grad(self, gy_points, weight):
        """gy_points [B, n_out, c_out] bf16 contiguous, weight [c_out, c_in*V] -> dX [B, n_in, c_in] bf16 (channels last)."""
        plan = self.dx_plan()
        w_t = weight.detach().reshape(self.c_out, self.c_in, self.V).permute(1, 0, 2).reshape(self.c_in, self.c_out * self.V)
        return plan.forward(gy_points, plan.pack_weights(w_t.contiguous()), out_dtype=torch.bfloat16)

    # ---- dW
    @property
    def dw_swapped(self):
        """Which operand gives the rows of the weight-gradient GEMM.  An MMA costs about the same whatever its width, so
        a layer with few input channels and many output channels (64 -> 192) is cheaper the other way round: rows = input
        channels (one 128-row tile on one SM instead of a 256-row tile on a CTA pair), columns = output channels."""
        return self.c_in_pad <= 128 < self.c_out

    def dw_plan(self, bp):
        if bp not in self._dw_plans:
            # Lists are cut so that there are a few hundred of them (several per SM pair), whatever the number of taps.
            limit = int(min(MAX_LIST, max(8, -(-self._v.size // 300 // 8) * 8)))
            order, gid, pos, n_groups, parts = _grouped(self._v, self.V, limit)
            kw = max(8, int(pos.max()) + 1 if pos.size else 8)
            # gathered side ("points") and streamed side ("taps") of a pair: (n, m), or (m, n) when swapped
            pts, taps = (self._m, self._n) if self.dw_swapped else (self._n, self._m)
            n_pts, n_taps = (self.n_in, self.n_out) if self.dw_swapped else (self.n_out, self.n_in)
            idx_w = np.full((kw, n_groups), n_pts, np.int32)
            tap_w = np.zeros((n_groups, kw), np.uint16)
            idx_w[pos, gid] = pts[order]
            tap_w[gid, pos] = taps[order]
            plan = ops.KnnConvPlan(idx_w, tap_w, n_pts, n_taps, bp, self.c_out if self.dw_swapped else self.c_in_pad, device=self.device)
            if not plan.tc_supported:
                raise NotImplementedError("the weight-gradient contraction is outside the tensor-core kernel's shapes")
            owner = np.arange(n_groups) // parts if isinstance(parts, int) else parts          # tap of each part
            self._dw_plans[bp] = (plan, torch.from_numpy(np.ascontiguousarray(owner, dtype=np.int32)).to(self.device))
        return self._dw_plans[bp]

    # ---- exact float32 route (precision='fp32' layers and shapes outside the tensor-core kernel): the same two derived
    # layers, run on the exact float32 kernel (fovi_knnconv_forward_f32) instead of the tensor cores
    def _f32_plans(self, B):
        key = ("f32", B)
        if key not in self._dw_plans:
            order, gid, pos, _, _ = _grouped(self._m, self.n_in)
            kt = max(1, int(pos.max()) + 1 if pos.size else 1)
            idx_t = np.full((kt, self.n_in), self.n_out, np.int32)
            tap_t = np.zeros((self.n_in, kt), np.uint16)
            idx_t[pos, gid] = self._n[order]
            tap_t[gid, pos] = self._v[order]
            dx = ops.KnnConvPlan(idx_t, tap_t, self.n_out, self.V, self.c_out, self.c_in, device=self.device)
            order, gid, pos, n_groups, parts = _grouped(self._v, self.V, 512)
            kw = max(1, int(pos.max()) + 1 if pos.size else 1)
            idx_w = np.full((kw, n_groups), self.n_out, np.int32)
            tap_w = np.zeros((n_groups, kw), np.uint16)
            idx_w[pos, gid] = self._n[order]
            tap_w[gid, pos] = self._m[order]
            dw = ops.KnnConvPlan(idx_w, tap_w, self.n_out, self.n_in, B, self.c_in, device=self.device)
            owner = np.arange(n_groups) // parts if isinstance(parts, int) else parts
            self._dw_plans[key] = (dx, dw, torch.from_numpy(np.ascontiguousarray(owner, dtype=np.int64)).to(self.device))
        return self._dw_plans[key]

    def input_grad_f32(self, gy, weight):
        """gy [B, c_out, n_out], weight [c_out, c_in*V] -> dX [B, c_in, n_in], float32 arithmetic throughout."""
        dx, _, _ = self._f32_plans(gy.shape[0])
        w_t = weight.detach().float().reshape(self.c_out, self.c_in, self.V).permute(1, 0, 2).reshape(self.c_in, self.c_out * self.V)
        return dx.forward_f32(gy.float(), dx.pack_weights(w_t.contiguous(), dtype=torch.float32))

    def weight_grad_f32(self, gy, x):
        """gy [B, c_out, n_out], x [B, c_in, n_in] -> dW [c_out, c_in*V] float32: rows = output channels, "channels" = the
        batch, "taps" = the input points holding X^T, one pseudo output point per part of a filter tap's pair list."""
        B = gy.shape[0]
        _, dw, owner = self._f32_plans(B)
        rows = gy.float().permute(1, 0, 2).contiguous()                               # [c_out, B, n_out]
        taps = torch.zeros((self.n_in, self.c_in, dw.cin_packed), dtype=torch.float32, device=gy.device)
        taps[:, :, :B] = x.float().permute(2, 1, 0)                                   # [n_in, c_in, B]
        parts = dw.forward_f32(rows, taps)                                            # [c_out, c_in, parts]
        out = torch.zeros((self.c_out, self.c_in, self.V), dtype=torch.float32, device=gy.device)
        out.index_add_(2, owner, parts)
        return out.reshape(self.c_out, self.c_in * self.V)

    # ---- dW of a layer with at most 4 input channels
    # One tap's pair list would give MMAs of only c_in columns (a 64x3 outer product per pair fills 9 % of an MMA).  Instead
    # there is one GEMM per output point n: rows = output channels, columns = (neighbour k, channel c), contraction over the
    # batch, P_n[o,(k,c)] = sum_b dY[b,n,o] * X[b,idx[k,n],c].  To the kernel this is a layer in which point n has the single
    # neighbour n and its own "weight slab": X^T gathered by n's neighbour list, [n][(k,c)][b].  The products of every
    # filter tap's pairs are then summed into dW[o,c,tap] by a segment-sum kernel (fovi_tap_segment_sum).  Points are processed in chunks so that the gathered operand stays near 256 MB.
    def _few_tables(self, idx, tap):
        K, kp = self.K, (-(-self.K // 4) * 4 if self.K <= 64 else -(-self.K // 64) * 64)
        gather = np.full((self.n_out, kp), self.n_in, np.int64)          # row n_in of the operand is zero
        gather[:, :K] = idx.T
        return kp, torch.from_numpy(gather).to(self.device)

    def _few_segments(self, n0, npts, kp):
        """Slots (n - n0) * kp + k of the chunk's valid (output point, neighbour) pairs, grouped by filter tap."""
        key = ("seg", n0, npts)
        if key not in self._dw_plans:
            sel = (self._n >= n0) & (self._n < n0 + npts)
            n, v, ks = self._n[sel], self._v[sel], self._k[sel]
            order = np.argsort(v, kind="stable")
            start = np.searchsorted(v[order], np.arange(self.V + 1)).astype(np.int32)
            slot = ((n[order] - n0) * kp + ks[order]).astype(np.int32)
            self._dw_plans[key] = (torch.from_numpy(start).to(self.device), torch.from_numpy(slot).to(self.device))
        return self._dw_plans[key]

    def _few_plan(self, bp, n0, npts):
        key = ("few", bp, n0, npts)
        if key not in self._dw_plans:
            idx = (n0 + np.arange(npts, dtype=np.int32))[None, :]
            tp = np.arange(npts, dtype=np.uint16)[:, None]
            plan = ops.KnnConvPlan(idx, tp, self.n_out, npts, bp, 4 * self._few[0], device=self.device)
            if not plan.tc_supported:
                raise NotImplementedError("the weight-gradient contraction is outside the tensor-core kernel's shapes")
            self._dw_plans[key] = plan
        return self._dw_plans[key]

    def _weight_grad_few(self, gy, x, gy_inner=None):
        B = gy.shape[0]
        bp = -(-B // 64) * 64
        if self._few is None:
            self._few = self._few_tables(self._idx, self._tap)
        kp, gather = self._few
        gy_t = gy_inner if gy_inner is not None else ops.batch_to_inner(gy, bp=bp)      # [c_out, n_out, bp]
        x_t = torch.zeros((self.n_in + 1, 4, bp), dtype=torch.bfloat16, device=x.device)
        ops.batch_to_inner(x.permute(0, 2, 1), jp=4, bp=bp, out=x_t[:self.n_in])        # [n_in (+ zero row), 4, bp]
        dw = torch.zeros((self.c_out, self.V * 4), dtype=torch.float32, device=gy.device)
        chunk = max(1, min(self.n_out, 0xFFFF, (256 << 20) // (kp * 4 * bp * 2)))
        for n0 in range(0, self.n_out, chunk):
            npts = min(chunk, self.n_out - n0)
            slab = x_t[gather[n0:n0 + npts]].reshape(npts, kp * 4, bp)                  # [n][(k,c)][b]
            prod = self._few_plan(bp, n0, npts).forward(gy_t, slab, out_dtype=torch.float32)    # [c_out, npts, kp*4]
            seg_start, seg_slot = self._few_segments(n0, npts, kp)
            ops.tap_segment_sum(prod.view(self.c_out, npts * kp, 4), seg_start, seg_slot, dw)   # every tap sums its pairs
        return dw.reshape(self.c_out, self.V, 4)[:, :, :self.c_in].permute(0, 2, 1).reshape(self.c_out, self.c_in * self.V)

    def gy_inner_view(self, gy_points):
        """The view of the upstream gradient ([B, n_out, c_out], channels last) whose batch-innermost copy `weight_grad`
        wants: logical [B, I, J] with dst [I, J, bp] = [c_out, n_out, bp], or [n_out, c_out, bp] for a turned GEMM."""
        return gy_points if (self.dw_swapped and self.c_in > 4) else gy_points.permute(0, 2, 1)

    def weight_grad(self, gy, x, gy_inner=None):
        """gy [B, c_out, n_out] and x [B, c_in, n_in] (any strides/dtype) -> dW [c_out, c_in*V] float32.
        `gy_inner`: the batch-innermost copy of gy (see gy_inner_view), when the caller already has it."""
        if self.c_in <= 4:
            return self._weight_grad_few(gy, x, gy_inner)
        B = gy.shape[0]
        bp = -(-B // 64) * 64
        plan, owner = self.dw_plan(bp)
        # every part of a tap's list is reduced into the tap's rows by the kernel's epilogue (float32 reductions in L2)
        if self.dw_swapped:
            x_r = ops.batch_to_inner(x, bp=bp)                                          # rows: [c_in, n_in, bp]
            gy_w = gy_inner if gy_inner is not None else ops.batch_to_inner(gy.permute(0, 2, 1), jp=self.c_out, bp=bp)   # "weights": [n_out, c_out, bp]
            dw_t = torch.zeros((self.c_in, self.V, self.c_out), dtype=torch.float32, device=gy.device)
            plan.forward_scatter_add(x_r, gy_w, owner, dw_t)
            return dw_t.permute(2, 0, 1).reshape(self.c_out, self.c_in * self.V)
        gy_t = gy_inner if gy_inner is not None else ops.batch_to_inner(gy, bp=bp)     # rows: [c_out, n_out, bp]
        x_t = ops.batch_to_inner(x.permute(0, 2, 1), jp=self.c_in_pad, bp=bp)          # "weights": [n_in, c_in_pad, bp]
        dw = torch.zeros((self.c_out, self.V, self.c_in_pad), dtype=torch.float32, device=gy.device)
        plan.forward_scatter_add(gy_t, x_t, owner, dw)
        return dw[:, :, :self.c_in].permute(0, 2, 1).reshape(self.c_out, self.c_in * self.V)


class _KnnConvFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, layer):
        ctx.layer = layer
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x, weight)
        with torch.no_grad():
            return layer._forward(x)

    @staticmethod
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        g = ctx.layer.grad_plans
        gx = gw = gb = None
        if ctx.layer.precision == "fp32" or not ctx.layer.plan.tc_supported:      # the forward ran on the exact float32 kernel
            if ctx.needs_input_grad[0]:
                gx = g.input_grad_f32(gy, weight).to(x.dtype)
            if ctx.needs_input_grad[1]:
                gw = g.weight_grad_f32(gy, x).to(weight.dtype)
            if ctx.has_bias and ctx.needs_input_grad[2]:
                gb = gy.sum((0, 2), dtype=torch.float32)
            return gx, gw, gb, None
        if ctx.needs_input_grad[0]:
            gyp = gy.permute(0, 2, 1).to(torch.bfloat16).contiguous()
            gx = g.input_grad(gyp, weight).permute(0, 2, 1).to(x.dtype)
        if ctx.needs_input_grad[1]:
            gw = g.weight_grad(gy, x).to(weight.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = gy.sum((0, 2), dtype=torch.float32)
        return gx, gw, gb, None


class _KnnConvPointsFunction(torch.autograd.Function):
    """A layer on the kernels' own activation layout (channels last, bf16) with the ReLU fused, so that a chain of layers
    trains without a layout change between them.  `x` is [B, n_in, c_in] bf16, or for a pair-layout first layer the
    [B, c_in, n_in] input itself (it is packed here)."""

    @staticmethod
    def forward(ctx, x, weight, bias, layer, relu):
        plan = layer.plan
        first = plan.x_layout == ops.X_PAIRS
        rows = x.shape[0]
        with torch.no_grad():
            xp = ops.pack_points(x, plan) if first else x.contiguous()
            y = plan.forward(xp, layer.packed_weight(), bias, relu=relu, out_dtype=torch.bfloat16, batch=rows)
        ctx.layer, ctx.relu, ctx.first, ctx.has_bias = layer, relu, first, bias is not None
        ctx.save_for_backward(x, weight, y if relu else None)
        return y

    @staticmethod
    def backward(ctx, gy):
        x, weight, y = ctx.saved_tensors
        g = ctx.layer.grad_plans
        gy = gy.to(torch.bfloat16)
        want_w, want_b = ctx.needs_input_grad[1], ctx.has_bias and ctx.needs_input_grad[2]
        gy_inner = gb = None
        if ctx.relu and want_w and gy.is_contiguous():
            # ReLU mask, bias sums and the batch-innermost copy the weight gradient needs, in one pass over the gradient
            bp = -(-gy.shape[0] // 64) * 64
            view = g.gy_inner_view(gy)
            fused = ops.relu_backward_to_inner(view, g.gy_inner_view(y), bp=bp, want_masked=ctx.needs_input_grad[0],
                                               want_colsum=want_b)    # the sums run over all but the contiguous index: per channel
            if fused is not None:
                masked, gy_inner, gb = fused
                gy = gy if masked is None else (masked if view is gy else masked.permute(0, 2, 1))
        if gy_inner is None:
            if ctx.relu:
                gy = torch.ops.aten.threshold_backward(gy, y, 0)       # gy where y > 0, else 0: one pass
            gy = gy.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            if ctx.first:
                raise NotImplementedError("input gradient of a pair-layout first layer is not built")
            gx = g.input_grad(gy, weight)                                      # [B, n_in, c_in] bf16
        if want_w:
            gw = g.weight_grad(gy.permute(0, 2, 1), x if ctx.first else x.permute(0, 2, 1), gy_inner=gy_inner).to(weight.dtype)
        if want_b and gb is None:
            gb = ops.column_sum(gy) if gy.shape[-1] % 2 == 0 else gy.sum((0, 1), dtype=torch.float32)
        return gx, gw, gb, None, None


def knnconv_points_autograd(layer, x, relu):
    return _KnnConvPointsFunction.apply(x, layer.weight, layer.bias, layer, relu)


def knnconv_autograd(layer, x):
    """layer(x) with gradients: forward on the layer's kernels, backward as described in this module."""
    return _KnnConvFunction.apply(x, layer.weight, layer.bias, layer)
