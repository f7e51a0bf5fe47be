"""Tensor-level wrappers over the C ABI: plans own device tables, functions take torch CUDA
tensors, pass raw pointers and the current stream, and allocate outputs with torch."""
import ctypes as C

import numpy as np
import torch

from ._lib import lib, check

F32, BF16, U8 = 0, 1, 2
NEAREST, BILINEAR = 0, 1
PAD_ZEROS, PAD_BORDER = 0, 1
OUT_BFCN, OUT_FBCN, OUT_BFNC, OUT_FBNC, OUT_FB_PAIRS, OUT_BF_PAIRS = 0, 1, 2, 3, 4, 5
X_BNC, X_PAIRS = 0, 1
ACT_BCN, ACT_BNC = 0, 1

_DT = {torch.float32: F32, torch.bfloat16: BF16}


def _dt(t):
    try:
        return _DT[t]
    except KeyError:
        raise TypeError(f"unsupported dtype {t}: the kernels take float32 or bfloat16") from None


def _stream():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t):
    return C.c_void_p(t.data_ptr())


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("fovi_b200 kernels need CUDA tensors; there is no CPU path")


class SamplerPlan:
    """Device copy of a sensor's sampling grid in visiting order (fovi_sampler_plan)."""

    def __init__(self, grid_xy, device=None):
        g = np.ascontiguousarray(np.asarray(grid_xy, np.float32).reshape(-1, 2))
        self.n_points = g.shape[0]
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.fovi_sampler_plan_create(g.ctypes.data_as(C.c_void_p), self.n_points, C.byref(h)), "fovi_sampler_plan_create")
        self._h = h

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None:          # `lib` is already gone when the interpreter is shutting down
            lib.fovi_sampler_plan_destroy(h)

    def check(self):
        """Synchronise the current stream and raise if a sampler launch gave up waiting for its image copies."""
        with torch.cuda.device(self.device):
            check(lib.fovi_sampler_check(self._h, _stream()), "fovi_sampler_check")


def sample(plan, img, fix_rc, fix_hw, mode=BILINEAR, pad=PAD_ZEROS, out_dtype=None, layout=OUT_BFCN, channel_stride=None, out=None):
    """img [B,C,H,W] (any strides; float32, bfloat16, or uint8 sampled as the float32 values it holds);
    fix_rc, fix_hw [B,F,2] float32 CUDA.  Returns the sampled
    tensor in `layout`: [B,F,C,N], [F,B,C,N], [B,F,N,Cp], [F,B,N,Cp], or the pair layout
    [ceil(rows/128), ceil(N/2), 128, 8] (rows = F*B or B*F) that a KNNConv plan with c_in <= 4
    consumes; rows past the last one are left unwritten."""
    _need_cuda(img, fix_rc, fix_hw)
    B, Cc, H, W = img.shape
    fix_rc = fix_rc.to(torch.float32).contiguous()
    fix_hw = fix_hw.to(torch.float32).contiguous()
    F = fix_rc.shape[1]
    assert fix_rc.shape == (B, F, 2) and fix_hw.shape == (B, F, 2)
    if out_dtype is None:
        out_dtype = torch.float32 if img.dtype == torch.uint8 else img.dtype
    nc = layout in (OUT_BFNC, OUT_FBNC)
    pairs = layout in (OUT_FB_PAIRS, OUT_BF_PAIRS)
    cp = (channel_stride or Cc) if nc else Cc
    lead = (F, B) if layout in (OUT_FBCN, OUT_FBNC) else (B, F)
    if pairs:
        out_dtype, cp = torch.bfloat16, 8
        shape = ((B * F + 127) // 128, (plan.n_points + 1) // 2, 128, 8)
    else:
        shape = lead + ((plan.n_points, cp) if nc else (Cc, plan.n_points))
    if out is None:
        out = torch.empty(shape, dtype=out_dtype, device=img.device)
    else:
        assert out.shape == shape and out.dtype == out_dtype and out.is_contiguous()
    strides = (C.c_int64 * 4)(*img.stride())
    with torch.cuda.device(img.device):
        check(lib.fovi_sample_forward(plan._h, _ptr(img), U8 if img.dtype == torch.uint8 else _dt(img.dtype), B, Cc, H, W, strides, _ptr(fix_rc), _ptr(fix_hw), F,
                                      mode, pad, _ptr(out), _dt(out_dtype), layout, cp, _stream()), "fovi_sample_forward")
    return out


def group_tables(idx, tap, n_in, G, max_list=256):
    """Tables of a grouped plan.  idx [K, n_out] int (pad == n_in), tap [n_out, K]; n_out a multiple of G.
    Returns (union lists int32 [Kq, n_out/G] padded with n_in, tap table uint16 [n_out/G, Kq] holding each entry's own
    position, member taps uint16 [n_out/G, Kq, G] with 0xFFFF where the entry is not a neighbour of that member), or
    None when a union list would exceed `max_list` entries or a member lists a point twice."""
    idx = np.asarray(idx)
    tap = np.asarray(tap)
    K, n_out = idx.shape
    ng = n_out // G
    cols = idx.T.reshape(ng, G * K).astype(np.int64)               # members' lists side by side
    taps = tap.reshape(ng, G * K).astype(np.int64)
    member = np.repeat(np.arange(G), K)[None, :].repeat(ng, 0)
    order = np.argsort(cols, axis=1, kind="stable")
    sc = np.take_along_axis(cols, order, 1)
    mem = np.take_along_axis(member, order, 1)
    first = np.ones_like(sc, dtype=bool)
    first[:, 1:] = sc[:, 1:] != sc[:, :-1]
    first &= sc != n_in                                              # pad entries join no list
    if ((sc[:, 1:] == sc[:, :-1]) & (mem[:, 1:] == mem[:, :-1]) & (sc[:, 1:] != n_in)).any():
        return None
    pos = np.cumsum(first, 1) - 1                                    # position of each entry's point in the union list
    ku = int(first.sum(1).max()) if first.size else 0
    if ku > max_list or ku == 0:
        return None
    kq = -(-ku // 8) * 8
    uidx = np.full((kq, ng), n_in, np.int32)
    mtap = np.full((ng, kq, G), 0xFFFF, np.uint16)
    rows = np.arange(ng)[:, None].repeat(G * K, 1)
    valid = sc != n_in
    uidx[pos[valid], rows[valid]] = sc[valid]
    mtap[rows[valid], pos[valid], mem[valid]] = np.take_along_axis(taps, order, 1)[valid]
    utap = np.ascontiguousarray(np.arange(kq, dtype=np.uint16)[None, :].repeat(ng, 0))
    return np.ascontiguousarray(uidx), utap, np.ascontiguousarray(mtap)


def sample_backward(plan, grad_out, img_shape, fix_rc, fix_hw, mode=BILINEAR, pad=PAD_ZEROS, layout=OUT_BFCN, grad_img=None):
    """Gradient of `sample` with respect to the image.  grad_out [B,F,C,N] (or [F,B,C,N]) float32/bf16 -> float32
    [B,C,H,W]; with `grad_img` given the gradient is accumulated into it."""
    _need_cuda(grad_out, fix_rc, fix_hw)
    B, Cc, H, W = img_shape
    F = fix_rc.shape[1]
    grad_out = grad_out.contiguous()
    assert grad_out.shape == ((B, F, Cc, plan.n_points) if layout == OUT_BFCN else (F, B, Cc, plan.n_points)), grad_out.shape
    if grad_img is None:
        grad_img = torch.zeros((B, Cc, H, W), dtype=torch.float32, device=grad_out.device)
    assert grad_img.dtype == torch.float32 and grad_img.is_contiguous() and tuple(grad_img.shape) == (B, Cc, H, W)
    with torch.cuda.device(grad_out.device):
        check(lib.fovi_sample_backward(plan._h, _ptr(grad_out), _dt(grad_out.dtype), layout, B, Cc, H, W, _ptr(fix_rc.to(torch.float32).contiguous()),
                                       _ptr(fix_hw.to(torch.float32).contiguous()), F, mode, pad, _ptr(grad_img), _stream()), "fovi_sample_backward")
    return grad_img


class KnnConvPlan:
    """Device copy of one layer's compacted neighbour/tap tables (fovi_knnconv_plan)."""

    def __init__(self, knn_idx_pad, tap, n_in, V, c_in, c_out, device=None, group=None):
        """`group`: output points per accumulator of a pair-layout (c_in <= 4) layer's tensor-core path; None picks the
        largest of 4, 3, 2 that divides n_out and keeps group*c_out <= 256 (1 = no grouping)."""
        idx = np.ascontiguousarray(np.asarray(knn_idx_pad, np.int32))
        tp = np.ascontiguousarray(np.asarray(tap, np.uint16))
        K, n_out = idx.shape
        assert tp.shape == (n_out, K), (tp.shape, idx.shape)
        self.n_in, self.n_out, self.K, self.V, self.c_in, self.c_out = int(n_in), n_out, K, int(V), int(c_in), int(c_out)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.fovi_knnconv_plan_create(idx.ctypes.data_as(C.c_void_p), tp.ctypes.data_as(C.c_void_p), self.n_in, n_out, K,
                                               self.V, self.c_in, self.c_out, C.byref(h)), "fovi_knnconv_plan_create")
        self._h = h
        self.cin_packed = lib.fovi_knnconv_cin_packed(h)
        self.nnz = lib.fovi_knnconv_nnz(h)
        self.x_layout = lib.fovi_knnconv_x_layout(h)
        self.tc_supported = bool(lib.fovi_knnconv_tc_supported(h))
        self.n_pairs = (self.n_in + 1) // 2
        self.group, self._hg, self._member_tap = 1, None, None
        if self.x_layout == X_PAIRS and self.tc_supported and group != 1:
            self._make_grouped(idx, tp, (int(group),) if group else (4, 3, 2))

    def _make_grouped(self, idx, tp, candidates):
        """A second plan whose "points" are groups of G consecutive output points (G*c_out channels side by side) and whose
        neighbour lists are the unions of the members' lists: with 3-4 input channels an MMA over one point's 64-96 output
        channels costs as much to issue as one over 256, and consecutive points share most of their neighbours."""
        for G in candidates:
            if G < 2 or self.n_out % G or G * self.c_out > 256:
                continue
            tables = group_tables(idx, tp, self.n_in, G)
            if tables is None:
                continue
            uidx, utap, mtap = tables
            kq, ng = uidx.shape
            hg = C.c_void_p()
            with torch.cuda.device(self.device):
                check(lib.fovi_knnconv_plan_create(uidx.ctypes.data_as(C.c_void_p), utap.ctypes.data_as(C.c_void_p), self.n_in, ng, kq, kq,
                                                   self.c_in, G * self.c_out, C.byref(hg)), "fovi_knnconv_plan_create")
            if not lib.fovi_knnconv_tc_supported(hg):
                lib.fovi_knnconv_plan_destroy(hg)
                continue
            self.group, self._hg, self._kq = G, hg, kq
            self._member_tap = torch.from_numpy(mtap.view(np.int16)).to(self.device)
            return

    @property
    def _h_tc(self):
        """Handle the tensor-core entry points take: the grouped plan when there is one."""
        return self._hg if self._hg else self._h

    def _tc_bias(self, bias):
        """Bias as the tensor-core entry point wants it: a grouped plan's "channels" are the members' channels side by
        side, so the layer's bias is repeated once per member.  Recomputed on every call (a few hundred bytes): any
        cache keyed on the tensor's address or version would go stale when a caller passes a freshly folded temporary
        that happens to reuse a freed address."""
        if bias is None or self.group == 1:
            return bias
        return bias.detach().float().repeat(self.group)

    def __del__(self):
        for name in ("_h", "_hg"):
            h = getattr(self, name, None)
            setattr(self, name, None)
            if h and lib is not None:
                lib.fovi_knnconv_plan_destroy(h)

    def flops_per_image(self):
        """Algorithmic FLOPs of one forward for one image: 2 * c_in * c_out * nnz."""
        return 2 * self.c_in * self.c_out * self.nnz

    def pack_weights(self, weight, dtype=torch.bfloat16):
        """weight [c_out, c_in*V] (KNNConvLayer.weight) -> packed operand: slabs [V, c_out, cin_packed], or
        (bf16, pair layout) per-output-point slabs [n_out, pair_slots, c_out, 8]."""
        _need_cuda(weight)
        weight = weight.detach().contiguous()
        assert weight.shape == (self.c_out, self.c_in * self.V)
        if self._hg and dtype == torch.bfloat16:
            nbytes = lib.fovi_knnconv_packed_weight_bytes(self._hg, _dt(dtype))
            ng, cg = self.n_out // self.group, self.group * self.c_out
            dst = torch.empty((ng, nbytes // (ng * cg * 16), cg, 8), dtype=dtype, device=weight.device)
            with torch.cuda.device(weight.device):
                check(lib.fovi_knnconv_pack_weights_grouped(self._hg, _ptr(weight), _dt(weight.dtype), _ptr(self._member_tap), self.group, self.V,
                                                            _ptr(dst), _stream()), "fovi_knnconv_pack_weights_grouped")
            return dst
        nbytes = lib.fovi_knnconv_packed_weight_bytes(self._h, _dt(dtype))
        if self.x_layout == X_PAIRS and dtype == torch.bfloat16:
            dst = torch.empty((self.n_out, nbytes // (self.n_out * self.c_out * 16), self.c_out, 8), dtype=dtype, device=weight.device)  # memory order [n_out, c_out tiles, slots, tile, 8]
        else:
            dst = torch.empty((self.V, self.c_out, self.cin_packed), dtype=dtype, device=weight.device)
        assert dst.numel() * dst.element_size() == nbytes
        with torch.cuda.device(weight.device):
            check(lib.fovi_knnconv_pack_weights(self._h, _ptr(weight), _dt(weight.dtype), _ptr(dst), _dt(dtype), _stream()), "fovi_knnconv_pack_weights")
        return dst

    def forward(self, x_bnc, wt, bias=None, relu=False, out_dtype=torch.bfloat16, out=None, batch=None):
        """Tensor-core path.  x_bnc: bf16 contiguous, [B,n_in,cin_packed] or (pair layout)
        [ceil(B/128),n_pairs,128,8] with `batch` = B  ->  [B,n_out,c_out]."""
        _need_cuda(x_bnc, wt, bias)
        assert x_bnc.dtype == torch.bfloat16 and x_bnc.is_contiguous() and wt.dtype == torch.bfloat16 and wt.is_contiguous()
        if self.x_layout == X_PAIRS:
            B = x_bnc.shape[0] * 128 if batch is None else int(batch)
            assert x_bnc.shape == ((B + 127) // 128, self.n_pairs, 128, 8), (x_bnc.shape, B)
            assert wt.dim() == 4 and wt.shape[0] == self.n_out // self.group and wt.shape[2:] == (self.group * self.c_out, 8), wt.shape
        else:
            B = x_bnc.shape[0]
            assert x_bnc.shape[1:] == (self.n_in, self.cin_packed), x_bnc.shape
            assert wt.shape == (self.V, self.c_out, self.cin_packed)
        if bias is not None:
            bias = self._tc_bias(bias).detach().to(torch.float32).contiguous()
        if out is None:
            out = torch.empty((B, self.n_out, self.c_out), dtype=out_dtype, device=x_bnc.device)
        with torch.cuda.device(x_bnc.device):   # a grouped plan writes [B, n_out/G, G*c_out]: the same memory
            check(lib.fovi_knnconv_forward(self._h_tc, _ptr(x_bnc), _ptr(wt), _ptr(bias) if bias is not None else None, _ptr(out),
                                           _dt(out.dtype), B, int(relu), _stream()), "fovi_knnconv_forward")
        return out

    def forward_scatter_add(self, x_bnc, wt, out_map, out):
        """Tensor-core path whose output point n is ADDED into out[:, out_map[n], :] (out: float32 [B, n_out_y, c_out],
        initialised by the caller; out_map: int32 [n_out] on the device).  See fovi_knnconv_forward_scatter_add."""
        _need_cuda(x_bnc, wt, out_map, out)
        assert self.x_layout != X_PAIRS and x_bnc.dtype == torch.bfloat16 and x_bnc.is_contiguous() and wt.dtype == torch.bfloat16 and wt.is_contiguous()
        B = x_bnc.shape[0]
        assert x_bnc.shape[1:] == (self.n_in, self.cin_packed) and wt.shape == (self.V, self.c_out, self.cin_packed)
        assert out_map.dtype == torch.int32 and out_map.is_contiguous() and out_map.numel() == self.n_out
        assert out.dtype == torch.float32 and out.is_contiguous() and out.dim() == 3 and out.shape[0] == B and out.shape[2] == self.c_out
        with torch.cuda.device(x_bnc.device):
            check(lib.fovi_knnconv_forward_scatter_add(self._h_tc, _ptr(x_bnc), _ptr(wt), _ptr(out), B, _ptr(out_map), int(out.shape[1]),
                                                       _stream()), "fovi_knnconv_forward_scatter_add")
        return out

    def forward_f32(self, x, wt_f32, bias=None, relu=False, x_layout=ACT_BCN, y_layout=ACT_BCN):
        """Exact float32 path.  x [B,c_in,n_in] (BCN) or [B,n_in,c_in] (BNC)."""
        _need_cuda(x, wt_f32, bias)
        x = x.contiguous()
        B = x.shape[0]
        assert x.shape[1:] == ((self.c_in, self.n_in) if x_layout == ACT_BCN else (self.n_in, self.c_in)), x.shape
        assert wt_f32.dtype == torch.float32 and wt_f32.shape == (self.V, self.c_out, self.cin_packed)
        if bias is not None:
            bias = bias.detach().to(torch.float32).contiguous()
        shape = (B, self.c_out, self.n_out) if y_layout == ACT_BCN else (B, self.n_out, self.c_out)
        out = torch.empty(shape, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            check(lib.fovi_knnconv_forward_f32(self._h, _ptr(x), _dt(x.dtype), x_layout, _ptr(wt_f32), _ptr(bias) if bias is not None else None,
                                               _ptr(out), y_layout, B, int(relu), _stream()), "fovi_knnconv_forward_f32")
        return out

    def selftest_wait_timeout(self, x_bnc, wt, batch=None, out_dtype=torch.bfloat16):
        """Diagnostic: launch the tensor-core kernel with its operand loads withheld and a short wait limit.  The next
        `check()` must raise FoviError (device timeout) and the context stays usable."""
        _need_cuda(x_bnc, wt)
        B = (x_bnc.shape[0] * 128 if batch is None else int(batch)) if self.x_layout == X_PAIRS else x_bnc.shape[0]
        out = torch.zeros((B, self.n_out, self.c_out), dtype=out_dtype, device=x_bnc.device)
        with torch.cuda.device(x_bnc.device):
            check(lib.fovi_knnconv_selftest_wait_timeout(self._h_tc, _ptr(x_bnc), _ptr(wt), _ptr(out), _dt(out.dtype), B, _stream()),
                  "fovi_knnconv_selftest_wait_timeout")

    def depthwise(self, x, wp, bias=None, relu=False, x_layout=ACT_BCN, y_layout=ACT_BCN, out_dtype=None):
        """Depthwise convolution on this plan's tables.  x [B,c_in,n_in] (BCN) or [B,n_in,c_in] (BNC), float32/bf16;
        wp float32 [V, c_out] with wp[v, c*g+j] = W[c, v, j]."""
        _need_cuda(x, wp, bias)
        x = x.contiguous()
        B = x.shape[0]
        assert x.shape[1:] == ((self.c_in, self.n_in) if x_layout == ACT_BCN else (self.n_in, self.c_in)), x.shape
        assert wp.dtype == torch.float32 and wp.shape == (self.V, self.c_out) and wp.is_contiguous()
        if bias is not None:
            bias = bias.detach().to(torch.float32).contiguous()
        out_dtype = x.dtype if out_dtype is None else out_dtype
        shape = (B, self.c_out, self.n_out) if y_layout == ACT_BCN else (B, self.n_out, self.c_out)
        out = torch.empty(shape, dtype=out_dtype, device=x.device)
        with torch.cuda.device(x.device):
            check(lib.fovi_knn_depthwise_forward(self._h, _ptr(x), _dt(x.dtype), x_layout, _ptr(wp), _ptr(bias) if bias is not None else None,
                                                 _ptr(out), _dt(out.dtype), y_layout, B, int(relu), _stream()), "fovi_knn_depthwise_forward")
        return out

    def depthwise_backward(self, x, wp, gy, x_layout=ACT_BCN, y_layout=ACT_BCN, need_gx=True, need_gw=True):
        """Gradients of `depthwise`: returns (gX float32 in x's layout or None, gWp float32 [V, c_out] or None)."""
        _need_cuda(x, wp, gy)
        x, gy = x.contiguous(), gy.contiguous()
        B = x.shape[0]
        gx = torch.zeros(x.shape, dtype=torch.float32, device=x.device) if need_gx else None
        gw = torch.zeros((self.V, self.c_out), dtype=torch.float32, device=x.device) if need_gw else None
        with torch.cuda.device(x.device):
            check(lib.fovi_knn_depthwise_backward(self._h, _ptr(x), _dt(x.dtype), x_layout, _ptr(wp), _ptr(gy), _dt(gy.dtype), y_layout, B,
                                                  _ptr(gx) if need_gx else None, _ptr(gw) if need_gw else None, _stream()), "fovi_knn_depthwise_backward")
        return gx, gw

    def check(self):
        """Synchronise the current stream and raise if a tensor-core launch gave up on a wait."""
        with torch.cuda.device(self.device):
            check(lib.fovi_knnconv_check(self._h, _stream()), "fovi_knnconv_check")
            if self._hg:
                check(lib.fovi_knnconv_check(self._hg, _stream()), "fovi_knnconv_check")


def sample_knnconv_fused(splan, cplan, img, fix_rc, fix_hw, wt, bias=None, relu=False, mode=BILINEAR, pad=PAD_ZEROS,
                         out_dtype=torch.bfloat16, intermediate=None, out=None, row_order="fb"):
    """Sensor -> first KNNConv in one C call, the sensor output held in L2 between the two kernels.  Rows '(f b)' or, with
    row_order "bf", '(b f)'.  Returns ([rows, n_out, c_out], intermediate buffer)."""
    _need_cuda(img, fix_rc, fix_hw, wt, bias)
    B, Cc, H, W = img.shape
    F = fix_rc.shape[1]
    need = lib.fovi_fused_intermediate_bytes(cplan._h_tc, B * F)
    if intermediate is None:
        intermediate = torch.zeros(need // 2, dtype=torch.bfloat16, device=img.device)
    assert intermediate.numel() * intermediate.element_size() >= need
    if out is None:
        out = torch.empty((B * F, cplan.n_out, cplan.c_out), dtype=out_dtype, device=img.device)
    if bias is not None:
        bias = cplan._tc_bias(bias).detach().to(torch.float32).contiguous()
    strides = (C.c_int64 * 4)(*img.stride())
    with torch.cuda.device(img.device):
        check(lib.fovi_sample_knnconv_fused(splan._h, cplan._h_tc, _ptr(img), U8 if img.dtype == torch.uint8 else _dt(img.dtype), B, Cc, H, W, strides, _ptr(fix_rc.contiguous()),
                                            _ptr(fix_hw.contiguous()), F, mode, pad, _ptr(intermediate), _ptr(wt),
                                            _ptr(bias) if bias is not None else None, _ptr(out), _dt(out.dtype), int(relu),
                                            {"fb": 0, "bf": 1}[row_order], _stream()),
              "fovi_sample_knnconv_fused")
    return out, intermediate


POOL_MODES = {"max": 0, "avg": 1, "sum": 2, "gaussian": 3}
NORM_MODES = {"channel": 0, "coord": 1, "layer": 2, "group": 3}


class KnnPoolPlan:
    """Device copy of a pooling layer's neighbour table (fovi_knnpool_plan)."""

    def __init__(self, knn_idx_pad, n_in, device=None):
        idx = np.ascontiguousarray(np.asarray(knn_idx_pad, np.int32))
        self.K, self.n_out = idx.shape
        self.n_in = int(n_in)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        h = C.c_void_p()
        with torch.cuda.device(self.device):
            check(lib.fovi_knnpool_plan_create(idx.ctypes.data_as(C.c_void_p), self.n_in, self.n_out, self.K, C.byref(h)), "fovi_knnpool_plan_create")
        self._h = h

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and lib is not None:
            lib.fovi_knnpool_plan_destroy(h)

    def set_weights(self, w_kn):
        """Neighbour weights [K, n_out] float32 of the 'gaussian' mode (KNNPoolingLayer.gaussian_weights)."""
        w = np.ascontiguousarray(np.asarray(w_kn, np.float32))
        assert w.shape == (self.K, self.n_out), w.shape
        with torch.cuda.device(self.device):
            check(lib.fovi_knnpool_set_weights(self._h, w.ctypes.data_as(C.c_void_p)), "fovi_knnpool_set_weights")

    def forward(self, x, mode="max", layout=ACT_BCN):
        """x [B,C,n_in] (ACT_BCN) or [B,n_in,C] (ACT_BNC), float32 or bf16 -> same layout with n_out points."""
        _need_cuda(x)
        x = x.contiguous()
        B = x.shape[0]
        Cc = x.shape[1] if layout == ACT_BCN else x.shape[2]
        assert (x.shape[2] if layout == ACT_BCN else x.shape[1]) == self.n_in, x.shape
        y = torch.empty((B, Cc, self.n_out) if layout == ACT_BCN else (B, self.n_out, Cc), dtype=x.dtype, device=x.device)
        with torch.cuda.device(x.device):
            check(lib.fovi_knnpool_forward(self._h, _ptr(x), _dt(x.dtype), layout, B, Cc, POOL_MODES[mode], _ptr(y), _stream()), "fovi_knnpool_forward")
        return y


    def backward(self, x, gy, mode="max", layout=ACT_BCN):
        """Gradient of `forward` with respect to x: x and gy in `layout` (float32 or bf16) -> float32 tensor of x's shape."""
        _need_cuda(x, gy)
        x, gy = x.contiguous(), gy.contiguous()
        B = x.shape[0]
        Cc = x.shape[1] if layout == ACT_BCN else x.shape[2]
        assert (x.shape[2] if layout == ACT_BCN else x.shape[1]) == self.n_in and gy.shape == ((B, Cc, self.n_out) if layout == ACT_BCN else (B, self.n_out, Cc))
        dx = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            check(lib.fovi_knnpool_backward(self._h, _ptr(x), _dt(x.dtype), _ptr(gy), _dt(gy.dtype), layout, B, Cc, POOL_MODES[mode], _ptr(dx), _stream()),
                  "fovi_knnpool_backward")
        return dx


def knn_norm(x, mode, weight=None, bias=None, eps=1e-5, groups=1, layout=ACT_BCN, relu=False, out_dtype=None):
    """Per-sample normalisation of x ([B,C,N] for ACT_BCN, [B,N,C] for ACT_BNC; float32 or bf16) over the channels
    ('channel'), the points ('coord'), both ('layer') or channel groups x points ('group'); weight / bias float32 of the
    shape the mode asks for (see fovi_knn_norm_forward).  Returns the same layout in `out_dtype` (default: x's)."""
    _need_cuda(x, weight, bias)
    x = x.contiguous()
    B = x.shape[0]
    Cc, N = (x.shape[1], x.shape[2]) if layout == ACT_BCN else (x.shape[2], x.shape[1])
    m = NORM_MODES[mode]
    ng = lib.fovi_knn_norm_stat_groups(m, B, Cc, N, int(groups))
    if ng < 0:
        raise ValueError(f"{Cc} channels do not split into {groups} groups")
    want = {"channel": Cc, "coord": N, "layer": Cc * N, "group": Cc}[mode]
    prm = []
    for t in (weight, bias):
        if t is not None:
            t = t.detach().to(torch.float32).contiguous()
            assert t.numel() == want, (mode, tuple(t.shape), want)
        prm.append(t)
    stats = torch.empty((max(ng, 1), 2), dtype=torch.float32, device=x.device)
    y = torch.empty_like(x, dtype=x.dtype if out_dtype is None else out_dtype)
    with torch.cuda.device(x.device):
        check(lib.fovi_knn_norm_forward(_ptr(x), _dt(x.dtype), layout, B, Cc, N, m, int(groups), _ptr(prm[0]) if prm[0] is not None else None,
                                        _ptr(prm[1]) if prm[1] is not None else None, float(eps), int(relu), _ptr(stats), _ptr(y), _dt(y.dtype),
                                        _stream()), "fovi_knn_norm_forward")
    return y


def pack_points(x, cp=8, x_layout=X_BNC):
    """x [B,C,N] float32/bf16 -> tensor-core input: [B,N,cp] bf16 (pad channels zero) or the pair
    layout [ceil(B/128),ceil(N/2),128,8].  Pass a KnnConvPlan as `cp` to get the layout that plan consumes."""
    _need_cuda(x)
    if isinstance(cp, KnnConvPlan):
        cp, x_layout = cp.cin_packed, cp.x_layout
    x = x.contiguous()
    B, Cc, N = x.shape
    shape = ((B + 127) // 128, (N + 1) // 2, 128, 8) if x_layout == X_PAIRS else (B, N, cp)
    # the pad rows of the last 128-row tile are zeroed so that the buffer holds no stray bit patterns
    dst = (torch.zeros if x_layout == X_PAIRS else torch.empty)(shape, dtype=torch.bfloat16, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.fovi_pack_points(_ptr(x), _dt(x.dtype), B, Cc, N, _ptr(dst), cp, x_layout, _stream()), "fovi_pack_points")
    return dst


def batch_to_inner(src, jp=None, bp=None, out=None):
    """src: logical [B, I, J] float32/bf16 CUDA tensor of any strides with one of the last two contiguous
    -> [I, jp, bp] bf16 with the batch innermost, zero-padded (jp >= J, bp >= B)."""
    _need_cuda(src)
    B, I, J = src.shape
    jp, bp = J if jp is None else int(jp), B if bp is None else int(bp)
    sb, si, sj = src.stride()
    if si != 1 and sj != 1:
        src = src.contiguous()
        sb, si, sj = src.stride()
    if out is None:
        out = torch.empty((I, jp, bp), dtype=torch.bfloat16, device=src.device)
    assert out.shape == (I, jp, bp) and out.dtype == torch.bfloat16 and out.is_contiguous()
    with torch.cuda.device(src.device):
        check(lib.fovi_batch_to_inner(_ptr(src), _dt(src.dtype), B, I, J, sb, si, sj, _ptr(out), jp, bp, _stream()), "fovi_batch_to_inner")
    return out


def relu_backward_to_inner(grad, act, jp=None, bp=None, want_masked=True, want_colsum=True):
    """Fused start of a layer's backward pass.  grad / act: logical [B, I, J] tensors of the same dtype and strides (one
    of the last two contiguous).  Returns (masked gradient in grad's layout or None, [I, jp, bp] bf16 batch-innermost copy
    of the masked gradient, float32 sums over everything but the contiguous index or None), or None when the shapes need
    the separate calls (odd extents or strides)."""
    _need_cuda(grad, act)
    B, I, J = grad.shape
    jp, bp = J if jp is None else int(jp), B if bp is None else int(bp)
    sb, si, sj = grad.stride()
    if (si != 1 and sj != 1) or act.stride() != grad.stride() or act.dtype != grad.dtype or act.shape != grad.shape:
        return None
    F = I if (si == 1 and not (sj == 1 and J >= I)) else J
    masked = torch.empty_strided(grad.shape, grad.stride(), dtype=grad.dtype, device=grad.device) if want_masked else None
    out = torch.empty((I, jp, bp), dtype=torch.bfloat16, device=grad.device)
    colsum = torch.empty(F, dtype=torch.float32, device=grad.device) if want_colsum else None
    with torch.cuda.device(grad.device):
        rc = lib.fovi_relu_backward_to_inner(_ptr(grad), _ptr(act), _dt(grad.dtype), B, I, J, sb, si, sj, _ptr(masked) if masked is not None else None,
                                             _ptr(out), jp, bp, _ptr(colsum) if colsum is not None else None, _stream())
    if rc == 2:   # FOVI_ERR_UNSUPPORTED: shapes the fused kernel does not take
        return None
    check(rc, "fovi_relu_backward_to_inner")
    return masked, out, colsum


def column_sum(x):
    """x [..., C] contiguous float32/bf16 CUDA tensor -> float32 [C]: the sum over all leading dimensions."""
    _need_cuda(x)
    x = x.contiguous()
    Cc = x.shape[-1]
    out = torch.empty(Cc, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        check(lib.fovi_column_sum(_ptr(x), _dt(x.dtype), x.numel() // Cc, Cc, _ptr(out), _stream()), "fovi_column_sum")
    return out


def tap_segment_sum(prod, seg_start, seg_slot, dst):
    """dst[o, 4*v + c] += sum over the slots of tap v of prod[o, slot, c]  (prod float32 [R, S, 4] contiguous, seg_start int32 [V+1],
    seg_slot int32, dst float32 [R, >= 4*V] contiguous).  See fovi_tap_segment_sum."""
    _need_cuda(prod, seg_start, seg_slot, dst)
    assert prod.dtype == torch.float32 and prod.is_contiguous() and prod.dim() == 3 and prod.shape[2] == 4
    assert seg_start.dtype == torch.int32 and seg_slot.dtype == torch.int32 and dst.dtype == torch.float32 and dst.is_contiguous()
    V = seg_start.numel() - 1
    with torch.cuda.device(prod.device):
        check(lib.fovi_tap_segment_sum(_ptr(prod), prod.shape[0], prod.shape[1], _ptr(seg_start), _ptr(seg_slot), V, _ptr(dst), dst.shape[1],
                                       _stream()), "fovi_tap_segment_sum")
    return dst


def launch_count():
    return lib.fovi_launch_count()
