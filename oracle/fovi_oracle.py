"""NumPy restatement of the reference's sensor sampler and KNNConv forward.

TEST INFRASTRUCTURE ONLY (see the package docstring).  Every function cites the
reference file:line it follows.  Two pieces of the arithmetic live in PyTorch
(third party, not vendored by the reference; ``torch`` is unpinned in
fovi/requirements.txt:17, installed build 2.11.0): ``grid_sample`` and the
BLAS-backed ``einsum``/``linear``.  Their published algorithms are restated
here:

* ``F.grid_sample`` on CPU, ``align_corners=False``: a normalised coordinate
  ``g`` is unnormalised as ``fma(g + 1, size/2, -0.5)``; bilinear weights are
  the rounded products ``(1-ty)(1-tx)``, ``(1-ty)tx``, ``ty(1-tx)``, ``ty tx``
  with ``tx = x - floor(x)``; the four taps are accumulated north-west,
  north-east, south-west, south-east with fused multiply-adds; out-of-image
  taps contribute 0 (``zeros`` padding) or the coordinate is first clamped to
  ``[0, size-1]`` (``border``); ``nearest`` rounds half to even.
  With this operation order the restatement is bit-exact against torch's CPU
  kernel on the committed fixtures.

All sampler arithmetic is float32.  Fused multiply-adds are emulated as a
float64 product-sum rounded once to float32 (the product of two float32 is
exact in float64).
"""
import numpy as np

__all__ = [
    "transform_sampling_grid", "grid_sample", "retinal_sample", "sampler_footprint_bytes",
    "tap_table_from_local_rf", "knn_gather", "knnconv_forward", "knnconv_forward_closed_form",
    "knnconv_stack", "knn_pool_max", "knn_pool_avg", "knn_pool_sum",
]

f32 = np.float32


def _fma(a, b, c):
    return (a.astype(np.float64) * b.astype(np.float64) + c.astype(np.float64)).astype(f32)


def transform_sampling_grid(grid_xy, fix_rc, fix_hw, H, W):
    """Fixation-space grid -> normalised image grid (fovi/sensing/coords.py:590-642).

    grid_xy : [N,2] float32, the sampler's ``sampling_grid`` entries (x, -y) in [-1,1]
              (fovi/sensing/samplers.py:35-47, 87).
    fix_rc  : [B,2] float32 fixation centre, normalised (row, col).
    fix_hw  : [B,2] fixation size in pixels (height, width).
    Returns [B,N,2] float32 in grid_sample's (x, y) convention.

    Operation order follows coords.py:624-640 one rounding per torch op:
    ``cx = col*W``; ``g = x*(fw/2)``; ``g = g + cx``; ``g = (2*g)/W - 1``.
    """
    grid_xy = np.asarray(grid_xy, f32)
    fix_rc = np.asarray(fix_rc, f32).reshape(-1, 2)
    fix_hw = np.asarray(fix_hw, f32).reshape(-1, 2)
    cy = (fix_rc[:, 0] * f32(H)).astype(f32)[:, None]
    cx = (fix_rc[:, 1] * f32(W)).astype(f32)[:, None]
    half_h = (fix_hw[:, 0] / f32(2)).astype(f32)[:, None]
    half_w = (fix_hw[:, 1] / f32(2)).astype(f32)[:, None]
    gx = (grid_xy[None, :, 0] * half_w).astype(f32)
    gy = (grid_xy[None, :, 1] * half_h).astype(f32)
    gx = (gx + cx).astype(f32)
    gy = (gy + cy).astype(f32)
    gx = (((f32(2) * gx).astype(f32) / f32(W)).astype(f32) - f32(1)).astype(f32)
    gy = (((f32(2) * gy).astype(f32) / f32(H)).astype(f32) - f32(1)).astype(f32)
    return np.stack([gx, gy], -1)


def _unnormalize(g, size):
    return _fma((g + f32(1)).astype(f32), np.full_like(g, f32(size / 2)), np.full_like(g, f32(-0.5)))


def grid_sample(img, grid, mode="bilinear", padding="zeros"):
    """``F.grid_sample(img, grid[:,None], mode, padding, align_corners=False)[:,:,0]``
    as called at fovi/sensing/samplers.py:108 (see the module docstring for the
    restated torch algorithm).

    img  : [B,C,H,W] float32;  grid : [B,N,2] float32 normalised (x, y).
    Returns [B,C,N] float32.
    """
    img = np.asarray(img, f32)
    B, C, H, W = img.shape
    ix = _unnormalize(grid[..., 0], W)
    iy = _unnormalize(grid[..., 1], H)
    if padding == "border":
        ix = np.clip(ix, f32(0), f32(W - 1))
        iy = np.clip(iy, f32(0), f32(H - 1))
    elif padding != "zeros":
        raise ValueError(padding)
    bidx = np.arange(B)[:, None]

    def fetch(xx, yy):
        ok = (xx >= 0) & (xx < W) & (yy >= 0) & (yy < H)
        v = img[bidx, :, np.clip(yy, 0, H - 1), np.clip(xx, 0, W - 1)]  # [B,N,C]
        return np.where(ok[..., None], v, f32(0)).transpose(0, 2, 1)

    if mode == "nearest":
        return np.ascontiguousarray(fetch(np.rint(ix).astype(np.int64), np.rint(iy).astype(np.int64)))
    if mode != "bilinear":
        raise ValueError(mode)
    x0f, y0f = np.floor(ix), np.floor(iy)
    tx = (ix - x0f).astype(f32); ux = (f32(1) - tx).astype(f32)
    ty = (iy - y0f).astype(f32); uy = (f32(1) - ty).astype(f32)
    x0, y0 = x0f.astype(np.int64), y0f.astype(np.int64)
    w_nw = (uy * ux).astype(f32)[:, None]; w_ne = (uy * tx).astype(f32)[:, None]
    w_sw = (ty * ux).astype(f32)[:, None]; w_se = (ty * tx).astype(f32)[:, None]
    acc = (fetch(x0, y0) * w_nw).astype(f32)
    acc = _fma(fetch(x0 + 1, y0), np.broadcast_to(w_ne, acc.shape), acc)
    acc = _fma(fetch(x0, y0 + 1), np.broadcast_to(w_sw, acc.shape), acc)
    acc = _fma(fetch(x0 + 1, y0 + 1), np.broadcast_to(w_se, acc.shape), acc)
    return acc


def retinal_sample(img, grid_xy, fix_rc=None, fix_hw=None, mode="bilinear", padding="zeros"):
    """Sensor forward for one or many fixations per image.

    One fixation: fovi/sensing/retina.py:118-156 -> samplers.py:91-112.  Many
    fixations: the loop of fovi/sensing/policies.py:266-277 stacked on dim 1.

    fix_rc : None (centre), [B,2] or [B,F,2];  fix_hw : None (image size), [B,2] or [B,F,2].
    Returns [B,C,N] for 2-D fixations, else [B,F,C,N].
    """
    img = np.asarray(img, f32)
    B, C, H, W = img.shape
    if fix_rc is None:
        fix_rc = np.full((B, 2), 0.5, f32)
    fix_rc = np.asarray(fix_rc, f32)
    single = fix_rc.ndim == 2
    if single:
        fix_rc = fix_rc[:, None]
    F = fix_rc.shape[1]
    if fix_hw is None:
        fix_hw = np.broadcast_to(np.array([H, W], f32), (B, F, 2))
    fix_hw = np.asarray(fix_hw, f32)
    if fix_hw.ndim == 2:
        fix_hw = np.broadcast_to(fix_hw[:, None], (B, F, 2))
    outs = []
    for f in range(F):
        g = transform_sampling_grid(grid_xy, fix_rc[:, f], fix_hw[:, f], H, W)
        outs.append(grid_sample(img, g, mode, padding))
    out = np.stack(outs, 1)
    return out[:, 0] if single else out


def sampler_footprint_bytes(grid_xy, fix_rc, fix_hw, H, W, C, in_bytes, out_bytes, mode="bilinear", padding="zeros"):
    """Algorithmic bytes of one sampler pass: per image x fixation,
    ``C * (U * in_bytes + N * out_bytes)`` with U the number of distinct in-image
    source pixels under the 2x2 (bilinear) or 1x1 (nearest) footprints.
    fix_rc/fix_hw : [M,2] (one row per image x fixation).  Returns (total_bytes, mean_U).
    """
    g = transform_sampling_grid(grid_xy, fix_rc, fix_hw, H, W)
    ix = _unnormalize(g[..., 0], W); iy = _unnormalize(g[..., 1], H)
    if padding == "border":
        ix = np.clip(ix, 0, W - 1); iy = np.clip(iy, 0, H - 1)
    total_u = 0
    for m in range(g.shape[0]):
        if mode == "nearest":
            xs = [np.rint(ix[m]).astype(np.int64)]; ys = [np.rint(iy[m]).astype(np.int64)]
        else:
            x0 = np.floor(ix[m]).astype(np.int64); y0 = np.floor(iy[m]).astype(np.int64)
            xs = [x0, x0 + 1, x0, x0 + 1]; ys = [y0, y0, y0 + 1, y0 + 1]
        xx = np.concatenate(xs); yy = np.concatenate(ys)
        ok = (xx >= 0) & (xx < W) & (yy >= 0) & (yy < H)
        total_u += np.unique(yy[ok] * W + xx[ok]).size
    M, N = g.shape[0], g.shape[1]
    return C * (total_u * in_bytes + M * N * out_bytes), total_u / M


# --------------------------------------------------------------------------- KNNConv

def tap_table_from_local_rf(local_rf):
    """One-hot ``local_rf`` [Nout,K,V] (fovi/arch/knn.py:636-647) -> tap index [Nout,K]."""
    local_rf = np.asarray(local_rf)
    assert np.all(local_rf.sum(-1) == 1) and np.all((local_rf == 0) | (local_rf == 1))
    return local_rf.argmax(-1).astype(np.int32)


def knn_gather(X, knn_idx_pad):
    """Zero-pad slot at index Nin, then gather (fovi/arch/knn.py:484-503).
    X [B,Cin,Nin]; knn_idx_pad [K,Nout] with values in [0,Nin] -> [B,Cin,K,Nout]."""
    B, C, Nin = X.shape
    Xp = np.concatenate([X, np.zeros((B, C, 1), X.dtype)], 2)
    K, Nout = knn_idx_pad.shape
    return Xp[:, :, knn_idx_pad.reshape(-1)].reshape(B, C, K, Nout)


def knnconv_forward(X, knn_idx_pad, tap, V, weight, bias=None):
    """``KNNConvLayer.forward`` in the reference's own three steps
    (fovi/arch/knn.py:538-557): gather (:484-503), one-hot tap scatter as a batched
    matmul ``'ank,nkv->anv'`` (:505-526), shared linear over ``Cin*V`` (:555).

    X [B,Cin,Nin] float32; knn_idx_pad [K,Nout] int; tap [Nout,K] int (argmax of the
    one-hot local_rf); weight [Cout,Cin*V] (c-major, v-minor); bias [Cout] or None.
    Returns [B,Cout,Nout] float32.
    """
    X = np.asarray(X, f32)
    B, Cin, _ = X.shape
    K, Nout = knn_idx_pad.shape
    g = knn_gather(X, knn_idx_pad)                      # [B,Cin,K,Nout]
    rf = np.zeros((Nout, K, V), f32)
    rf[np.arange(Nout)[:, None], np.arange(K)[None, :], tap] = 1
    a = g.transpose(0, 1, 3, 2).reshape(B * Cin, Nout, K)  # '(b d) n k'
    s = np.einsum("ank,nkv->anv", a, rf, optimize=True)    # [(B Cin), Nout, V]
    feat = s.reshape(B, Cin, Nout, V).transpose(0, 2, 1, 3).reshape(B, Nout, Cin * V)
    out = feat @ np.asarray(weight, f32).T
    if bias is not None:
        out = out + np.asarray(bias, f32)
    return np.ascontiguousarray(out.transpose(0, 2, 1))


def knnconv_forward_closed_form(X, knn_idx_pad, tap, V, weight, bias=None, relu=False, dtype=np.float64):
    """Same result as :func:`knnconv_forward` written as the table-driven sum the
    three steps collapse to: ``out[b,o,n] = bias[o] + sum_k sum_c Xpad[b,c,idx[k,n]] *
    W[o, c*V + tap[n,k]]`` (pad neighbours contribute 0; colliding taps add).
    Accumulates in ``dtype`` (float64 by default) and returns float32."""
    X = np.asarray(X, dtype)
    B, Cin, Nin = X.shape
    K, Nout = knn_idx_pad.shape
    Cout = weight.shape[0]
    Wv = np.asarray(weight, dtype).reshape(Cout, Cin, V)
    out = np.zeros((B, Nout, Cout), dtype)
    Xp = np.concatenate([X, np.zeros((B, Cin, 1), dtype)], 2)
    for k in range(K):
        xk = Xp[:, :, knn_idx_pad[k]]                   # [B,Cin,Nout]
        wk = Wv[:, :, tap[:, k]]                        # [Cout,Cin,Nout]
        out += np.einsum("bcn,ocn->bno", xk, wk, optimize=True)
    if bias is not None:
        out += np.asarray(bias, dtype)
    if relu:
        out = np.maximum(out, 0)
    return np.ascontiguousarray(out.transpose(0, 2, 1)).astype(f32)


def knnconv_backward(X, knn_idx_pad, tap, V, weight, grad_out, dtype=np.float64):
    """Gradients of :func:`knnconv_forward_closed_form` (what autograd computes through the reference's
    gather / one-hot matmul / linear, fovi/arch/knn.py:538-557) for an upstream gradient ``grad_out [B,Cout,Nout]``:

        dX[b,c,m]      = sum over (n,k) with idx[k,n] == m of  sum_o grad_out[b,o,n] * W[o, c*V + tap[n,k]]
        dW[o,c*V + v]  = sum over (n,k) with tap[n,k] == v, idx[k,n] != pad of  sum_b grad_out[b,o,n] * X[b,c,idx[k,n]]
        dbias[o]       = sum_{b,n} grad_out[b,o,n]

    Returns (dX [B,Cin,Nin], dW [Cout,Cin*V], dbias [Cout]) as float32, accumulated in ``dtype``."""
    X = np.asarray(X, dtype)
    G = np.asarray(grad_out, dtype)
    B, Cin, Nin = X.shape
    K, Nout = knn_idx_pad.shape
    Cout = weight.shape[0]
    Wv = np.asarray(weight, dtype).reshape(Cout, Cin, V)
    Xp = np.concatenate([X, np.zeros((B, Cin, 1), dtype)], 2)
    dXp = np.zeros((B, Cin, Nin + 1), dtype)
    dW = np.zeros((Cout, Cin, V), dtype)
    for k in range(K):
        wk = Wv[:, :, tap[:, k]]                                          # [Cout,Cin,Nout]
        contrib = np.einsum("bon,ocn->bcn", G, wk, optimize=True)         # [B,Cin,Nout] -> scattered to idx[k]
        np.add.at(dXp, (slice(None), slice(None), knn_idx_pad[k]), contrib)
        xk = Xp[:, :, knn_idx_pad[k]]                                     # [B,Cin,Nout], zero at pad neighbours
        gw = np.einsum("bon,bcn->ocn", G, xk, optimize=True)              # [Cout,Cin,Nout] -> scattered to tap[:,k]
        np.add.at(dW, (slice(None), slice(None), tap[:, k]), gw)
    return (dXp[:, :, :Nin].astype(f32), dW.reshape(Cout, Cin * V).astype(f32), G.sum((0, 2)).astype(f32))


def knn_depthwise_forward(X, knn_idx_pad, tap, weight, bias=None, dtype=np.float64):
    """``KNNDepthwiseConvLayer.forward`` (fovi/arch/knn.py:847-872; also the depthwise half of the separable layer,
    :776-800): ``out[b, c*g + j, n] = bias[c*g + j] + sum_k Xpad[b, c, idx[k,n]] * W[c, tap[n,k], j]``.
    X [B,Cin,Nin]; weight [Cin, V, g]; returns [B, Cin*g, Nout] float32."""
    X = np.asarray(X, dtype)
    B, Cin, Nin = X.shape
    K, Nout = knn_idx_pad.shape
    W = np.asarray(weight, dtype)
    g = W.shape[2]
    Xp = np.concatenate([X, np.zeros((B, Cin, 1), dtype)], 2)
    out = np.zeros((B, Cin, g, Nout), dtype)
    for k in range(K):
        out += Xp[:, :, None, knn_idx_pad[k]] * W[:, tap[:, k], :].transpose(0, 2, 1)[None]
    out = out.reshape(B, Cin * g, Nout)
    if bias is not None:
        out = out + np.asarray(bias, dtype)[None, :, None]
    return out.astype(f32)


def knnconv_stack(X, layers, relu_between=True):
    """A chain of KNNConv layers with ReLU between them (the conv->ReLU skeleton of
    fovi/arch/knnalexnet.py:109-127 without norm/pool).  ``layers`` is a list of dicts
    with keys knn_idx_pad, tap, V, weight, bias.  Returns the list of layer outputs."""
    outs = []
    for i, L in enumerate(layers):
        X = knnconv_forward(X, L["knn_idx_pad"], L["tap"], L["V"], L["weight"], L.get("bias"))
        if relu_between and i + 1 < len(layers):
            X = np.maximum(X, 0)
        outs.append(X)
    return outs


def knn_pool_max(X, knn_idx_pad):
    """``KNNPoolingLayer.forward`` in 'max' mode (fovi/arch/knn.py:345-369): pad slot is
    NaN, replaced by -inf before the max over the K neighbours."""
    B, C, Nin = X.shape
    Xp = np.concatenate([np.asarray(X, f32), np.full((B, C, 1), -np.inf, f32)], 2)
    K, Nout = knn_idx_pad.shape
    return Xp[:, :, knn_idx_pad.reshape(-1)].reshape(B, C, K, Nout).max(2)


def _pool_gather(X, knn_idx_pad):
    B, C, Nin = X.shape
    Xp = np.concatenate([np.asarray(X, f32), np.full((B, C, 1), np.nan, f32)], 2)     # pad slot is NaN (knn.py:356)
    K, Nout = knn_idx_pad.shape
    return Xp[:, :, knn_idx_pad.reshape(-1)].reshape(B, C, K, Nout)


def knn_pool_sum(X, knn_idx_pad):
    """'sum' mode: nansum over the K neighbours (fovi/arch/knn.py:370-371), accumulated in order k = 0..K-1."""
    g = _pool_gather(X, knn_idx_pad)
    acc = np.zeros(g[:, :, 0].shape, f32)
    for k in range(g.shape[2]):
        acc = (acc + np.where(np.isnan(g[:, :, k]), f32(0), g[:, :, k])).astype(f32)
    return acc


def knn_pool_avg(X, knn_idx_pad):
    """'avg' mode: nanmean over the K neighbours (fovi/arch/knn.py:365-366) = nansum / number of non-NaN."""
    g = _pool_gather(X, knn_idx_pad)
    cnt = (~np.isnan(g)).sum(2).astype(f32)
    with np.errstate(invalid="ignore", divide="ignore"):
        return (knn_pool_sum(X, knn_idx_pad) / cnt).astype(f32)


def knn_pool_weighted(X, knn_idx_pad, weights):
    """'gaussian' pooling (fovi/arch/knn.py:372-390): weighted mean over the valid neighbours with the weights of pad / NaN
    neighbours dropped and the rest renormalised, ``sum_k x_k w_k / (sum_valid w_k + 1e-8)``.  weights [K, n_out]."""
    g = _pool_gather(np.asarray(X, np.float64), knn_idx_pad)          # [B,C,K,n_out], NaN at pad neighbours
    valid = ~np.isnan(g)
    w = np.where(valid, np.asarray(weights, np.float64)[None, None], 0.0)
    w = w / (w.sum(2, keepdims=True) + 1e-8)
    return (np.where(valid, g, 0.0) * w).sum(2).astype(f32)


def knn_pool_backward(X, knn_idx_pad, grad_out, mode, weights=None):
    """Gradient of the KNN pooling with respect to its input (autograd through the gather and nan-aware reductions of
    fovi/arch/knn.py:345-394): every output element gives its upstream gradient back to the valid neighbours it read --
    'sum' 1 each, 'avg' 1/count, 'gaussian' w_k / (sum of valid w + 1e-8), 'max' all to the first neighbour in list order
    holding the maximum.  X [B,C,n_in], grad_out [B,C,n_out] -> [B,C,n_in] float32 (float64 accumulation)."""
    X = np.asarray(X, np.float64)
    G = np.asarray(grad_out, np.float64)
    K, n_out = knn_idx_pad.shape
    n_in = X.shape[2]
    g = _pool_gather(X, knn_idx_pad)                                   # [B,C,K,n_out], NaN at pad neighbours
    valid = ~np.isnan(g)
    if mode == "max":
        first = np.argmax(np.where(valid, g, -np.inf), axis=2)         # first maximum in list order
        coeff = (np.arange(K)[None, None, :, None] == first[:, :, None, :]) & valid.any(2, keepdims=True)
        coeff = coeff.astype(np.float64)
    elif mode == "sum":
        coeff = valid.astype(np.float64)
    elif mode == "avg":
        coeff = valid / np.maximum(valid.sum(2, keepdims=True), 1)
    elif mode == "gaussian":
        w = np.where(valid, np.asarray(weights, np.float64)[None, None], 0.0)
        coeff = w / (w.sum(2, keepdims=True) + 1e-8)
    else:
        raise ValueError(mode)
    dX = np.zeros((X.shape[0], X.shape[1], n_in + 1))
    idx = np.broadcast_to(np.asarray(knn_idx_pad, np.int64)[None, None], coeff.shape)
    b, c = np.meshgrid(np.arange(X.shape[0]), np.arange(X.shape[1]), indexing="ij")
    np.add.at(dX, (b[:, :, None, None], c[:, :, None, None], idx), coeff * G[:, :, None, :])
    return dX[:, :, :n_in].astype(f32)


def knn_norm(X, mode, weight=None, bias=None, eps=1e-5, groups=1):
    """Per-sample norms of [B,C,N] activations (fovi/arch/norm.py:14-101 = torch LayerNorm / GroupNorm, biased variance):
    'channel' over C, 'coord' over N, 'layer' over (C, N), 'group' over (C/groups, N).  weight / bias broadcast as torch
    does: [C] for channel and group, [N] for coord, [C, N] for layer."""
    X = np.asarray(X, np.float64)
    B, C, N = X.shape
    if mode == "channel":
        m, v = X.mean(1, keepdims=True), X.var(1, keepdims=True)
        shape = (1, C, 1)
    elif mode == "coord":
        m, v = X.mean(2, keepdims=True), X.var(2, keepdims=True)
        shape = (1, 1, N)
    elif mode == "layer":
        m, v = X.mean((1, 2), keepdims=True), X.var((1, 2), keepdims=True)
        shape = (1, C, N)
    elif mode == "group":
        Xg = X.reshape(B, groups, (C // groups) * N)
        m = np.repeat(Xg.mean(2), C // groups, 1)[:, :, None]
        v = np.repeat(Xg.var(2), C // groups, 1)[:, :, None]
        shape = (1, C, 1)
    else:
        raise ValueError(mode)
    y = (X - m) / np.sqrt(v + eps)
    if weight is not None:
        y = y * np.asarray(weight, np.float64).reshape(shape)
    if bias is not None:
        y = y + np.asarray(bias, np.float64).reshape(shape)
    return y.astype(f32)
