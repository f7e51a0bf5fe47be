"""Per-layer tables of a KNN layer, built on the host once per layer: the K nearest input points of
every output point on the cortical manifold, and for each (output point, neighbour) the tap of the
filter's reference frame it is assigned to.

Mirror of fovi/arch/knn.py:23-57, 101-152 (neighbour search) and :559-647 (reference frame,
``local_rf``).  The ranking is ill-conditioned — rings are symmetric, so the K-th and (K+1)-th
neighbours often tie exactly — which makes the table a function of the exact float32 distance
values.  It is therefore produced by the same PyTorch CPU calls the reference makes (``torch.cdist``
in its default mode, which switches to a matrix-multiply formulation above 25 rows, then
``torch.topk``/``argmin``), and the fixtures recorded from the reference are reproduced bit for bit
on the machine that recorded them.  The reference materialises ``local_rf`` as a one-hot float tensor
``[n_out, K, V]``; here the same information is the ``uint16 [n_out, K]`` tap index.

Two builders:

* ``'torch'`` (default) — the reference's own library calls, as described above: tables equal to the reference's on
  the same machine, which is what loading a checkpoint trained on the reference needs.
* ``'native'`` — the library's host routines (``fovi_knn_table_build`` / ``fovi_tap_table_build``): double-precision
  distances from the float32 coordinates, ties to the lower index; the same tables on every machine and 10-100x
  faster.  Differs from ``'torch'`` only where the reference's float32 rounding decides a (near) tie.

The default can be changed with the environment variable ``FOVI_B200_TABLES`` (``torch`` | ``native``).
"""
import ctypes as C
import os

import numpy as np
import torch

__all__ = ["knn_table", "reference_frame", "tap_table", "pad_token_table", "default_builder"]


def default_builder():
    b = os.environ.get("FOVI_B200_TABLES", "torch")
    if b not in ("torch", "native"):
        raise ValueError("FOVI_B200_TABLES must be 'torch' or 'native'")
    return b


def _f32(t):
    return np.ascontiguousarray(t.detach().cpu().numpy(), dtype=np.float32)


def _native_knn(pts, targets, k):
    from ._lib import check, lib
    p, t = _f32(pts), _f32(targets)
    n_out = t.shape[0]
    idx = np.empty((k, n_out), np.int32)
    dist = np.empty((k, n_out), np.float32)
    check(lib.fovi_knn_table_build(p.ctypes.data_as(C.c_void_p), p.shape[0], p.shape[1], t.ctypes.data_as(C.c_void_p), n_out, k,
                                   idx.ctypes.data_as(C.c_void_p), dist.ctypes.data_as(C.c_void_p)), "fovi_knn_table_build")
    return torch.from_numpy(idx.astype(np.int64)), torch.from_numpy(dist)


def knn_table(in_coords, out_coords, k, sample_cortex=True, batch_size=None, builder=None):
    """K nearest input points (pad ring included) of each output point.

    Returns (indices int64 [K, n_out], distances float32 [K, n_out], sample points [n_in+n_pad, d],
    their visual-field cartesian coordinates [n_in+n_pad, 2]).  Indices >= n_in address the pad ring.
    Distances are Euclidean in cortical space (`sample_cortex=True`) or in the visual field (False);
    geodesic ranking is not built (it needs a mesh library the reference treats as optional)."""
    if sample_cortex == "geodesic":
        raise NotImplementedError("geodesic neighbour ranking is not built; use sample_cortex=True (Euclidean on the manifold)")
    cart = torch.cat([in_coords.cartesian, in_coords.cartesian_pad_coords], 0).cpu()
    if sample_cortex:
        pts = torch.cat([in_coords.cortical, in_coords.cortical_pad_coords], 0).cpu()
        targets = out_coords.cortical.clone().cpu()
    else:
        pts, targets = cart, out_coords.cartesian.cpu()
    n_out = targets.shape[0]
    k = int(min(int(k), in_coords.shape[0]))
    if (builder or default_builder()) == "native":
        idx, dist = _native_knn(pts, targets, k)
        return idx, dist, pts, cart
    if batch_size is None:
        # keep a distance block under ~5e8 entries (the reference's default chunking)
        batch_size = int(np.minimum(n_out / np.maximum(0.0001, pts.shape[0] * n_out / 500000000), n_out))
    batch_size = max(1, min(int(batch_size), n_out))
    idx = torch.zeros((k, n_out), dtype=torch.long)
    dist = torch.zeros((k, n_out), dtype=torch.float32)
    for lo in range(0, n_out, batch_size):
        hi = min(lo + batch_size, n_out)
        d, i = torch.topk(torch.cdist(pts, targets[lo:hi]), k, dim=0, largest=False)
        idx[:, lo:hi], dist[:, lo:hi] = i, d
    return idx, dist, pts, cart


def pad_token_table(knn_indices, n_in):
    """Indices with every pad-ring neighbour replaced by the single pad token n_in (knn.py:451-453)."""
    out = knn_indices.clone()
    out[knn_indices >= n_in] = n_in
    return out


def reference_frame(k, ref_frame_side_length=None, arch_flag="", dtype=torch.float32):
    """The filter's tap grid: side x side nodes on [-1,1]^2, x-major (knn.py:559-597).
    side = `ref_frame_side_length`, else ceil(sqrt(k)) (doubled by the 'doubleres' flag)."""
    if ref_frame_side_length is not None:
        if len(arch_flag):
            raise ValueError("ref_frame_side_length cannot be combined with an arch_flag")
        side = int(ref_frame_side_length)
    else:
        side = int(torch.ceil(torch.sqrt(torch.tensor(float(k)))).long())
        if "doubleres" in arch_flag:
            side *= 2
    if "fovref" in arch_flag or "circref" in arch_flag:
        raise NotImplementedError("only the square reference frame is built")
    axis = torch.linspace(-1, 1, side)
    gx, gy = torch.meshgrid(axis, axis, indexing="ij")
    return torch.stack([gx, gy], -1).reshape(-1, 2).to(dtype), side


def _native_taps(knn_indices, pts, cart, out_coords, side, sample_cortex):
    from ._lib import check, lib
    idx = np.ascontiguousarray(knn_indices.numpy().astype(np.int32))
    K, n_out = idx.shape
    p = _f32(pts)
    pc = _f32(cart)
    op = _f32(out_coords.cortical if sample_cortex else out_coords.cartesian)
    oc = _f32(out_coords.cartesian)
    tap = np.empty((n_out, K), np.uint16)
    nb = np.empty((K, n_out, 2), np.float32)
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
    check(lib.fovi_tap_table_build(ptr(idx), K, n_out, ptr(p), p.shape[0], p.shape[1], ptr(pc), ptr(op), ptr(oc), int(side),
                                   1 if sample_cortex else 0, ptr(tap), ptr(nb)), "fovi_tap_table_build")
    return torch.from_numpy(tap.astype(np.int64)), torch.from_numpy(nb)


def tap_table(knn_indices, pts, cart, out_coords, ref_coords, sample_cortex=True, builder=None):
    """Tap index [n_out, K] (int64) of every neighbour: the neighbour's offset from the output point is
    expressed in a polar frame (cortical distance, visual-field direction), the neighbourhood is min-max
    normalised to [-1,1]^2 and each neighbour takes the nearest node of the reference frame
    (knn.py:599-647).  Also returns the normalised neighbour coordinates [K, n_out, 2]."""
    if (builder or default_builder()) == "native":
        side = int(round(ref_coords.shape[0] ** 0.5))
        if side * side != ref_coords.shape[0]:
            raise ValueError("the native tap builder needs a square reference frame")
        return _native_taps(knn_indices, pts, cart, out_coords, side, bool(sample_cortex))
    nb = pts[knn_indices]                                            # [K, n_out, d]
    if sample_cortex:
        oc, ov = out_coords.cortical.cpu(), out_coords.cartesian.cpu()
        nbv = cart[knn_indices]
        direction = torch.arctan2(nbv[:, :, 1] - ov[:, 1], nbv[:, :, 0] - ov[:, 0])
        radius = torch.stack([torch.cdist(oc[i].unsqueeze(0), nb[:, i]).squeeze(0) for i in range(nb.shape[1])], dim=1)
        nb = torch.stack([radius * torch.cos(direction), radius * torch.sin(direction)], dim=2)
    lo = nb.min(dim=0, keepdim=True)[0]
    hi = nb.max(dim=0, keepdim=True)[0]
    nb = 2 * (nb - lo) / (hi - lo + 1e-6) - 1
    tap = torch.argmin(torch.cdist(nb, ref_coords.cpu()), dim=2)     # [K, n_out]
    return tap.t().contiguous(), nb
