"""Sensor geometry on the host: the foveated sample points and their cortical-manifold coordinates.

Host-side mirror of the reference's setup code (fovi/sensing/coords.py:10-447 and
fovi/sensing/manifold.py:32-48, 117-154, 347-374) for the ``isotropic`` sampling style, which is what
every shipped configuration and every benchmark configuration uses.  It runs once per sensor or
layer, never per batch.  The numbers it produces are inputs of the kernels (sample grid, neighbour
tables), and they must equal the reference's bit for bit, so each quantity is computed in the same
dtype and operation order, with the same library routine where the result depends on one
(``torch.linspace``/``exp``/``arange`` in float32 for the ring radii, NumPy float64 trigonometry
for the points, SciPy's trapezoid integral + linear interpolant for the manifold's z) — but
vectorised over rings and points instead of the reference's per-point Python loops.

Geometry.  Rings are evenly spaced in cortical radius ``w = log(r + a)`` between ``log a`` and
``log(fov/2 + a)``, so ``r = exp(w) - a``; each ring gets as many equally spaced angles as keeps the
arc spacing equal to the local ring spacing (isotropy).  A point at eccentricity r (degrees) and
angle theta sits on the 3-D cortical manifold at ``(rho cos theta, rho sin theta, z)`` with
``rho = M(r) sin(r) 180/pi``, ``M(r) = k/(a + r)`` and ``z = integral sqrt(M^2 - rho'^2) dr``.
"""
import ctypes as C
import math
import os

import numpy as np
import torch
from scipy.integrate import cumulative_trapezoid
from scipy.interpolate import interp1d

__all__ = ["SamplingCoords", "ring_layout", "num_sampling_coords", "find_desired_res", "auto_match_num_coords",
           "get_in_out_coords", "cortical_coords"]

_MANIFOLD_K = 10.0          # mm scale of the magnification function (fovi/sensing/manifold.py:32)
_MESH_STEP = 0.0001         # degrees, integration mesh of the manifold's z (manifold.py:44-48)


def default_builder():
    """'torch' (default): the reference's own library calls, bit-identical coordinates on the machine that recorded
    the fixtures.  'native': the library's host routines (``fovi_sensor_ring_layout`` / ``fovi_sensor_points`` /
    ``fovi_sensor_pad_points``): the same point counts, coordinates within a few float32 ulps, no torch / SciPy call
    and 10-100x faster ring-count searches.  Set with the environment variable ``FOVI_B200_GEOMETRY``."""
    b = os.environ.get("FOVI_B200_GEOMETRY", "torch")
    if b not in ("torch", "native"):
        raise ValueError("FOVI_B200_GEOMETRY must be 'torch' or 'native'")
    return b


def _native_ring_layout(fov, cmf_a, res):
    from ._lib import lib
    radius, counts = np.empty(res, np.float32), np.empty(res, np.int32)
    n = lib.fovi_sensor_ring_layout(float(fov), float(cmf_a), int(res), radius.ctypes.data_as(C.c_void_p), counts.ctypes.data_as(C.c_void_p))
    if n < 0:
        raise ValueError(f"fovi_sensor_ring_layout({fov}, {cmf_a}, {res}) failed with code {n}")
    return torch.from_numpy(radius), [int(c) for c in counts]


def _native_points(fov, cmf_a, res, max_val):
    """(cartesian [N,2], polar [N,2], cortical [N,3]) float64 tensors, (cartesian_pad [P,2], cortical_pad [P,3]) float32."""
    from ._lib import check, lib
    ptr = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
    n = lib.fovi_sensor_ring_layout(float(fov), float(cmf_a), int(res), None, None)
    cart, polar, cort = np.empty((n, 2)), np.empty((n, 2)), np.empty((n, 3))
    check(lib.fovi_sensor_points(float(fov), float(cmf_a), int(res), float(max_val), n, ptr(cart), ptr(polar), ptr(cort)), "fovi_sensor_points")
    n_pad = lib.fovi_sensor_pad_points(float(fov), float(cmf_a), int(res), float(max_val), 0.5, 0, None, None)
    if n_pad < 0:
        raise ValueError(f"fovi_sensor_pad_points failed with code {n_pad}")
    cart_pad, cort_pad = np.empty((n_pad, 2), np.float32), np.empty((n_pad, 3), np.float32)
    lib.fovi_sensor_pad_points(float(fov), float(cmf_a), int(res), float(max_val), 0.5, n_pad, ptr(cart_pad), ptr(cort_pad))
    return [torch.from_numpy(a) for a in (cart, polar, cort, cart_pad, cort_pad)]


def ring_layout(fov, cmf_a, res, builder=None):
    """Ring radii (float32 tensor [res], normalised so that fov/2 -> 1) and angles per ring (list of int).
    Follows fovi/sensing/coords.py:322-370: float32 ``linspace``/``exp``; a ring's angle count is the
    length of ``arange(0, 2*pi*r, mean ring spacing)``, i.e. ``ceil`` of the ratio taken in double."""
    res = int(res)
    if (builder or default_builder()) == "native":
        return _native_ring_layout(fov, cmf_a, res)
    w_lo, w_hi = np.log(cmf_a), np.log(fov / 2 + cmf_a)
    dw = (w_hi - w_lo) / (res - 1)
    r = torch.exp(torch.linspace(w_lo, w_hi + dw, steps=res + 1)) - cmf_a      # one extra ring for the last spacing
    spacing = ((r[1:-1] - r[:-2]) + (r[2:] - r[1:-1])) / 2
    circumference = 2 * torch.pi * r[1:-1]
    counts = [1] + [int(math.ceil(float(c) / float(s))) for c, s in zip(circumference, spacing)]
    return 1 * (r[:-1] / (fov / 2)), counts


def num_sampling_coords(fov, cmf_a, res, style="isotropic", device="cpu"):
    """Number of sample points for `res` rings (fovi/sensing/coords.py:374-390, 567-586)."""
    _check_style(style)
    return 1 if int(res) <= 1 else int(sum(ring_layout(fov, cmf_a, res)[1]))


def find_desired_res(fov, cmf_a, n_points_desired, style="isotropic", device="cpu", bounds=(1, 1000), force_less_than=False, quiet=True):
    """Ring count whose point count is closest to `n_points_desired` (binary search, the count is
    monotonic), then stepped down until it does not exceed the target (`force_less_than`) or up until
    it reaches it.  Same outcome as fovi/sensing/coords.py:394-447.  Returns (res, n_points)."""
    count = lambda r: num_sampling_coords(fov, cmf_a, r, style)  # noqa: E731
    lo, hi = bounds
    best, best_gap = None, float("inf")
    while lo <= hi:
        mid = (lo + hi) // 2
        n = count(mid)
        if abs(n - n_points_desired) < best_gap:
            best, best_gap = mid, abs(n - n_points_desired)
        if n < n_points_desired:
            lo = mid + 1
        else:
            hi = mid - 1
    n = count(best)
    step = -1 if force_less_than else 1
    while (n > n_points_desired) if force_less_than else (n < n_points_desired):
        best += step
        n = count(best)
    return best, n


def auto_match_num_coords(fov, cmf_a, cart_res, style, auto_match_cart_resources, device="cpu", force_less_than=True, quiet=True):
    """(ring count, cartesian resolution) for a sensor matched to a `cart_res`^2 grid
    (fovi/sensing/coords.py:646-670)."""
    _check_style(style)
    if auto_match_cart_resources != 0:
        return find_desired_res(fov, cmf_a, cart_res ** 2, style, force_less_than=force_less_than)[0], cart_res
    return cart_res, cart_res


def _check_style(style):
    if style != "isotropic":
        raise NotImplementedError(f"sampling style {style!r}: only 'isotropic' (the style of all shipped configurations) is built")


class _Manifold:
    """z(r) of the cortical manifold, tabulated once per (a, fov) (fovi/sensing/manifold.py:32-48, 93-126)."""
    _cache = {}

    def __new__(cls, cmf_a, fov):
        key = (float(cmf_a), float(fov))
        if key not in cls._cache:
            self = super().__new__(cls)
            self.cmf_a = cmf_a
            mesh = np.arange(0, 2 * fov, _MESH_STEP)                      # well past fov/2: pad points lie outside
            m = _MANIFOLD_K / (cmf_a + mesh)
            dm = -_MANIFOLD_K * ((cmf_a + mesh) ** (-2))
            drho = dm * np.sin(np.deg2rad(mesh)) * (180 / np.pi) + m * np.cos(np.deg2rad(mesh))
            integrand = (m ** 2 - drho ** 2) ** 0.5
            self.z = interp1d(mesh, cumulative_trapezoid(integrand, x=mesh, initial=0), kind="linear")
            cls._cache[key] = self
        return cls._cache[key]


def cortical_coords(cartesian, cmf_a, fov):
    """Visual cartesian points (normalised, numpy [n,2], float64 or float32) -> cortical cartesian
    [n,3] float64.  Arithmetic stays in the input's dtype except z, as in the reference's per-point
    path (fovi/sensing/manifold.py:139-170, 202-211, 347-374).  float64 input (the sample points) is
    vectorised.  float32 input (the few hundred pad points) is evaluated point by point on NumPy
    scalars: NumPy's float32 scalar and array code paths (power, sin/cos) can differ in the last bit,
    and these values feed a nearest-neighbour ranking."""
    man = _Manifold(cmf_a, fov)
    deg = cartesian * (fov / 2)
    if deg.dtype == np.float64:
        x, y = deg[:, 0], deg[:, 1]
        r = np.sqrt(x ** 2 + y ** 2)
        theta = np.arctan2(y, x)
        rho = _MANIFOLD_K / (cmf_a + r) * np.sin(np.deg2rad(r)) * (180 / np.pi)
        return np.stack([rho * np.cos(theta), rho * np.sin(theta), np.asarray(man.z(r), np.float64)], 1)
    out = np.empty((deg.shape[0], 3), np.float64)
    for i, (x, y) in enumerate(deg):
        r = np.sqrt(x ** 2 + y ** 2)
        theta = np.arctan2(y, x)
        rho = _MANIFOLD_K / (cmf_a + r) * np.sin(np.deg2rad(r)) * (180 / np.pi)
        out[i] = (rho * np.cos(theta), rho * np.sin(theta), man.z(r))
    return out


class SamplingCoords:
    """The coordinate systems of one set of foveated sample points; mirror of the reference class
    (fovi/sensing/coords.py:10-201) for ``style='isotropic'``.

    Attributes (torch tensors of `dtype` on `device`): ``cartesian`` [N,2] in [-1,1] (x, y), ``polar`` [N,2]
    (radius, angle), ``cortical`` [N,3], ``cartesian_rowcol`` [N,2] (-y, x), the pad ring(s) outside the
    field of view ``cartesian_pad_coords`` / ``cortical_pad_coords``, and ``shape``.
    """

    def __init__(self, fov, cmf_a, res, device="cpu", style="isotropic", dtype=torch.float, max_val=1, builder=None):
        _check_style(style)
        self.fov, self.cmf_a, self.resolution = fov, cmf_a, res
        self.device, self.style, self.dtype, self.max_val = device, style, dtype, max_val
        self.builder = builder or default_builder()
        self.plotting = None      # the reference's plotting coordinates are not part of the hot path
        if res == 1:
            z2, z3 = torch.zeros(1, 2, dtype=dtype), torch.zeros(1, 3, dtype=dtype)
            self.cartesian, self.polar, self.cortical = z2, z2.clone(), z3
        elif self.builder == "native":
            cart64, polar64, cort64, cart_pad, cort_pad = _native_points(fov, cmf_a, res, float(max_val))
            self.cartesian_rowcol = torch.stack([-cart64[:, 1], cart64[:, 0]], 1)
            self.cartesian_pad_coords, self.cortical_pad_coords = cart_pad.to(dtype), cort_pad.to(dtype)
            self.cartesian, self.polar, self.cortical = cart64, polar64, cort64
        else:
            radius, counts = ring_layout(fov, cmf_a, res, builder="torch")
            radius = radius * max_val
            ring = torch.repeat_interleave(radius.double(), torch.tensor(counts))
            angle = torch.from_numpy(np.concatenate([np.linspace(0, 2 * np.pi, n, endpoint=False) for n in counts]))
            cart64 = torch.stack([ring * torch.cos(angle), ring * torch.sin(angle)], 1)      # float64 until the end
            polar64 = torch.stack([ring, angle], 1)
            self.cartesian_rowcol = torch.stack([-cart64[:, 1], cart64[:, 0]], 1)
            self.cartesian_pad_coords = self._pad_ring_points(polar64[:, 0]).to(dtype)
            self.cortical = torch.from_numpy(cortical_coords(cart64.numpy(), cmf_a, fov))
            self.cortical_pad_coords = torch.from_numpy(cortical_coords(self.cartesian_pad_coords.numpy(), cmf_a, fov)).to(dtype)
            self.cartesian, self.polar = cart64, polar64
        self.cartesian = self.cartesian.to(dtype)
        self.cortical = self.cortical.to(dtype)
        self.polar = self.polar.to(dtype)
        self.shape = self.cartesian.shape
        if str(device) != "cpu":
            self.to(device)

    @staticmethod
    def _pad_ring_points(radii, padding_distance=0.5):
        """Rings continuing outward past the field of view at the last ring spacing, sampled at that same
        spacing in angle: what neighbourhoods at the edge reach into (fovi/sensing/coords.py:68-87).
        float32 arithmetic on float32 ``arange`` values, as there."""
        rr = torch.sort(torch.unique(radii)).values
        gap = rr[-1] - rr[-2]
        first = rr[-1] + gap
        ring_r = torch.arange(first, first + padding_distance, gap).numpy()
        ang = torch.arange(0, 2 * np.pi, gap).numpy()
        pts = [np.stack([r * np.cos(ang), r * np.sin(ang)], 1) for r in ring_r]
        return torch.from_numpy(np.concatenate(pts, 0).astype(np.float32))

    def get_strided_coords(self, stride, auto_match_cart_resources=0, in_cart_res=None, force_less_than=True, max_val=1):
        """Coordinates of the next, `stride`-times coarser layer (fovi/sensing/coords.py:89-131).
        Returns (coords, ring count, cartesian resolution or None)."""
        out_cart_res = None
        if auto_match_cart_resources > 0 and in_cart_res is not None:
            out_cart_res = in_cart_res // stride
            rings, _ = find_desired_res(self.fov, self.cmf_a, out_cart_res ** 2, self.style, force_less_than=force_less_than)
        else:
            rings = self.resolution // stride
        if rings < 1:
            raise ValueError(f"stride {stride} leaves fewer than one ring ({rings})")
        return SamplingCoords(self.fov, self.cmf_a, rings, self.device, self.style, self.dtype, max_val=max_val, builder=self.builder), rings, out_cart_res

    def to(self, device=None, dtype=None):
        self.dtype = self.dtype if dtype is None else dtype
        self.device = self.device if device is None else device
        for name in ("cartesian", "cortical", "polar", "cartesian_pad_coords", "cortical_pad_coords", "cartesian_rowcol"):
            if getattr(self, name, None) is not None:
                setattr(self, name, getattr(self, name).to(device=self.device, dtype=self.dtype))
        return self

    def clone(self, **overrides):
        args = dict(fov=self.fov, cmf_a=self.cmf_a, res=self.resolution, device=self.device, style=self.style, dtype=self.dtype, max_val=self.max_val,
                    builder=self.builder)
        if "resolution" in overrides:
            overrides["res"] = overrides.pop("resolution")
        args.update({k: v for k, v in overrides.items() if v is not None})
        return SamplingCoords(**args)

    def get_scatter_sizes(self):
        """Marker sizes growing linearly with eccentricity (fovi/sensing/coords.py:153-167)."""
        return self.polar[:, 0] * self.fov / self.resolution

    def __len__(self):
        return self.cartesian.shape[0]

    def __repr__(self):
        return f"SamplingCoords(length={len(self)}, fov={self.fov}, cmf_a={self.cmf_a}, resolution={self.resolution}, style={self.style})"


def get_in_out_coords(in_res, fov, cmf_a, stride, style="isotropic", auto_match_cart_resources=1, in_cart_res=None, device="cpu",
                      in_coords=None, force_out_match_less_than=True, max_out_coord_val=1):
    """Input and output point sets of one KNN layer (fovi/arch/knn.py:959-1003).  With
    ``max_out_coord_val='auto'`` the output points are shrunk so that their outermost ring falls midway
    between the two outermost rings of the unshrunk set (used by the patch embeddings).
    Returns (in_coords, out_coords, out_cart_res)."""
    if in_coords is None:
        if auto_match_cart_resources:
            in_res, in_cart_res = auto_match_num_coords(fov, cmf_a, in_cart_res, style, auto_match_cart_resources, device)
        in_coords = SamplingCoords(fov, cmf_a, in_res, device=device, style=style)
    auto = isinstance(max_out_coord_val, str) and max_out_coord_val == "auto"
    kw = dict(auto_match_cart_resources=auto_match_cart_resources, in_cart_res=in_cart_res, force_less_than=force_out_match_less_than)
    out_coords, _, out_cart_res = in_coords.get_strided_coords(stride, max_val=1 if auto else max_out_coord_val, **kw)
    if auto:
        rings = torch.unique(out_coords.polar[:, 0])
        out_coords, _, out_cart_res = in_coords.get_strided_coords(stride, max_val=(rings[-1] + rings[-2]) / 2, **kw)
    return in_coords, out_coords, out_cart_res
