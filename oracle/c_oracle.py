"""ctypes wrapper of the oracle's C restatement (``oracle/fovi_oracle.c``).  TEST INFRASTRUCTURE ONLY."""
import ctypes as C
import os

import numpy as np

from . import build_c

_lib = None


def load():
    global _lib
    if _lib is None:
        _lib = C.CDLL(build_c.build())
        _lib.fovi_oracle_sample.restype = None
        _lib.fovi_oracle_knnconv.restype = None
    return _lib


def _p(a):
    return a.ctypes.data_as(C.c_void_p)


def threads():
    """Worker threads the C functions use (FOVI_ORACLE_THREADS, default: all online cores)."""
    lib = load()
    lib.fovi_oracle_threads.restype = C.c_int
    return int(lib.fovi_oracle_threads())


def retinal_sample(img, grid_xy, fix_rc, fix_hw, mode="bilinear", padding="zeros"):
    """img [B,C,H,W], grid_xy [N,2], fix_rc/fix_hw [B,F,2] -> [B,F,C,N] float32."""
    lib = load()
    img = np.ascontiguousarray(img, np.float32); grid_xy = np.ascontiguousarray(grid_xy, np.float32)
    fix_rc = np.ascontiguousarray(fix_rc, np.float32); fix_hw = np.ascontiguousarray(fix_hw, np.float32)
    B, Cc, H, W = img.shape
    F, N = fix_rc.shape[1], grid_xy.shape[0]
    out = np.empty((B, F, Cc, N), np.float32)
    lib.fovi_oracle_sample(_p(img), B, Cc, H, W, _p(grid_xy), N, _p(fix_rc), _p(fix_hw), F, 1 if mode == "bilinear" else 0,
                           1 if padding == "border" else 0, _p(out))
    return out


def knnconv_forward_closed_form(X, knn_idx_pad, tap, V, weight, bias=None, relu=False):
    """X [B,Cin,Nin], knn_idx_pad [K,Nout], tap [Nout,K], weight [Cout,Cin*V] -> [B,Cout,Nout] float32."""
    lib = load()
    X = np.ascontiguousarray(X, np.float32); idx = np.ascontiguousarray(knn_idx_pad, np.int32)
    tap = np.ascontiguousarray(tap, np.int64); weight = np.ascontiguousarray(weight, np.float32)
    B, Cin, Nin = X.shape
    K, Nout = idx.shape
    Cout = weight.shape[0]
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    Y = np.empty((B, Cout, Nout), np.float32)
    lib.fovi_oracle_knnconv(_p(X), B, Cin, Nin, _p(idx), _p(tap), K, Nout, int(V), _p(weight), None if b is None else _p(b), Cout, int(relu), _p(Y))
    return Y
