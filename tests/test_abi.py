"""CPU: the C-ABI library loads and exports every symbol the public header declares."""
import ctypes
import os
import re

from conftest import ROOT


def _declared_symbols():
    src = open(os.path.join(ROOT, "include", "fovi_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(fovi_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported():
    import __graft_entry__
    __graft_entry__.build()
    lib = ctypes.CDLL(os.path.join(ROOT, "fovi_b200", "libfovi_b200.so"))
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/fovi_b200.h but not exported"


def test_binding_covers_header():
    from fovi_b200 import _lib
    assert sorted(_lib.SIGNATURES) == _declared_symbols()


def test_status_strings_and_argument_checks_without_gpu():
    from fovi_b200._lib import lib
    assert lib.fovi_status_string(0) == b"ok"
    assert lib.fovi_status_string(3) == b"neighbour or tap table entry out of range"
    assert lib.fovi_version() == b"0.1"
    # null / nonsense arguments are rejected before any CUDA call
    assert lib.fovi_sampler_plan_create(None, 10, None) == 1
    assert lib.fovi_knnconv_plan_create(None, None, 1, 1, 1, 1, 1, 1, None) == 1
    assert lib.fovi_sampler_plan_num_points(None) == -1
    # table range validation happens on the host, before any device work
    idx = (ctypes.c_int32 * 4)(0, 1, 5, 2)       # K=2, n_out=2, n_in=3: value 5 is out of range
    tap = (ctypes.c_uint16 * 4)(0, 0, 0, 0)
    h = ctypes.c_void_p()
    assert lib.fovi_knnconv_plan_create(idx, tap, 3, 2, 2, 4, 3, 16, ctypes.byref(h)) == 3
    tap_bad = (ctypes.c_uint16 * 4)(0, 9, 0, 0)
    idx_ok = (ctypes.c_int32 * 4)(0, 1, 3, 2)
    assert lib.fovi_knnconv_plan_create(idx_ok, tap_bad, 3, 2, 2, 4, 3, 16, ctypes.byref(h)) == 3
