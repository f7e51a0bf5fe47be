"""ctypes binding of ``libfovi_b200.so`` (the C ABI declared in ``include/fovi_b200.h``).

There is no fallback: if the shared object is missing or a symbol cannot be bound, importing
this module raises.  Build it with ``python -m fovi_b200.build``.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# FOVI_B200_LIBRARY points at another build of the same ABI (e.g. a debug build); default: in-tree.
LIB_PATH = os.environ.get("FOVI_B200_LIBRARY") or os.path.join(HERE, "libfovi_b200.so")

# name -> (restype, argtypes); must list every symbol the header declares.
_P = C.c_void_p
SIGNATURES = {
    "fovi_status_string": (C.c_char_p, [C.c_int]),
    "fovi_last_cuda_error": (C.c_char_p, []),
    "fovi_version": (C.c_char_p, []),
    "fovi_sampler_plan_create": (C.c_int, [_P, C.c_int, C.POINTER(_P)]),
    "fovi_sampler_plan_destroy": (None, [_P]),
    "fovi_sampler_plan_num_points": (C.c_int, [_P]),
    "fovi_sample_forward": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int64), _P, _P,
                                      C.c_int, C.c_int, C.c_int, _P, C.c_int, C.c_int, C.c_int, _P]),
    "fovi_sampler_check": (C.c_int, [_P, _P]),
    "fovi_sample_backward": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P]),
    "fovi_knnconv_plan_create": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(_P)]),
    "fovi_knnconv_plan_destroy": (None, [_P]),
    "fovi_knnconv_cin_packed": (C.c_int, [_P]),
    "fovi_knnconv_nnz": (C.c_int64, [_P]),
    "fovi_knnconv_x_layout": (C.c_int, [_P]),
    "fovi_knnconv_tc_supported": (C.c_int, [_P]),
    "fovi_knnconv_pack_weights": (C.c_int, [_P, _P, C.c_int, _P, C.c_int, _P]),
    "fovi_knnconv_packed_weight_bytes": (C.c_int64, [_P, C.c_int]),
    "fovi_pack_points": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, _P, C.c_int, C.c_int, _P]),
    "fovi_knnconv_forward": (C.c_int, [_P, _P, _P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "fovi_knnconv_forward_f32": (C.c_int, [_P, _P, C.c_int, C.c_int, _P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "fovi_knnconv_forward_scatter_add": (C.c_int, [_P, _P, _P, _P, C.c_int, _P, C.c_int, _P]),
    "fovi_knnconv_selftest_wait_timeout": (C.c_int, [_P, _P, _P, _P, C.c_int, C.c_int, _P]),
    "fovi_knnconv_check": (C.c_int, [_P, _P]),
    "fovi_static_scratch_bytes": (C.c_int64, []),
    "fovi_knnconv_forward_bcn_static": (C.c_int, [_P, _P, C.c_int, _P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "fovi_fused_intermediate_bytes": (C.c_int64, [_P, C.c_int]),
    "fovi_sample_knnconv_fused": (C.c_int, [_P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int64), _P, _P,
                                            C.c_int, C.c_int, C.c_int, _P, _P, _P, _P, C.c_int, C.c_int, C.c_int, _P]),
    "fovi_knnconv_pack_weights_grouped": (C.c_int, [_P, _P, C.c_int, _P, C.c_int, C.c_int, _P, _P]),
    "fovi_knn_depthwise_forward": (C.c_int, [_P, _P, C.c_int, C.c_int, _P, _P, _P, C.c_int, C.c_int, C.c_int, C.c_int, _P]),
    "fovi_knn_depthwise_backward": (C.c_int, [_P, _P, C.c_int, C.c_int, _P, _P, C.c_int, C.c_int, C.c_int, _P, _P, _P]),
    "fovi_sensor_ring_layout": (C.c_longlong, [C.c_double, C.c_double, C.c_int, _P, _P]),
    "fovi_sensor_points": (C.c_int, [C.c_double, C.c_double, C.c_int, C.c_double, C.c_longlong, _P, _P, _P]),
    "fovi_sensor_pad_points": (C.c_longlong, [C.c_double, C.c_double, C.c_int, C.c_double, C.c_double, C.c_longlong, _P, _P]),
    "fovi_column_sum": (C.c_int, [_P, C.c_int, C.c_longlong, C.c_int, _P, _P]),
    "fovi_relu_backward_to_inner": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_longlong, C.c_longlong, _P, _P, C.c_int, C.c_int, _P, _P]),
    "fovi_tap_segment_sum": (C.c_int, [_P, C.c_int, C.c_longlong, _P, _P, C.c_int, _P, C.c_int, _P]),
    "fovi_batch_to_inner": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_longlong, C.c_longlong, _P, C.c_int, C.c_int, _P]),
    "fovi_knn_table_build": (C.c_int, [_P, C.c_int, C.c_int, _P, C.c_int, C.c_int, _P, _P]),
    "fovi_tap_table_build": (C.c_int, [_P, C.c_int, C.c_int, _P, C.c_int, C.c_int, _P, _P, _P, C.c_int, C.c_int, _P, _P]),
    "fovi_knnpool_plan_create": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.POINTER(_P)]),
    "fovi_knnpool_plan_destroy": (None, [_P]),
    "fovi_knnpool_set_weights": (C.c_int, [_P, _P]),
    "fovi_knn_norm_stat_groups": (C.c_int64, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "fovi_knn_norm_forward": (C.c_int, [_P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P, C.c_float, C.c_int, _P, _P,
                                        C.c_int, _P]),
    "fovi_knnpool_forward": (C.c_int, [_P, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "fovi_knnpool_backward": (C.c_int, [_P, _P, C.c_int, _P, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, _P, _P]),
    "fovi_launch_count": (C.c_int64, []),
}

if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} not found: the CUDA library has not been built (run `python -m fovi_b200.build`); "
                      "fovi_b200 has no CPU or PyTorch fallback")

lib = C.CDLL(LIB_PATH)
for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)          # AttributeError if the library lacks a declared symbol
    _fn.restype = _res
    _fn.argtypes = _args


class FoviError(RuntimeError):
    def __init__(self, status, where):
        self.status = status
        detail = lib.fovi_last_cuda_error().decode() if status in (4, 6) else ""
        super().__init__(f"{where}: {lib.fovi_status_string(status).decode()}" + (f" ({detail})" if detail else ""))


def check(status, where):
    if status != 0:
        raise FoviError(status, where)
