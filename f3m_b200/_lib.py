"""ctypes binding of libf3m.so (the C ABI declared in include/f3m.h).

There is no fallback: if the shared library is missing or cannot be loaded, importing the
engine raises, and every call on a machine without a CUDA device returns an error status that
is raised as F3MError.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libf3m.so")

MATH_FASTMATH = 0
MATH_IEEE = 1
FLAG_NEAR_MOMENTS = 1
FLAG_NEAR_TENSOR_CORES = 2

# array ids of f3m_plan_copy_array
ARR_SORTED_INDEX, ARR_BOX_OFFSETS, ARR_BOX_CENTERS = 0, 1, 2
ARR_FAR_PTR, ARR_FAR_IDX, ARR_SMALL_PTR, ARR_SMALL_IDX, ARR_KEEP_PTR, ARR_KEEP_IDX, ARR_BOX_CODES = 3, 4, 5, 6, 7, 8, 9


class F3MError(RuntimeError):
    def __init__(self, status: int, where: str, message: str):
        super().__init__(f"{where}: status {status} ({message})")
        self.status = status


class Params(C.Structure):
    _fields_ = [("ls", C.c_float), ("min_points", C.c_float), ("nr_interpolation", C.c_int32),
                ("var_compression", C.c_int32), ("eff_var_limit", C.c_float), ("small_field_points", C.c_int32),
                ("math_mode", C.c_int32), ("flags", C.c_int32)]


class LevelInfo(C.Structure):
    _fields_ = [("level", C.c_int32), ("boxes_x", C.c_int32), ("boxes_y", C.c_int32), ("max_count_x", C.c_int32),
                ("max_count_y", C.c_int32), ("n_far", C.c_int64), ("n_small", C.c_int64), ("n_keep", C.c_int64),
                ("edge", C.c_float), ("nodes_per_dim", C.c_int32)]


class PlanStats(C.Structure):
    _fields_ = [("levels", C.c_int32), ("shared_tree", C.c_int32), ("direct_pairs", C.c_int64),
                ("node_pairs", C.c_int64), ("far_box_pairs", C.c_int64), ("near_box_pairs", C.c_int64),
                ("edge0", C.c_float), ("build_ms", C.c_float)]


_P = C.c_void_p
_I64, _I32, _F32, _F64 = C.c_int64, C.c_int32, C.c_float, C.c_double

# name -> (restype, argtypes); every symbol declared in include/f3m.h
SIGNATURES = {
    "f3m_version": (C.c_int, []),
    "f3m_release_cached_memory": (C.c_int, []),
    "f3m_status_string": (C.c_char_p, [C.c_int]),
    "f3m_last_error": (C.c_char_p, []),
    "f3m_kmvm_f32": (C.c_int, [_P, _I64, _P, _I64, _P, _I32, _I32, C.POINTER(Params), _P, _P]),
    "f3m_workspace_bytes": (C.c_size_t, [_I64, _I64, _I32, _I32, C.POINTER(Params)]),
    "f3m_kmvm_ws_f32": (C.c_int, [_P, _I64, _P, _I64, _P, _I32, _I32, C.POINTER(Params), _P, _P, C.c_size_t, _P]),
    "f3m_last_workspace_peak": (C.c_size_t, []),
    "f3m_kmvm_host_f32": (C.c_int, [_P, _I64, _P, _I64, _P, _I32, _I32, C.POINTER(Params), _P]),
    "f3m_plan_create": (C.c_int, [C.POINTER(_P), _P, _I64, _P, _I64, _I32, C.POINTER(Params), _P]),
    "f3m_plan_apply": (C.c_int, [_P, _P, _I32, _P, _P]),
    "f3m_plan_apply_range": (C.c_int, [_P, _P, _I32, _P, _I64, _I64, _P]),
    "f3m_plan_moments_size": (C.c_int, [_P, _I32, C.POINTER(_I64)]),
    "f3m_plan_moments_range": (C.c_int, [_P, _P, _I32, _I64, _I64, _P, _P]),
    "f3m_plan_apply_range_moments": (C.c_int, [_P, _P, _I32, _P, _I64, _I64, _P, _P]),
    "f3m_sort_depth": (C.c_int, [_I64, _I32, _F32]),
    "f3m_record_words": (C.c_int, [_I32]),
    "f3m_bounding_box_f32": (C.c_int, [_P, _I64, _I32, C.POINTER(_F32), C.POINTER(_F32), _P]),
    "f3m_sort_shard_f32": (C.c_int, [_P, _I64, _I64, _I32, C.POINTER(_F32), _F32, _I32, _I32, _P, _P, _P]),
    "f3m_plan_create_from_cell_counts": (C.c_int, [C.POINTER(_P), _P, _I32, _I32, C.POINTER(_F32), _F32, _I32, C.POINTER(Params), _P]),
    "f3m_plan_attach_runs": (C.c_int, [_P, _P, _I64, _P]),
    "f3m_plan_partition_rows": (C.c_int, [_P, _I32, _I32, C.POINTER(_I64), _P]),
    "f3m_plan_shard_begin": (C.c_int, [_P, _P, _I32, _I64, _I64, _I64, _I64, _P, _P]),
    "f3m_plan_shard_near": (C.c_int, [_P, _P, _P]),
    "f3m_plan_shard_far": (C.c_int, [_P, _P, _P, _P]),
    "f3m_plan_shard_end": (C.c_int, [_P]),
    "f3m_plan_rows_to_input_order": (C.c_int, [_P, _P, _I32, _I64, _I64, _P, _P]),
    "f3m_plan_gathered_rows_to_input_order": (C.c_int, [_P, _P, _I32, C.POINTER(_I64), _I32, _I64, _I64, _I64, _P, _P]),
    "f3m_plan_count_rows_by_owner": (C.c_int, [_P, _I64, _I64, C.POINTER(_I64), _I32, C.POINTER(_I64), _P]),
    "f3m_plan_pack_rows_by_owner": (C.c_int, [_P, _P, _I32, _I64, _I64, C.POINTER(_I64), _I32, C.POINTER(_I64), _P, _P]),
    "f3m_plan_place_rows": (C.c_int, [_P, _P, _I64, _I32, _I64, _I64, _P, _P]),
    "f3m_plan_destroy": (C.c_int, [_P]),
    "f3m_plan_get_stats": (C.c_int, [_P, C.POINTER(PlanStats)]),
    "f3m_plan_get_level": (C.c_int, [_P, _I32, C.POINTER(LevelInfo)]),
    "f3m_plan_copy_array": (C.c_int, [_P, _I32, _I32, _I32, _P, C.c_size_t]),
    "f3m_rbf_dense_f32": (C.c_int, [_P, _I64, _P, _I64, _P, _I32, _I32, _F32, _P, _P]),
    "f3m_rbf_dense_f64": (C.c_int, [_P, _I64, _P, _I64, _P, _I32, _I32, _F64, _P, _P]),
    "f3m_rbf_dense_grad_f32": (C.c_int, [_P, _I64, _P, _I64, _P, _I32, _I32, _F32, _P, _P]),
    "f3m_rbf_dense_f32_static": (C.c_int, [_P, _I64, _P, _I64, _P, _I32, _I32, _F32, _P, _P]),
    "f3m_measure_peaks": (C.c_int, [C.POINTER(_F64), C.POINTER(_F64), _P]),
    "f3m_plan_last_timings": (C.c_int, [_P, C.POINTER(_F32)]),
    "f3m_plan_last_direct_launches": (C.c_int, [_P]),
    "f3m_plan_last_direct_variants": (C.c_int, [_P, C.POINTER(_I32)]),
    "f3m_launch_count": (C.c_longlong, []),
}

_lib = None


def lib():
    """The loaded library; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'` "
                              "or `make -C f3m_b200/csrc`.  There is no fallback path.")
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def check(status: int, where: str):
    if status != 0:
        L = lib()
        raise F3MError(status, where, (L.f3m_last_error() or b"").decode() or L.f3m_status_string(status).decode())
