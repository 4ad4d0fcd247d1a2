"""ctypes binding of ``libblkattn.so`` (the C ABI declared in ``include/blkattn.h``).

The library is the product; there is no fallback.  If the shared object is
missing or does not load, importing this module raises and every operator of
the package fails with it.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libblkattn.so")

BLK_OK = 0
BLK_ERR_INVALID, BLK_ERR_CUDA, BLK_ERR_UNSUPPORTED, BLK_ERR_UNALIGNED, BLK_ERR_NOMEM, BLK_ERR_TIMEOUT = (
    -1, -2, -3, -4, -5, -6)
BLK_F16, BLK_BF16, BLK_F32 = 0, 1, 2
BLK_EPI_SCORES, BLK_EPI_SOFTMAX = 0, 1

_i64p = C.POINTER(C.c_int64)
_i32p = C.POINTER(C.c_int32)
_f64p = C.POINTER(C.c_double)
_vp = C.c_void_p

# name -> (restype, argtypes); one entry per function declared in include/blkattn.h
SIGNATURES = {
    "blk_last_error": (C.c_char_p, []),
    "blk_version": (C.c_char_p, []),
    "blk_offsets_from_lists": (C.c_int, [_i64p, _i64p, _i64p, C.c_int64, _i64p, _i64p, _i64p]),
    "blk_softmax_offsets": (C.c_int, [_i64p, _i64p, C.c_int64, _i64p]),
    "blk_lists_from_offsets": (C.c_int, [_i64p, _i64p, _i64p, C.c_int64, _i64p, _i64p, _i64p]),
    "blk_segment_cost": (C.c_int, [_i64p, _i64p, _i64p, C.c_int64, C.c_int64, C.c_int, C.c_int, C.c_double,
                                   C.c_double, _f64p]),
    "blk_partition_contiguous": (C.c_int, [_f64p, C.c_int64, C.c_int, _i64p]),
    "blk_partition_lpt": (C.c_int, [_f64p, C.c_int64, C.c_int, _i32p]),
    "blk_gemm_plan_create": (C.c_int, [C.POINTER(_vp), _i64p, _i64p, _i64p, _i64p, _i64p, _i64p, C.c_int64,
                                       C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "blk_gemm_run": (C.c_int, [_vp, _vp, _vp, _vp, C.c_float, _vp]),
    "blk_gemm_run_strided": (C.c_int, [_vp, _vp, C.c_int64, C.c_int64, _vp, C.c_int64, C.c_int64, _vp, C.c_float, _vp]),
    "blk_attention_plan_create": (C.c_int, [C.POINTER(_vp), _i64p, _i64p, C.c_int64, C.c_int64, C.c_int, C.c_int]),
    "blk_attention_plan_create_dim": (C.c_int, [C.POINTER(_vp), _i64p, _i64p, C.c_int64, C.c_int64, C.c_int64, C.c_int,
                                                C.c_int]),
    "blk_attention_run": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_float, _vp]),
    "blk_attention_run_strided": (C.c_int, [_vp, _vp, _vp, _vp, _vp, C.c_int64, C.c_int64, C.c_float, _vp]),
    "blk_softmax_plan_create": (C.c_int, [C.POINTER(_vp), _i64p, _i64p, _i64p, C.c_int64, C.c_int64, C.c_int,
                                          C.c_int]),
    "blk_softmax_run": (C.c_int, [_vp, _vp, _vp, C.c_float, _vp]),
    "blk_softmax_backward_run": (C.c_int, [_vp, _vp, _vp, _vp, C.c_float, _vp]),
    "blk_softmax_noalloc": (C.c_int, [_vp, _vp, _i64p, _i64p, C.c_int64, C.c_int64, C.c_int, C.c_float, _vp]),
    "blk_plan_destroy": (None, [_vp]),
    "blk_plan_extents": (C.c_int, [_vp, _i64p, _i64p, _i64p]),
    "blk_plan_offsets": (C.c_int, [_vp, _i64p, _i64p, _i64p]),
    "blk_plan_summary": (C.c_int, [_vp, _i64p]),
    "blk_plan_table": (C.c_int, [_vp, C.c_int, _vp, C.c_int64, _i64p, _i64p]),
    "blk_plan_work": (C.c_int, [_vp, _f64p, _f64p]),
    "blk_plan_check": (C.c_int, [_vp, _vp]),
}


class BlkError(RuntimeError):
    """A libblkattn call failed; ``code`` is the blk_status_t value."""

    def __init__(self, code: int, message: str):
        super().__init__(f"libblkattn error {code}: {message}")
        self.code = code


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python blockedattention_b200/build.py` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def check(rc: int) -> None:
    if rc != BLK_OK:
        raise BlkError(rc, lib.blk_last_error().decode("utf-8", "replace"))


def i64(arr):
    """ctypes pointer to a contiguous int64 numpy array (or None)."""
    if arr is None:
        return None
    return arr.ctypes.data_as(_i64p)
