"""ctypes binding of ``libmtb200.so`` (declarations: ``include/mtb200.h``).

The shared library is built in-tree by :mod:`minitensor_b200.build`.  There is
no fallback: if the library is missing, or a call returns a non-zero status,
an exception is raised.  The exception classes follow the mapping minitensor's
Python bindings use for engine errors (``bindings/src/error.rs:15-67``):
shape / argument problems -> ``ValueError``, dtype problems -> ``TypeError``,
allocation -> ``MemoryError``, everything else -> ``RuntimeError``.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libmtb200.so")

OK, ERR_INVALID, ERR_CUDA, ERR_NOMEM, ERR_UNSUPPORTED, ERR_DEVICE_WAIT, ERR_BAD_LABEL = range(7)
F32, F64, I32, I64, BOOL = range(5)
EPI_NONE, EPI_RELU, EPI_GELU_ERF, EPI_GELU_TANH, EPI_RELU_BWD = range(5)

_i32, _i64, _vp, _f32, _f64 = C.c_int32, C.c_int64, C.c_void_p, C.c_float, C.c_double

# name -> (restype, argtypes); mirrors include/mtb200.h one to one
SIGNATURES = {
    "mtb200_version": (_i32, []),
    "mtb200_last_error": (C.c_char_p, []),
    "mtb200_create": (_i32, [_i32, C.POINTER(_vp)]),
    "mtb200_destroy": (_i32, [_vp]),
    "mtb200_set_stream": (_i32, [_vp, _vp]),
    "mtb200_set_gemm_sm_limit": (_i32, [_vp, _i32]),
    "mtb200_sync": (_i32, [_vp]),
    "mtb200_profile_enable": (_i32, [_vp, _i32]),
    "mtb200_profile_read": (_i32, [_vp, _i32, C.POINTER(_i64), C.POINTER(_f64), C.POINTER(_f64)]),
    "mtb200_workspace_bytes": (_i32, [_vp, C.POINTER(C.c_size_t)]),
    "mtb200_alloc": (_i32, [_vp, C.c_size_t, C.POINTER(_vp)]),
    "mtb200_free": (_i32, [_vp, _vp, C.c_size_t]),
    "mtb200_h2d": (_i32, [_vp, _vp, _vp, C.c_size_t]),
    "mtb200_d2h": (_i32, [_vp, _vp, _vp, C.c_size_t]),
    "mtb200_memset_zero": (_i32, [_vp, _vp, C.c_size_t]),
    "mtb200_gemm": (_i32, [_vp, _i32, _i32, _i32, _i64, _i64, _i64, _i64, _vp, _i64, _vp, _i64,
                           _vp, _i64, _vp, _i32, _vp, _i32]),
    "mtb200_dense_saved_bytes": (_i32, [_i32, _i64, _i64, _i64, C.POINTER(C.c_size_t)]),
    "mtb200_dense_forward": (_i32, [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _i32, _vp, _vp]),
    "mtb200_dense_backward": (_i32, [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32]),
    "mtb200_dense_dy_bytes": (_i32, [_i32, _i64, _i64, _i64, C.POINTER(C.c_size_t)]),
    "mtb200_colsum": (_i32, [_vp, _i32, _i64, _i64, _vp, _vp]),
    "mtb200_colsum_noalloc": (_i32, [_vp, _i32, _i64, _i64, _vp, _vp]),
    "mtb200_act_fwd": (_i32, [_vp, _i32, _i32, _i64, _vp, _vp]),
    "mtb200_act_bwd": (_i32, [_vp, _i32, _i32, _i64, _vp, _vp, _vp]),
    "mtb200_bias_act": (_i32, [_vp, _i32, _i64, _i64, _vp, _vp, _i32, _vp]),
    "mtb200_cross_entropy": (_i32, [_vp, _i64, _i64, _vp, _vp, _i32, _i32, _f32, _vp, _vp]),
    "mtb200_cross_entropy_ex": (_i32, [_vp, _i64, _i64, _vp, _vp, _i32, _i32, _f32, _vp, _vp, _vp]),
    "mtb200_batch_norm_fwd": (_i32, [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _f64, _f64, _vp, _vp, _vp]),
    "mtb200_batch_norm_bwd": (_i32, [_vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _vp, _i32, _vp, _vp, _vp]),
    "mtb200_dropout_mask": (_i32, [_vp, _i32, _i64, _f64, C.c_uint64, C.c_uint64, _vp]),
    "mtb200_dropout_apply": (_i32, [_vp, _i32, _i64, _i64, _vp, _f64, C.c_uint64, C.c_uint64, _vp]),
    "mtb200_mask_mul": (_i32, [_vp, _i32, _i64, _i64, _vp, _vp, _vp]),
    "mtb200_sgd_step": (_i32, [_vp, _i32, _i64, _vp, _vp, _vp, _f64, _f64, _f64, _f64, _i32]),
    "mtb200_rmsprop_step": (_i32, [_vp, _i32, _i64, _vp, _vp, _vp, _vp, _vp, _f64, _f64, _f64, _f64, _f64]),
    "mtb200_sumsq": (_i32, [_vp, _i32, _i64, _vp, _vp, _i32]),
    "mtb200_scale": (_i32, [_vp, _i32, _i64, _vp, _f64]),
    "mtb200_add_inplace": (_i32, [_vp, _i32, _i64, _vp, _vp]),
    "mtb200_swap_dims": (_i32, [_vp, _i32, _i64, _i64, _i64, _i64, _i64, _vp, _vp]),
    "mtb200_clamp": (_i32, [_vp, _i32, _i64, _vp, _f64, _f64]),
    "mtb200_adam_step": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _f64, _f64, _f64, _f64, _f64, _i32,
                                _i64, _f32]),
    "mtb200_adam_step_counted": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _f64, _f64, _f64, _f64, _f64, _i32, _vp, _i32, _f32]),
    "mtb200_conv2d_fwd": (_i32, [_vp] + [_i64] * 11 + [_vp, _vp, _vp, _vp, _i32]),
    "mtb200_conv2d_bwd_data": (_i32, [_vp] + [_i64] * 11 + [_vp, _vp, _vp, _i32]),
    "mtb200_conv2d_bwd_weight": (_i32, [_vp] + [_i64] * 11 + [_vp, _vp, _vp, _i32]),
    "mtb200_conv2d_bwd_bias": (_i32, [_vp, _i64, _i64, _i64, _i64, _vp, _vp]),
    "mtb200_comm_unique_id": (_i32, [_vp]),
    "mtb200_comm_init_rank": (_i32, [_i32, _i32, _vp, _i32, C.POINTER(_vp)]),
    "mtb200_comm_init": (_i32, [_i32, C.POINTER(_i32), C.POINTER(_vp)]),
    "mtb200_comm_set_stream": (_i32, [_vp, _i32, _vp]),
    "mtb200_comm_group_begin": (_i32, [_vp]),
    "mtb200_comm_group_end": (_i32, [_vp]),
    "mtb200_allreduce_sum_f32": (_i32, [_vp, _i32, _vp, C.c_size_t, _f32]),
    "mtb200_comm_destroy": (_i32, [_vp]),
    "mtb200_selftest_wait_expiry": (_i32, [_vp, _i32]),
}

_lib = None


class Mtb200Error(RuntimeError):
    """A library call failed; ``.status`` holds the MTB200_ERR_* code."""

    def __init__(self, status: int, message: str):
        super().__init__(message)
        self.status = status


def load() -> C.CDLL:
    """Load the in-tree shared library, binding every declared entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m minitensor_b200.build` "
            "(nvcc, sm_100a). There is no CPU or PyTorch fallback for this path.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the build lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def last_error() -> str:
    return load().mtb200_last_error().decode("utf-8", "replace")


def check(status: int) -> None:
    """Raise the Python exception that corresponds to a non-zero status."""
    if status == OK:
        return
    msg = last_error()
    if status == ERR_INVALID:
        raise ValueError(msg)
    if status == ERR_UNSUPPORTED:
        raise (TypeError if "dtype" in msg or "boolean" in msg else ValueError)(msg)
    if status == ERR_NOMEM:
        raise MemoryError(msg)
    if status == ERR_BAD_LABEL:
        raise IndexError(msg)
    raise Mtb200Error(status, msg)
