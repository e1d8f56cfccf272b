"""ctypes binding of the C ABI in include/fa2_b200.h (libfa2_b200.so).

This is the lowest Python layer: it passes raw device pointers, sizes and strides and fails
loudly when the CUDA library is missing; there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_DIR = Path(__file__).resolve().parent.parent / "lib"
LIB_PATH = _LIB_DIR / "libfa2_b200.so"

FA2_F16, FA2_BF16 = 0, 1
FA2_BWD_STATIC_MAX_ELEMENTS = 4194304


class FwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("lse", C.c_void_p),
        ("alibi_slopes", C.c_void_p), ("alibi_batch_stride", C.c_int32), ("dtype", C.c_int32),
        ("batch", C.c_int32), ("seqlen_q", C.c_int32), ("seqlen_k", C.c_int32),
        ("heads", C.c_int32), ("heads_k", C.c_int32), ("head_dim", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("o_stride", C.c_int64 * 3),
        ("softmax_scale", C.c_float), ("causal", C.c_int32),
        ("window_left", C.c_int32), ("window_right", C.c_int32), ("softcap", C.c_float),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("total_q", C.c_int32), ("total_k", C.c_int32), ("zero_tensors", C.c_int32),
    ]


class BwdPreprocessArgs(C.Structure):
    _fields_ = [
        ("dout", C.c_void_p), ("out", C.c_void_p), ("delta", C.c_void_p), ("dtype", C.c_int32),
        ("batch", C.c_int32), ("seqlen_q", C.c_int32), ("heads", C.c_int32), ("head_dim", C.c_int32),
        ("do_stride", C.c_int64 * 3), ("o_stride", C.c_int64 * 3),
        ("cu_seqlens_q", C.c_void_p), ("total_q", C.c_int32),
    ]


class BwdArgs(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("dout", C.c_void_p),
        ("lse", C.c_void_p), ("delta", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dq_accum", C.c_void_p), ("dq_accum_bytes", C.c_int64), ("dtype", C.c_int32),
        ("batch", C.c_int32), ("seqlen_q", C.c_int32), ("seqlen_k", C.c_int32),
        ("heads", C.c_int32), ("heads_k", C.c_int32), ("head_dim", C.c_int32),
        ("q_stride", C.c_int64 * 3), ("k_stride", C.c_int64 * 3), ("v_stride", C.c_int64 * 3),
        ("do_stride", C.c_int64 * 3),
        ("softmax_scale", C.c_float), ("causal", C.c_int32),
        ("window_left", C.c_int32), ("window_right", C.c_int32), ("which", C.c_int32),
        ("cu_seqlens_q", C.c_void_p), ("cu_seqlens_k", C.c_void_p),
        ("total_q", C.c_int32), ("total_k", C.c_int32),
        ("ev_kernel_start", C.c_void_p), ("ev_kernel_stop", C.c_void_p),
        ("alibi_slopes", C.c_void_p), ("alibi_batch_stride", C.c_int32), ("softcap", C.c_float),
    ]


# Every symbol include/fa2_b200.h declares; the CPU test suite checks that the library exports them.
EXPORTS = (
    "fa2_fwd", "fa2_varlen_fwd", "fa2_bwd_preprocess", "fa2_bwd_workspace_bytes", "fa2_bwd",
    "fa2_bwd_static", "fa2_bwd_static_status", "fa2_layout_is_addressable", "fa2_pack_16bit", "fa2_copy_16bit",
    "fa2_last_error", "fa2_device_status", "fa2_sm_count",
)

_lib = None


def load() -> C.CDLL:
    """Loads libfa2_b200.so (built by build.py); raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python kernels-community-rs_b200/build.py` "
                "(this package has no CPU fallback)")
        lib = C.CDLL(str(LIB_PATH))
        lib.fa2_last_error.restype = C.c_char_p
        for name in ("fa2_fwd", "fa2_varlen_fwd"):
            getattr(lib, name).argtypes = [C.POINTER(FwdArgs), C.c_void_p]
            getattr(lib, name).restype = C.c_int
        if hasattr(lib, "fa2_bwd_preprocess"):
            lib.fa2_bwd_preprocess.argtypes = [C.POINTER(BwdPreprocessArgs), C.c_void_p]
            lib.fa2_bwd_preprocess.restype = C.c_int
            lib.fa2_bwd.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
            lib.fa2_bwd.restype = C.c_int
            lib.fa2_bwd_workspace_bytes.argtypes = [C.POINTER(BwdArgs)]
            lib.fa2_bwd_workspace_bytes.restype = C.c_int64
        if hasattr(lib, "fa2_bwd_static"):
            lib.fa2_bwd_static.argtypes = [C.POINTER(BwdArgs), C.c_void_p]
            lib.fa2_bwd_static.restype = C.c_int
            lib.fa2_bwd_static_status.argtypes = [C.c_int]
            lib.fa2_bwd_static_status.restype = C.c_int
        lib.fa2_device_status.argtypes = [C.c_int]
        lib.fa2_device_status.restype = C.c_int
        lib.fa2_sm_count.argtypes = [C.c_int]
        lib.fa2_sm_count.restype = C.c_int
        _lib = lib
    return _lib


_ERRORS = {-1: ValueError, -2: TypeError, -3: RuntimeError}


def check(rc: int) -> None:
    if rc != 0:
        msg = load().fa2_last_error().decode()
        raise _ERRORS.get(rc, RuntimeError)(msg)
