"""ctypes binding of libnvnorms.so: the same C ABI a TensorFlow OpKernel binds
(include/nvnorms.h).  There is no fallback: if the library has not been built
the import of the ops fails with instructions, and nothing here computes on the
CPU.
"""
from __future__ import annotations

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libnvnorms.so")

NVN_F32, NVN_F16, NVN_BF16 = 0, 1, 2

NVN_OK = 0
NVN_ERR_INVALID_ARGUMENT = -1
NVN_ERR_AXIS_RANGE = -2
NVN_ERR_AXIS_NOT_PACKED = -3
NVN_ERR_DATA_FORMAT = -4
NVN_ERR_RANK = -5
NVN_ERR_WORKSPACE = -6
NVN_ERR_CUDA = -7
NVN_ERR_UNSUPPORTED = -8
NVN_ERR_LIMIT = -9
NVN_ERR_TIMEOUT = -10

_c = ctypes
_i64 = _c.c_int64
_vp = _c.c_void_p
_int = _c.c_int
_sz = _c.c_size_t

NVN_DP_MAX_RANKS = 16


class DpComm(ctypes.Structure):
    """nvn_dp_comm of include/nvnorms.h."""
    _fields_ = [("rank", ctypes.c_int), ("world", ctypes.c_int),
                ("recv", ctypes.c_void_p * NVN_DP_MAX_RANKS),
                ("epoch", ctypes.c_uint32), ("defer", ctypes.c_int),
                ("device_epochs", ctypes.c_void_p)]


# name -> (restype, argtypes); mirrors include/nvnorms.h declaration by declaration
SIGNATURES = {
    "nvn_version": (_int, []),
    "nvn_status_string": (_c.c_char_p, [_int]),
    "nvn_last_cuda_error": (_int, []),
    "nvn_launch_count": (_c.c_uint64, []),
    "nvn_device_status": (_int, []),
    "nvn_ln_dims": (_int, [_int, _c.POINTER(_i64), _int, _c.POINTER(_int), _c.POINTER(_i64),
                           _c.POINTER(_i64)]),
    "nvn_in_dims": (_int, [_int, _c.POINTER(_i64), _c.c_char_p, _c.POINTER(_i64), _c.POINTER(_i64),
                           _c.POINTER(_i64), _c.POINTER(_int)]),
    "nvn_ln_fwd_workspace_bytes": (_sz, [_int, _i64, _i64]),
    "nvn_ln_bwd_workspace_bytes": (_sz, [_int, _i64, _i64]),
    "nvn_in_fwd_workspace_bytes": (_sz, [_int, _i64, _i64, _i64, _int]),
    "nvn_in_bwd_workspace_bytes": (_sz, [_int, _i64, _i64, _i64, _int]),
    "nvn_ln_fwd": (_int, [_int, _vp, _vp, _vp, _i64, _i64, _c.c_float, _vp, _vp, _vp, _vp, _sz, _vp]),
    "nvn_ln_fwd_residual": (_int, [_int, _vp, _vp, _vp, _vp, _i64, _i64, _c.c_float, _vp, _vp, _vp, _vp,
                                   _vp, _sz, _vp]),
    "nvn_ln_bwd": (_int, [_int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "nvn_in_fwd": (_int, [_int, _vp, _vp, _vp, _i64, _i64, _i64, _int, _c.c_float, _vp, _vp, _vp,
                          _vp, _sz, _vp]),
    "nvn_in_bwd": (_int, [_int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp,
                          _vp, _sz, _vp]),
    "nvn_describe_plan": (_int, [_int, _int, _i64, _i64, _i64, _int, _c.c_char_p, _sz]),
    "nvn_dp_finish": (_int, [_i64, _c.POINTER(DpComm), _vp, _vp, _vp]),
    "nvn_dp_recv_bytes": (_sz, [_i64, _int]),
    "nvn_ln_bwd_dp": (_int, [_int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp, _sz,
                             _c.POINTER(DpComm), _vp]),
    "nvn_ln_bwd_noalloc": (_int, [_int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _vp, _vp, _vp, _vp]),
    "nvn_in_bwd_dp": (_int, [_int, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _int, _vp, _vp, _vp,
                             _vp, _sz, _c.POINTER(DpComm), _vp]),
}

_lib = None


def load() -> ctypes.CDLL:
    """dlopen libnvnorms.so (once) and attach the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: the CUDA library has not been built. "
            "Run `python -m atex_b200.build` (needs nvcc with sm_100a support). "
            "There is no CPU or PyTorch fallback for these ops.")
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def status_string(code: int) -> str:
    return load().nvn_status_string(code).decode()


def describe_plan(op: int, dtype: int, N: int, C: int, D: int, channel_first: int) -> str:
    buf = ctypes.create_string_buffer(256)
    st = load().nvn_describe_plan(op, dtype, N, C, D, channel_first, buf, 256)
    if st != NVN_OK:
        return f"<{status_string(st)}>"
    return buf.value.decode()
