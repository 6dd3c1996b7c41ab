"""ctypes front end of the C oracle (oracle/norms_oracle.c).  TEST INFRASTRUCTURE ONLY.

Arrays are NumPy: activations as float32, float16 or - for bfloat16 - uint16 bit
patterns together with ``dtype="bf16"``.  The ``*_64`` entry points return float64
results (the checker); the ``*_32`` entry points are a port of the reference's fp32
CPU functors that write outputs in the activation dtype and exist to be timed.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "liboracle.so")
_lib = None

DTYPE_CODE = {"f32": 0, "f16": 1, "bf16": 2}
_NP_OF = {"f32": np.float32, "f16": np.float16, "bf16": np.uint16}


def build(force: bool = False) -> str:
    """Compile the C oracle with the Makefile beside it (gcc, OpenMP)."""
    src_m = max(os.path.getmtime(os.path.join(_HERE, f)) for f in ("norms_oracle.c", "norms_core.inc"))
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < src_m:
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_half_to_f32.restype = ctypes.c_float
        _lib.oracle_half_to_f32.argtypes = [ctypes.c_uint16]
        _lib.oracle_f32_to_half.restype = ctypes.c_uint16
        _lib.oracle_f32_to_half.argtypes = [ctypes.c_float]
        _lib.oracle_f32_to_bf16.restype = ctypes.c_uint16
        _lib.oracle_f32_to_bf16.argtypes = [ctypes.c_float]
    return _lib


def set_num_threads(n: int) -> int:
    """Size of the OpenMP team used by the C oracle from now on; returns what is in effect."""
    fn = lib().oracle_set_num_threads
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int]
    return int(fn(int(n)))


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _act(a, dtype):
    a = np.ascontiguousarray(a)
    if a.dtype != _NP_OF[dtype]:
        raise TypeError(f"activation array must be {_NP_OF[dtype]} for dtype {dtype}, got {a.dtype}")
    return a


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _i64(v):
    return ctypes.c_int64(int(v))


def ln_fwd(x, gamma, beta, eps, dtype, want_y=True, fp32_port=False):
    """x [N, D].  Returns (y or None, mean, inv_std)."""
    x = _act(x, dtype)
    N, D = x.shape
    gamma, beta = _f32(gamma), _f32(beta)
    acc = np.float32 if fp32_port else np.float64
    y = None
    if want_y:
        y = np.empty((N, D), dtype=_NP_OF[dtype] if fp32_port else np.float64)
    mean = np.empty(N, dtype=acc)
    ivar = np.empty(N, dtype=acc)
    fn = lib().oracle_ln_fwd_32 if fp32_port else lib().oracle_ln_fwd_64
    fn(ctypes.c_int(DTYPE_CODE[dtype]), _p(x), _p(gamma), _p(beta), _i64(N), _i64(D),
       ctypes.c_double(eps), _p(y), _p(mean), _p(ivar))
    return y, mean, ivar


def ln_bwd(dy, x, gamma, mean, inv_std, dtype, want_dx=True, fp32_port=False):
    """Returns (dx or None, dgamma, dbeta)."""
    x = _act(x, dtype)
    dy = _act(dy, dtype)
    N, D = x.shape
    gamma, mean, inv_std = _f32(gamma), _f32(mean), _f32(inv_std)
    acc = np.float32 if fp32_port else np.float64
    dx = None
    if want_dx:
        dx = np.empty((N, D), dtype=_NP_OF[dtype] if fp32_port else np.float64)
    dg = np.empty(D, dtype=acc)
    db = np.empty(D, dtype=acc)
    fn = lib().oracle_ln_bwd_32 if fp32_port else lib().oracle_ln_bwd_64
    fn(ctypes.c_int(DTYPE_CODE[dtype]), _p(dy), _p(x), _p(gamma), _p(mean), _p(inv_std), _i64(N),
       _i64(D), _p(dx), _p(dg), _p(db))
    return dx, dg, db


def _ncd(shape, channel_first):
    return (shape[0], shape[1], shape[2]) if channel_first else (shape[0], shape[2], shape[1])


def in_fwd(x, gamma, beta, eps, channel_first, dtype, want_y=True, fp32_port=False):
    """x [N, C, D] (channel_first) or [N, D, C].  Returns (y or None, mean [N, C], inv_std [N, C])."""
    x = _act(x, dtype)
    N, C, D = _ncd(x.shape, channel_first)
    gamma, beta = _f32(gamma), _f32(beta)
    acc = np.float32 if fp32_port else np.float64
    y = None
    if want_y:
        y = np.empty(x.shape, dtype=_NP_OF[dtype] if fp32_port else np.float64)
    mean = np.empty((N, C), dtype=acc)
    ivar = np.empty((N, C), dtype=acc)
    fn = lib().oracle_in_fwd_32 if fp32_port else lib().oracle_in_fwd_64
    fn(ctypes.c_int(DTYPE_CODE[dtype]), _p(x), _p(gamma), _p(beta), _i64(N), _i64(C), _i64(D),
       ctypes.c_int(1 if channel_first else 0), ctypes.c_double(eps), _p(y), _p(mean), _p(ivar))
    return y, mean, ivar


def in_bwd(dy, x, gamma, mean, inv_std, channel_first, dtype, want_dx=True, fp32_port=False):
    """Returns (dx or None, dgamma [C], dbeta [C])."""
    x = _act(x, dtype)
    dy = _act(dy, dtype)
    N, C, D = _ncd(x.shape, channel_first)
    gamma, mean, inv_std = _f32(gamma), _f32(mean), _f32(inv_std)
    acc = np.float32 if fp32_port else np.float64
    dx = None
    if want_dx:
        dx = np.empty(x.shape, dtype=_NP_OF[dtype] if fp32_port else np.float64)
    dg = np.empty(C, dtype=acc)
    db = np.empty(C, dtype=acc)
    fn = lib().oracle_in_bwd_32 if fp32_port else lib().oracle_in_bwd_64
    fn(ctypes.c_int(DTYPE_CODE[dtype]), _p(dy), _p(x), _p(gamma), _p(mean), _p(inv_std), _i64(N),
       _i64(C), _i64(D), ctypes.c_int(1 if channel_first else 0), _p(dx), _p(dg), _p(db))
    return dx, dg, db
