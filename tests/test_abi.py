"""The C-ABI library loads, exports every symbol declared in include/nvnorms.h, and its
host-only entry points (shape bookkeeping, status text) behave like the reference's
OpKernel checks.  No compute call is made here: these tests run without a GPU."""
import ctypes
import os
import re

import pytest

from atex_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    with open(os.path.join(ROOT, "include", "nvnorms.h")) as f:
        text = f.read()
    return sorted(set(re.findall(r"NVN_API\s+[\w\s\*]+?\b(nvn_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = _declared_symbols()
    for must in ("nvn_ln_fwd", "nvn_ln_bwd", "nvn_in_fwd", "nvn_in_bwd", "nvn_ln_dims", "nvn_in_dims",
                 "nvn_ln_bwd_workspace_bytes", "nvn_status_string"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    for name in _declared_symbols():
        assert hasattr(lib, name), f"{name} declared in nvnorms.h but not exported"


def test_python_binding_covers_every_declared_symbol():
    assert sorted(L.SIGNATURES) == _declared_symbols()


def test_version_and_status_strings(lib):
    assert lib.nvn_version() >= 100
    assert L.status_string(0) == "ok"
    assert L.status_string(L.NVN_ERR_AXIS_NOT_PACKED) == "axis is not packed from last dim."
    assert L.status_string(L.NVN_ERR_AXIS_RANGE) == "axis contains invalid value"
    assert "data format" in L.status_string(L.NVN_ERR_DATA_FORMAT)
    assert L.status_string(-12345) == "unknown status"


def _ln_dims(lib, dims, axis):
    d = (ctypes.c_int64 * len(dims))(*dims)
    a = (ctypes.c_int * max(1, len(axis)))(*axis)
    N, D = ctypes.c_int64(), ctypes.c_int64()
    st = lib.nvn_ln_dims(len(dims), d, len(axis), a, ctypes.byref(N), ctypes.byref(D))
    return st, N.value, D.value


def test_ln_dims_follow_the_reference_axis_rule(lib):
    # axis variants of the reference layer test: [1,2], [-2,-1], [1,-1], [-2,2], -1
    for axis in ([1, 2], [-2, -1], [1, -1], [-2, 2]):
        assert _ln_dims(lib, [2, 3, 4], axis) == (0, 2, 12)
    assert _ln_dims(lib, [2, 3, 4], [-1]) == (0, 6, 4)
    assert _ln_dims(lib, [12000, 128, 8, 8], [1, 2, 3]) == (0, 12000, 8192)
    assert _ln_dims(lib, [7], [0]) == (0, 1, 7)
    assert _ln_dims(lib, [2, 2, 2], [2, 2, 2]) == (0, 4, 2)  # duplicates collapse
    assert _ln_dims(lib, [0, 5], [1]) == (0, 0, 5)  # empty batch
    assert _ln_dims(lib, [2, 3, 4], [0])[0] == L.NVN_ERR_AXIS_NOT_PACKED
    assert _ln_dims(lib, [2, 3, 4], [0, 2])[0] == L.NVN_ERR_AXIS_NOT_PACKED
    assert _ln_dims(lib, [2, 3, 4], [3])[0] == L.NVN_ERR_AXIS_RANGE
    assert _ln_dims(lib, [2, 3, 4], [-4])[0] == L.NVN_ERR_AXIS_RANGE


def _in_dims(lib, dims, fmt):
    d = (ctypes.c_int64 * len(dims))(*dims)
    N, C, D, cf = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int()
    st = lib.nvn_in_dims(len(dims), d, fmt.encode(), ctypes.byref(N), ctypes.byref(C), ctypes.byref(D),
                         ctypes.byref(cf))
    return st, N.value, C.value, D.value, cf.value


def test_in_dims_follow_the_reference_format_rule(lib):
    assert _in_dims(lib, [2, 32, 8, 8], "NC...") == (0, 2, 32, 64, 1)
    assert _in_dims(lib, [2, 8, 8, 32], "N...C") == (0, 2, 32, 64, 0)
    assert _in_dims(lib, [2, 32, 4, 4, 4], "NCDHW") == (0, 2, 32, 64, 1)
    assert _in_dims(lib, [2, 4, 4, 4, 32], "NDHWC") == (0, 2, 32, 64, 0)
    assert _in_dims(lib, [2, 3, 4, 5], "NHWC") == (0, 2, 5, 12, 0)
    for bad in ("NC", "XYZ", "CN..", "", "N..."):
        assert _in_dims(lib, [2, 3, 4, 5], bad)[0] == L.NVN_ERR_DATA_FORMAT
    assert _in_dims(lib, [2, 3, 4], "NC...")[0] == L.NVN_ERR_RANK


def test_null_pointers_are_rejected_not_dereferenced(lib):
    assert lib.nvn_ln_dims(2, None, 1, None, None, None) == L.NVN_ERR_INVALID_ARGUMENT
    assert lib.nvn_in_dims(4, None, None, None, None, None, None) == L.NVN_ERR_INVALID_ARGUMENT
    # Bad dtype and null buffers are refused before anything touches CUDA.
    assert lib.nvn_ln_fwd(9, None, None, None, 4, 4, 1e-3, None, None, None, None, 0, None) == L.NVN_ERR_INVALID_ARGUMENT
    assert lib.nvn_ln_fwd(0, None, None, None, 4, 4, 1e-3, None, None, None, None, 0, None) == L.NVN_ERR_INVALID_ARGUMENT
    assert lib.nvn_in_bwd(0, None, None, None, None, None, 2, 3, 4, 1, None, None, None, None, 0, None) == L.NVN_ERR_INVALID_ARGUMENT
    # Empty forward problems are a no-op that needs no buffers.
    assert lib.nvn_ln_fwd(0, None, None, None, 0, 8, 1e-3, None, None, None, None, 0, None) == L.NVN_OK
    assert lib.nvn_in_fwd(1, None, None, None, 2, 0, 8, 1, 1e-3, None, None, None, None, 0, None) == L.NVN_OK
