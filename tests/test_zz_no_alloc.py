"""nvn_ln_bwd_noalloc: the LayerNorm backward entry point for callers that cannot pass a
workspace (a plugin callback that only gets input / output pointers, a process whose
device memory belongs to another pool, a loop where cudaMalloc is not allowed).  Its
scratch is a fixed array inside the library, shared by all calls on a device.

Called here straight through the C ABI and compared with the regular nvn_ln_bwd on the
same inputs, twice in a row: the second call finds the first call's data in the shared
array and must not be disturbed by it.
"""
import ctypes

import pytest
import torch

from atex_b200 import _lib as L
from atex_b200 import testing as T

pytestmark = pytest.mark.gpu

_vp, _i64 = ctypes.c_void_p, ctypes.c_int64
NOALLOC_MAX = 16 << 20  # NVN_NOALLOC_SCRATCH_BYTES in include/nvnorms.h


def _noalloc(lib):
    return lib.nvn_ln_bwd_noalloc   # prototype attached by atex_b200._lib.load()


def _inputs(N, D, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    dt = T.TORCH_DTYPE[dtype]
    x = (torch.randn(N, D, generator=g) * 2 + 0.5).to(dt).cuda()
    dy = torch.randn(N, D, generator=g).to(dt).cuda()
    gamma = (torch.rand(D, generator=g) + 0.5).cuda()
    xf = x.float()
    mean = xf.mean(dim=1)
    inv_std = torch.rsqrt(xf.var(dim=1, unbiased=False) + 1e-5)
    return x, dy, gamma, mean.contiguous(), inv_std.contiguous()


@pytest.mark.parametrize("dtype,N,D", [("bf16", 2048, 4096), ("f32", 777, 1000), ("f16", 5000, 128),
                                       ("f16", 64, 8192)])
def test_noalloc_backward_matches_the_workspace_entry_point_twice(lib, dtype, N, D):
    assert torch.cuda.is_available()
    code = {"f32": L.NVN_F32, "f16": L.NVN_F16, "bf16": L.NVN_BF16}[dtype]
    fn = _noalloc(lib)
    stream = torch.cuda.current_stream().cuda_stream
    need = lib.nvn_ln_bwd_workspace_bytes(code, N, D)
    assert 0 < need <= NOALLOC_MAX
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    for call in range(2):
        x, dy, gamma, mean, inv_std = _inputs(N, D, dtype, seed=100 * call + N)
        dx_ref, dg_ref, db_ref = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
        st = lib.nvn_ln_bwd(code, dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                            inv_std.data_ptr(), N, D, dx_ref.data_ptr(), dg_ref.data_ptr(),
                            db_ref.data_ptr(), ws.data_ptr(), need, stream)
        assert st == L.NVN_OK
        dx, dg, db = torch.empty_like(x), torch.empty_like(gamma), torch.empty_like(gamma)
        st = fn(code, dy.data_ptr(), x.data_ptr(), gamma.data_ptr(), mean.data_ptr(),
                inv_std.data_ptr(), N, D, dx.data_ptr(), dg.data_ptr(), db.data_ptr(), stream)
        assert st == L.NVN_OK, L.status_string(st)
        torch.cuda.synchronize()
        # same kernels, same reduction order: within the suite's tolerances (in fact identical)
        assert T.activation_error(dx, T.to_float64(dx_ref), dtype)[0] <= 1.0
        assert T.grad_param_error(dg, T.to_float64(dg_ref))[0] <= 1.0
        assert T.grad_param_error(db, T.to_float64(db_ref))[0] <= 1.0
        assert torch.equal(dx, dx_ref) and torch.equal(dg, dg_ref) and torch.equal(db, db_ref)


def test_noalloc_rejects_problems_beyond_its_fixed_scratch(lib):
    fn = _noalloc(lib)
    # 2^23 columns: the partial rows alone need far more than the built-in array
    N, D = 2, 1 << 23
    assert lib.nvn_ln_bwd_workspace_bytes(L.NVN_F32, N, D) > NOALLOC_MAX
    x = torch.zeros(N, D, device="cuda")
    g = torch.ones(D, device="cuda")
    m = torch.zeros(N, device="cuda")
    dgdb = torch.full((2, D), 5.0, device="cuda")
    launches = lib.nvn_launch_count()
    st = fn(L.NVN_F32, x.data_ptr(), x.data_ptr(), g.data_ptr(), m.data_ptr(), m.data_ptr(), N, D,
            x.data_ptr(), dgdb[0].data_ptr(), dgdb[1].data_ptr(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == L.NVN_ERR_LIMIT
    assert "capacity" in L.status_string(st)
    assert lib.nvn_launch_count() == launches and torch.all(dgdb == 5.0)


def test_noalloc_empty_input_zero_fills_like_the_regular_entry_point(lib):
    fn = _noalloc(lib)
    D = 16
    dgdb = torch.full((2, D), 3.0, device="cuda")
    st = fn(L.NVN_F16, None, None, None, None, None, 0, D, None, dgdb[0].data_ptr(), dgdb[1].data_ptr(),
            torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert st == L.NVN_OK and torch.all(dgdb == 0)
