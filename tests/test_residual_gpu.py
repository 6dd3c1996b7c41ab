"""Residual add fused into the LayerNorm forward (nvn_ln_fwd_residual).

s = T(x + residual) must be bit-exact (one fp32 addition, one rounding to T); y and the
saved statistics are checked against the float64 oracle evaluated ON s - the tensor the
backward pass will read.  Shapes cover the fused kernel (every shape family of its table,
widths that do not fill a shape), the fallback (rows beyond 4096 vectors, widths that rule
out 128-bit accesses, misaligned buffers) and in-place use (sum_out = x).
"""
import numpy as np
import pytest
import torch

import atex_b200 as A
from atex_b200 import _lib
from atex_b200 import testing as T

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _sum_reference(x, r):
    """fp32 addition rounded once to the activation type."""
    return (x.float() + r.float()).to(x.dtype)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
@pytest.mark.parametrize("N,D", [(7, 32), (300, 128), (64, 512), (33, 1024), (257, 4096), (40, 768),
                                 (19, 5120), (6, 16384), (5, 32768), (3, 65536), (9, 1000), (11, 33)])
def test_residual_forward_matches_the_oracle_on_the_sum(lib, dtype, N, D):
    from oracle import oracle
    g = torch.Generator().manual_seed(N * 131 + D)
    dt = T.TORCH_DTYPE[dtype]
    x = (torch.randn(N, D, generator=g) * 2 + 0.5).to(dt)
    r = (torch.randn(N, D, generator=g) * 3 - 1.0).to(dt)
    gamma = torch.rand(D, generator=g) + 0.5
    beta = torch.randn(D, generator=g) * 0.1
    y, s, m, iv = A.fused_layer_norm_residual_op(x.to(DEV), r.to(DEV), gamma.to(DEV), beta.to(DEV),
                                                 epsilon=1e-5)
    torch.cuda.synchronize()
    s_ref = _sum_reference(x, r)
    assert torch.equal(s.cpu(), s_ref), "the residual sum must be bit-exact"
    y64, m64, s64 = oracle.ln_fwd(T.to_numpy(s_ref), gamma.numpy(), beta.numpy(), 1e-5, dtype)
    assert T.activation_error(y, y64, dtype)[0] <= 1.0
    assert T.stats_error(m, iv, m64, s64)[0] <= 1.0
    # and it is the same as the two separate steps, bit for bit
    y2, m2, iv2 = A.fused_layer_norm_op(s_ref.to(DEV), gamma.to(DEV), beta.to(DEV), epsilon=1e-5)
    torch.cuda.synchronize()
    assert T.activation_error(y, T.to_float64(y2), dtype)[0] <= 1.0
    assert lib.nvn_device_status() == _lib.NVN_OK


def test_residual_in_place_and_backward_on_the_sum(lib):
    from oracle import oracle
    g = torch.Generator().manual_seed(3)
    N, D = 512, 2048
    x = torch.randn(N, D, generator=g).bfloat16()
    r = torch.randn(N, D, generator=g).bfloat16()
    dy = torch.randn(N, D, generator=g).bfloat16()
    gamma, beta = torch.rand(D, generator=g) + 0.5, torch.zeros(D)
    xd = x.to(DEV)
    y, s, m, iv = A.fused_layer_norm_residual_op(xd, r.to(DEV), gamma.to(DEV), beta.to(DEV),
                                                 out_sum=xd)   # the residual stream, updated in place
    assert s.data_ptr() == xd.data_ptr()
    dx, dg, db = A.fused_layer_norm_grad_op(dy.to(DEV), s, gamma.to(DEV), m, iv)
    torch.cuda.synchronize()
    s_ref = _sum_reference(x, r)
    assert torch.equal(s.cpu(), s_ref)
    dx64, dg64, db64 = oracle.ln_bwd(T.to_numpy(dy), T.to_numpy(s_ref), gamma.numpy(), m.cpu().numpy(),
                                     iv.cpu().numpy(), "bf16")
    assert T.activation_error(dx, dx64, "bf16")[0] <= 1.0
    assert T.grad_param_error(dg, dg64)[0] <= 1.0
    assert T.grad_param_error(db, db64)[0] <= 1.0


def test_residual_with_misaligned_buffers_takes_the_two_step_path(lib):
    g = torch.Generator().manual_seed(5)
    N, D = 37, 256
    base_x = torch.randn(N * D + 1, generator=g).half().to(DEV)
    base_r = torch.randn(N * D + 1, generator=g).half().to(DEV)
    x, r = base_x[1:].view(N, D), base_r[1:].view(N, D)      # 2-byte aligned only
    gamma, beta = (torch.rand(D, generator=g) + 0.5).to(DEV), torch.zeros(D, device=DEV)
    y, s, m, iv = A.fused_layer_norm_residual_op(x, r, gamma, beta)
    torch.cuda.synchronize()
    s_ref = _sum_reference(x.cpu(), r.cpu())
    assert torch.equal(s.cpu(), s_ref)
    y2, m2, iv2 = A.fused_layer_norm_op(s_ref.to(DEV), gamma, beta)
    assert T.activation_error(y, T.to_float64(y2), "f16")[0] <= 1.0


def test_residual_argument_checks():
    x = torch.zeros(4, 8, device=DEV)
    with pytest.raises(A.InvalidArgumentError):
        A.fused_layer_norm_residual_op(x, torch.zeros(4, 9, device=DEV), torch.ones(8, device=DEV),
                                       torch.zeros(8, device=DEV))
    y, s, m, iv = A.fused_layer_norm_residual_op(torch.zeros(0, 8, device=DEV), torch.zeros(0, 8, device=DEV),
                                                 torch.ones(8, device=DEV), torch.zeros(8, device=DEV))
    assert y.shape == (0, 8) and m.shape == (0,)
