"""Helpers of the GPU parity tests: run an op through the public API (which calls the
C ABI), run the float64 C oracle on the same inputs, and compare within the stated
tolerances (atex_b200.testing)."""
import numpy as np
import torch

import atex_b200 as A
from atex_b200 import testing as T
from oracle import oracle

DEV = "cuda:0"


def rand_ln(N, D, dtype, seed, x_scale=3.0, x_shift=1.0):
    g = torch.Generator().manual_seed(seed)
    dt = T.TORCH_DTYPE[dtype]
    x = (torch.randn(N, D, generator=g) * x_scale + x_shift).to(dt)
    dy = torch.randn(N, D, generator=g).to(dt)
    gamma = torch.rand(D, generator=g) + 0.5
    beta = torch.randn(D, generator=g) * 0.1
    return x, dy, gamma, beta


def check_ln(x, dy, gamma, beta, eps, axis=(-1,), shape=None):
    """x, dy [N, D] CPU tensors; `shape` optionally reshapes them to a higher rank."""
    dtype = T.dtype_name(x)
    N, D = x.shape
    xs = x if shape is None else x.reshape(shape)
    dys = dy if shape is None else dy.reshape(shape)
    y, mean, inv_std = A.fused_layer_norm_op(xs.to(DEV), gamma.to(DEV), beta.to(DEV), axis=list(axis), epsilon=eps)
    dx, dgamma, dbeta = A.fused_layer_norm_grad_op(dys.to(DEV), xs.to(DEV), gamma.to(DEV), mean, inv_std, axis=list(axis))
    torch.cuda.synchronize()
    assert y.shape == xs.shape and dx.shape == xs.shape
    assert mean.shape == (N,) and inv_std.shape == (N,)
    assert dgamma.shape == gamma.shape and dbeta.shape == gamma.shape
    g1, b1 = gamma.reshape(-1).numpy(), beta.reshape(-1).numpy()
    y64, m64, s64 = oracle.ln_fwd(T.to_numpy(x), g1, b1, eps, dtype)
    dx64, dg64, db64 = oracle.ln_bwd(T.to_numpy(dy), T.to_numpy(x), g1, mean.cpu().numpy(), inv_std.cpu().numpy(), dtype)
    report(y.reshape(N, D), y64, mean, inv_std, m64, s64, dx.reshape(N, D), dx64, dgamma, dg64, dbeta, db64, dtype)
    return y, mean, inv_std, dx, dgamma, dbeta


def rand_in(N, C, spatial, channel_first, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    dt = T.TORCH_DTYPE[dtype]
    shape = (N, C) + tuple(spatial) if channel_first else (N,) + tuple(spatial) + (C,)
    x = (torch.randn(shape, generator=g) * 3 + 2).to(dt)
    dy = torch.randn(shape, generator=g).to(dt)
    gamma = torch.rand(C, generator=g) + 0.5
    beta = torch.randn(C, generator=g) * 0.1
    return x, dy, gamma, beta


def check_in(x, dy, gamma, beta, eps, channel_first):
    dtype = T.dtype_name(x)
    fmt = "NC..." if channel_first else "N...C"
    N = x.shape[0]
    C = x.shape[1] if channel_first else x.shape[-1]
    D = x.numel() // (N * C)
    s3 = (N, C, D) if channel_first else (N, D, C)
    y, mean, inv_std = A.fused_instance_norm_op(x.to(DEV), gamma.to(DEV), beta.to(DEV), data_format=fmt, epsilon=eps)
    dx, dgamma, dbeta = A.fused_instance_norm_grad_op(dy.to(DEV), x.to(DEV), gamma.to(DEV), mean, inv_std, data_format=fmt)
    torch.cuda.synchronize()
    assert y.shape == x.shape and dx.shape == x.shape
    assert mean.shape == (N, C) and inv_std.shape == (N, C)
    assert dgamma.shape == (C,) and dbeta.shape == (C,)
    x3, dy3 = T.to_numpy(x).reshape(s3), T.to_numpy(dy).reshape(s3)
    y64, m64, s64 = oracle.in_fwd(x3, gamma.numpy(), beta.numpy(), eps, channel_first, dtype)
    dx64, dg64, db64 = oracle.in_bwd(dy3, x3, gamma.numpy(), mean.cpu().numpy(), inv_std.cpu().numpy(), channel_first, dtype)
    report(y.reshape(s3), y64, mean, inv_std, m64, s64, dx.reshape(s3), dx64, dgamma, dg64, dbeta, db64, dtype)
    return y, mean, inv_std, dx, dgamma, dbeta


def report(y, y64, mean, inv_std, m64, s64, dx, dx64, dgamma, dg64, dbeta, db64, dtype):
    checks = {
        "y": T.activation_error(y, y64, dtype),
        "stats": T.stats_error(mean, inv_std, m64, s64),
        "dx": T.activation_error(dx, dx64, dtype),
        "dgamma": T.grad_param_error(dgamma, dg64),
        "dbeta": T.grad_param_error(dbeta, db64),
    }
    bad = {k: v[1] for k, v in checks.items() if not v[0] <= 1.0}
    assert not bad, f"outside tolerance: {bad}"
