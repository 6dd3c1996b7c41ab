"""Pure-NumPy float64 restatement of the reference's LayerNorm / InstanceNorm
forward and gradient formulas.  TEST INFRASTRUCTURE ONLY.

Forward follows the reference's CPU functors
(atex/nv_norms/cc/kernels/fused_layer_norm_op.cc:63-83,
atex/nv_norms/cc/kernels/fused_instance_norm_op.cc:85-106); backward follows the
NumPy functions in the reference's tests
(atex/nv_norms/tests/fused_layer_norm_test.py:20-62,
atex/nv_norms/tests/fused_instance_norm_test.py:21-65).

Parity status: backward is pinned against those reference functions executed in
the build container (tests/golden/); forward is restated from C++ that needs
TensorFlow to compile and is therefore "parity unpinned" against the compiled
reference.

Inputs are taken as they are (already rounded to the activation dtype) and
promoted to float64; nothing here rounds.
"""
from __future__ import annotations

import numpy as np


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    """uint16 bfloat16 bit patterns -> float32 values."""
    return (bits.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bfloat16 bit patterns, round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> 16) & np.uint32(1))
    return (rounded >> 16).astype(np.uint16)


def ln_fwd(x, gamma, beta, eps):
    """x [N, D] -> y [N, D], mean [N], inv_std [N], all float64."""
    x = np.asarray(x, dtype=np.float64)
    gamma = np.asarray(gamma, dtype=np.float64)
    beta = np.asarray(beta, dtype=np.float64)
    D = x.shape[1]
    mean = x.sum(axis=1) / D
    xc = x - mean[:, None]
    inv_std = 1.0 / np.sqrt((xc * xc).sum(axis=1) / D + eps)
    y = xc * inv_std[:, None] * gamma[None, :] + beta[None, :]
    return y, mean, inv_std


def ln_bwd(dy, x, gamma, mean, inv_std):
    """-> dx [N, D], dgamma [D], dbeta [D] (float64)."""
    dy = np.asarray(dy, dtype=np.float64)
    x = np.asarray(x, dtype=np.float64)
    gamma = np.asarray(gamma, dtype=np.float64)
    mean = np.asarray(mean, dtype=np.float64)[:, None]
    istd = np.asarray(inv_std, dtype=np.float64)[:, None]
    D = x.shape[1]
    xm = x - mean
    dgamma = (dy * xm * istd).sum(axis=0)
    dbeta = dy.sum(axis=0)
    dl_dvar = (dy * gamma * xm * (-0.5) * istd**3).sum(axis=1, keepdims=True)
    dl_dmean = (-dy * gamma * istd).sum(axis=1, keepdims=True)
    dx = dy * gamma * istd + dl_dvar * 2.0 * xm / D + dl_dmean / D
    return dx, dgamma, dbeta


def _in_view(a, channel_first):
    """[N, C, D] or [N, D, C] -> [N, C, D] float64 view/copy."""
    a = np.asarray(a, dtype=np.float64)
    return a if channel_first else np.transpose(a, (0, 2, 1))


def in_fwd(x, gamma, beta, eps, channel_first):
    """x [N, C, D] (channel_first) or [N, D, C] -> y (same layout), mean [N, C], inv_std [N, C]."""
    xv = _in_view(x, channel_first)
    gamma = np.asarray(gamma, dtype=np.float64)
    beta = np.asarray(beta, dtype=np.float64)
    D = xv.shape[2]
    mean = xv.sum(axis=2) / D
    xc = xv - mean[:, :, None]
    inv_std = 1.0 / np.sqrt((xc * xc).sum(axis=2) / D + eps)
    y = xc * inv_std[:, :, None] * gamma[None, :, None] + beta[None, :, None]
    if not channel_first:
        y = np.transpose(y, (0, 2, 1))
    return np.ascontiguousarray(y), mean, inv_std


def in_bwd(dy, x, gamma, mean, inv_std, channel_first):
    """-> dx (input layout), dgamma [C], dbeta [C] (float64)."""
    dyv = _in_view(dy, channel_first)
    xv = _in_view(x, channel_first)
    gamma = np.asarray(gamma, dtype=np.float64)[None, :, None]
    mean = np.asarray(mean, dtype=np.float64)[:, :, None]
    istd = np.asarray(inv_std, dtype=np.float64)[:, :, None]
    D = xv.shape[2]
    xm = xv - mean
    dgamma = (dyv * xm * istd).sum(axis=(0, 2))
    dbeta = dyv.sum(axis=(0, 2))
    dl_dvar = (dyv * gamma * xm * (-0.5) * istd**3).sum(axis=2, keepdims=True)
    dl_dmean = (-dyv * gamma * istd).sum(axis=2, keepdims=True)
    dx = dyv * gamma * istd + dl_dvar * 2.0 * xm / D + dl_dmean / D
    if not channel_first:
        dx = np.transpose(dx, (0, 2, 1))
    return np.ascontiguousarray(dx), dgamma, dbeta
