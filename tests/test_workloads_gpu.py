"""The seven benchmark configurations at full size on the GPU.

Where the float64 oracle finishes in seconds on the host the whole tensor is compared;
for the two largest InstanceNorm workloads y / dx are compared on the first and last batch
items while the statistics and dgamma / dbeta are compared over everything.  On top of
that, size-independent properties of the operators are checked on the full outputs.
"""
import numpy as np
import pytest
import torch

import atex_b200 as A
from atex_b200 import testing as T
from oracle import oracle

from _gpu_util import DEV, report

pytestmark = pytest.mark.gpu


def _run(w, x, dy, gamma, beta):
    xd, dyd, gd, bd = x.to(DEV), dy.to(DEV), gamma.to(DEV), beta.to(DEV)
    if w.op == "ln":
        y, m, s = A.fused_layer_norm_op(xd, gd, bd, epsilon=w.eps)
        dx, dg, db = A.fused_layer_norm_grad_op(dyd, xd, gd, m, s)
    else:
        y, m, s = A.fused_instance_norm_op(xd, gd, bd, data_format=w.data_format, epsilon=w.eps)
        dx, dg, db = A.fused_instance_norm_grad_op(dyd, xd, gd, m, s, data_format=w.data_format)
    torch.cuda.synchronize()
    return y, m, s, dx, dg, db


@pytest.mark.parametrize("name", ["c1", "c2", "c3a", "c3b", "c3c"])
def test_layer_norm_workloads_full_size(name):
    w = T.WORKLOADS[name]
    x, dy = T.make_activations(w)
    gamma, beta = T.make_params(w)
    y, m, s, dx, dg, db = _run(w, x, dy, gamma, beta)
    y64, m64, s64 = oracle.ln_fwd(T.to_numpy(x), gamma.numpy(), beta.numpy(), w.eps, w.dtype)
    dx64, dg64, db64 = oracle.ln_bwd(T.to_numpy(dy), T.to_numpy(x), gamma.numpy(), m.cpu().numpy(),
                                     s.cpu().numpy(), w.dtype)
    report(y, y64, m, s, m64, s64, dx, dx64, dg, dg64, db, db64, w.dtype)
    # size-independent property, in fp64 on the device outputs: every dx row sums to zero
    # (the gradient has no component along the direction the mean removes), up to output
    # rounding
    dxd = dx.double()
    row_scale = dxd.abs().sum(dim=1).clamp_min(1e-30)
    tol = {"f32": 1e-5, "f16": 2e-3, "bf16": 1.6e-2}[w.dtype]
    assert float((dxd.sum(dim=1).abs() / row_scale).max()) < tol
    # and y is an affine image of a zero-mean, (almost) unit-variance row
    g64, b64 = gamma.to(DEV).double(), beta.to(DEV).double()
    z = (y.double() - b64) / g64
    assert float(z.mean(dim=1).abs().max()) < tol * 4
    assert float((z.var(dim=1, unbiased=False) - 1).abs().max()) < max(tol * 8, 2 * w.eps * float(s.max()) ** 2 + tol)


@pytest.mark.parametrize("name", ["c4", "c5"])
def test_instance_norm_workloads_full_size(name):
    w = T.WORKLOADS[name]
    x, dy = T.make_activations(w)
    gamma, beta = T.make_params(w)
    y, m, s, dx, dg, db = _run(w, x, dy, gamma, beta)
    cf = w.channel_first
    s3 = (w.N, w.C, w.D) if cf else (w.N, w.D, w.C)
    x3, dy3 = T.to_numpy(x).reshape(s3), T.to_numpy(dy).reshape(s3)
    # statistics and parameter gradients over the whole batch (no y / dx materialised)
    _, m64, s64 = oracle.in_fwd(x3, gamma.numpy(), beta.numpy(), w.eps, cf, w.dtype, want_y=False)
    _, dg64, db64 = oracle.in_bwd(dy3, x3, gamma.numpy(), m.cpu().numpy(), s.cpu().numpy(), cf, w.dtype, want_dx=False)
    assert T.stats_error(m, s, m64, s64)[0] <= 1.0, T.stats_error(m, s, m64, s64)[1]
    assert T.grad_param_error(dg, dg64)[0] <= 1.0, T.grad_param_error(dg, dg64)[1]
    assert T.grad_param_error(db, db64)[0] <= 1.0, T.grad_param_error(db, db64)[1]
    # y / dx on the first and the last batch item
    for n in (0, w.N - 1):
        y64, _, _ = oracle.in_fwd(x3[n:n + 1], gamma.numpy(), beta.numpy(), w.eps, cf, w.dtype)
        dx64, _, _ = oracle.in_bwd(dy3[n:n + 1], x3[n:n + 1], gamma.numpy(), m[n:n + 1].cpu().numpy(),
                                   s[n:n + 1].cpu().numpy(), cf, w.dtype)
        e = T.activation_error(y[n:n + 1].reshape(y64.shape), y64, w.dtype)
        assert e[0] <= 1.0, e[1]
        e = T.activation_error(dx[n:n + 1].reshape(dx64.shape), dx64, w.dtype)
        assert e[0] <= 1.0, e[1]
    # property on the full output: per (n, c) the dx values sum to ~0
    red = (2, 3) if cf else (1, 2, 3)
    dxd = dx.double()
    tol = {"f16": 2e-3, "bf16": 1.6e-2}[w.dtype]
    assert float((dxd.sum(dim=red).abs() / dxd.abs().sum(dim=red).clamp_min(1e-30)).max()) < tol


def test_sharded_backward_equals_unsharded():
    """Batch sharding is exact for y / dx and sums to the same dgamma / dbeta: emulate two
    ranks on one GPU by running the two halves of c2 one after the other."""
    w = T.scaled(T.WORKLOADS["c2"], 4096)
    x, dy = T.make_activations(w)
    gamma, beta = T.make_params(w)
    y, m, s, dx, dg, db = _run(w, x, dy, gamma, beta)
    parts = []
    from atex_b200.sharding import shard_range
    for r in range(2):
        a, b = shard_range(w.N, r, 2)
        parts.append(_run(T.scaled(w, b - a), x[a:b], dy[a:b], gamma, beta))
    assert torch.equal(torch.cat([p[0] for p in parts]), y)
    assert torch.equal(torch.cat([p[3] for p in parts]), dx)
    dg2 = parts[0][4] + parts[1][4]
    assert T.grad_param_error(dg2, T.to_float64(dg))[0] <= 1.0
