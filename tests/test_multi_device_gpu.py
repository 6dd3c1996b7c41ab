"""One process, several GPUs.

TensorFlow - the reference's host - drives every GPU of a node from one process and
registers one kernel object for all of them (fused_layer_norm_op.cc:465-484).  Kernel
attributes such as the opt-in to more than 48 KB of dynamic shared memory belong to one
device's context, so the library has to set them on every device it is used on, in
whatever order the devices are first seen.  The shapes below take the TMA-ring kernels
(64 ... 200 KB of shared memory) and the on-chip channels-last kernels on cuda:1 FIRST and
on cuda:0 second, and check both against the float64 oracle.
"""
import pytest
import torch

import atex_b200 as A
from atex_b200 import _lib
from atex_b200 import testing as T

pytestmark = pytest.mark.gpu


def _check_ln_on(dev, lib):
    from oracle import oracle
    w = T.scaled(T.WORKLOADS["c2"], 2048)          # bf16 [2048, 4096]: ring shapes fwd and bwd
    x, dy = T.make_activations(w)
    gamma, beta = T.make_params(w)
    xd, dyd, g, b = x.to(dev), dy.to(dev), gamma.to(dev), beta.to(dev)
    y, m, s = A.fused_layer_norm_op(xd, g, b, epsilon=w.eps)
    dx, dg, db = A.fused_layer_norm_grad_op(dyd, xd, g, m, s)
    torch.cuda.synchronize(dev)
    y64, m64, s64 = oracle.ln_fwd(T.to_numpy(x), gamma.numpy(), beta.numpy(), w.eps, w.dtype)
    dx64, dg64, db64 = oracle.ln_bwd(T.to_numpy(dy), T.to_numpy(x), gamma.numpy(), m.cpu().numpy(),
                                     s.cpu().numpy(), w.dtype)
    assert T.activation_error(y, y64, w.dtype)[0] <= 1.0
    assert T.stats_error(m, s, m64, s64)[0] <= 1.0
    assert T.activation_error(dx, dx64, w.dtype)[0] <= 1.0
    assert T.grad_param_error(dg, dg64)[0] <= 1.0
    assert T.grad_param_error(db, db64)[0] <= 1.0
    with torch.cuda.device(dev):
        assert lib.nvn_device_status() == _lib.NVN_OK


def _check_in_on(dev):
    from oracle import oracle
    g0 = torch.Generator().manual_seed(5)
    x = (torch.randn(6, 24, 24, 32, generator=g0) * 3 + 2).half()     # 36 KB items: on-chip kernels
    dy = torch.randn(6, 24, 24, 32, generator=g0).half()
    gamma, beta = torch.rand(32, generator=g0) + 0.5, torch.randn(32, generator=g0) * 0.1
    y, m, s = A.fused_instance_norm_op(x.to(dev), gamma.to(dev), beta.to(dev), data_format="N...C")
    dx, dg, db = A.fused_instance_norm_grad_op(dy.to(dev), x.to(dev), gamma.to(dev), m, s,
                                               data_format="N...C")
    torch.cuda.synchronize(dev)
    x3, dy3 = x.numpy().reshape(6, 576, 32), dy.numpy().reshape(6, 576, 32)
    y64, m64, s64 = oracle.in_fwd(x3, gamma.numpy(), beta.numpy(), 1e-3, False, "f16")
    dx64, dg64, db64 = oracle.in_bwd(dy3, x3, gamma.numpy(), m.cpu().numpy(), s.cpu().numpy(), False, "f16")
    assert T.activation_error(y.reshape(6, 576, 32), y64, "f16")[0] <= 1.0
    assert T.activation_error(dx.reshape(6, 576, 32), dx64, "f16")[0] <= 1.0
    assert T.grad_param_error(dg, dg64)[0] <= 1.0
    assert T.grad_param_error(db, db64)[0] <= 1.0


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs in one process")
def test_second_device_first_then_first_device(lib):
    for dev in (torch.device("cuda:1"), torch.device("cuda:0")):
        _check_ln_on(dev, lib)
        _check_in_on(dev)
