"""Parity of the CUDA ops (called through the public API -> C ABI) with the float64
oracle, over the shape matrix of the reference's own tests
(atex/nv_norms/tests/fused_layer_norm_test.py:115-179,
atex/nv_norms/tests/fused_instance_norm_test.py:143-214) and the edge cases around them.

Tolerances (atex_b200.testing): y / dx max-abs <= 1e-5 for fp32 and <= 2 ulp of the output
type (+ an fp32 round-off floor) for fp16 / bf16; saved statistics <= 1e-5 relative;
dgamma / dbeta <= 1e-4 relative, norm-wise.
"""
import os

import numpy as np
import pytest
import torch

import atex_b200 as A
from atex_b200 import _lib
from atex_b200 import testing as T

from _gpu_util import DEV, check_in, check_ln, rand_in, rand_ln

pytestmark = pytest.mark.gpu

DTYPES = ["f32", "f16", "bf16"]


@pytest.fixture(scope="module", autouse=True)
def _need_cuda(lib):
    assert torch.cuda.is_available(), "these tests need a CUDA device"


# D = 2^{4,8,10,15,18,19} x batch {1,2,5,8}: every width class of the dispatcher
# (sub-warp, warp, CTA, cluster, two-phase)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,D", [(1, 16), (5, 256), (8, 1024), (2, 32768), (5, 262144), (2, 524288),
                                 (3, 4096), (2, 8192), (2, 65536), (2, 2048)])
def test_layer_norm_typical_shapes(dtype, N, D):
    x, dy, g, b = rand_ln(N, D, dtype, seed=N * 7 + D)
    check_ln(x, dy, g, b, 1e-3)


# odd / non-vectorisable / wide (fused_layer_norm_test.py:130-139)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [11, 12, 31, 2003, 4001, 5002, 2 ** 14 + 1, 2 ** 16 + 2, 2 ** 18 + 3])
def test_layer_norm_non_typical_widths(dtype, D):
    x, dy, g, b = rand_ln(2, D, dtype, seed=D)
    check_ln(x, dy, g, b, 1e-3)


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_layer_norm_many_rows_multi_axis(dtype):
    # "brittle" 4-D shapes, axis = [1, 2, 3] (fused_layer_norm_test.py:141-151)
    for shape in [(12000, 128, 1, 1), (12000, 16, 4, 2), (3000, 8, 8, 8)]:
        N, D = shape[0], int(np.prod(shape[1:]))
        x, dy, g, b = rand_ln(N, D, dtype, seed=N + D)
        check_ln(x, dy, g.reshape(shape[1:]), b.reshape(shape[1:]), 1e-3, axis=(1, 2, 3), shape=shape)


def test_layer_norm_rank3_and_axis_variants():
    x, dy, g, b = rand_ln(6, 20, "f32", seed=3)
    for axis in ([1, 2], [-2, -1], [1, -1], [-2, 2]):
        check_ln(x, dy, g.reshape(4, 5), b.reshape(4, 5), 1e-3, axis=axis, shape=(6, 4, 5))
    x, dy, g, b = rand_ln(6 * 4, 5, "f32", seed=4)
    check_ln(x, dy, g, b, 1e-3, axis=[-1], shape=(6, 4, 5))


@pytest.mark.parametrize("dtype", DTYPES)
def test_layer_norm_large_offset_and_scale(dtype):
    # x ~ U(10, 1000) as in the reference's layer test (fused_layer_norm_test.py:186)
    g = torch.Generator().manual_seed(11)
    dt = T.TORCH_DTYPE[dtype]
    x = (torch.rand(64, 768, generator=g) * 990 + 10).to(dt)
    dy = torch.randn(64, 768, generator=g).to(dt)
    check_ln(x, dy, torch.rand(768, generator=g) + 0.5, torch.randn(768, generator=g), 1e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_golden_layer_norm_gradients(golden, dtype):
    """CUDA backward against the outputs of the reference's layer_norm_grad_np."""
    dt = T.TORCH_DTYPE[dtype]
    for k in range(int(golden["ln_count"])):
        p = f"ln{k}_"
        x = torch.from_numpy(golden[p + "x"])
        ax = [int(a) for a in golden[p + "axis"]]
        if dtype != "f32":
            continue_exact = False
        dy = torch.from_numpy(golden[p + "dy"])
        gamma = torch.from_numpy(golden[p + "gamma"])
        xs, dys = x.to(dt), dy.to(dt)
        mean = torch.from_numpy(golden[p + "mean"]).to(DEV)
        istd = torch.from_numpy(golden[p + "istd"]).to(DEV)
        dx, dg, db = A.fused_layer_norm_grad_op(dys.to(DEV), xs.to(DEV), gamma.to(DEV), mean, istd, axis=ax)
        torch.cuda.synchronize()
        if dtype == "f32":
            # identical inputs: compare straight with the reference's numbers
            assert T.activation_error(dx, golden[p + "dx"], "f32")[0] <= 1.0
            assert T.grad_param_error(dg, golden[p + "dgamma"])[0] <= 1.0
            assert T.grad_param_error(db, golden[p + "dbeta"])[0] <= 1.0
        else:
            # inputs were rounded to 16 bits: the reference numbers only bound the result loosely
            ref = golden[p + "dx"]
            tol = 0.05 * np.abs(ref).max() + 1e-3
            assert np.abs(T.to_float64(dx) - ref).max() <= tol


@pytest.mark.parametrize("dtype", DTYPES)
def test_golden_instance_norm_gradients(golden, dtype):
    dt = T.TORCH_DTYPE[dtype]
    for k in range(int(golden["in_count"])):
        p = f"in{k}_"
        cf = bool(golden[p + "cf"])
        fmt = "NC..." if cf else "N...C"
        x = torch.from_numpy(golden[p + "x"]).to(dt)
        dy = torch.from_numpy(golden[p + "dy"]).to(dt)
        gamma = torch.from_numpy(golden[p + "gamma"])
        mean = torch.from_numpy(golden[p + "mean"]).to(DEV)
        istd = torch.from_numpy(golden[p + "istd"]).to(DEV)
        dx, dg, db = A.fused_instance_norm_grad_op(dy.to(DEV), x.to(DEV), gamma.to(DEV), mean, istd, data_format=fmt)
        torch.cuda.synchronize()
        ref = golden[p + "dx"]
        if dtype == "f32":
            assert T.activation_error(dx, ref, "f32")[0] <= 1.0
            assert T.grad_param_error(dg, golden[p + "dgamma"])[0] <= 1.0
            assert T.grad_param_error(db, golden[p + "dbeta"])[0] <= 1.0
        else:
            assert np.abs(T.to_float64(dx) - ref).max() <= 0.05 * np.abs(ref).max() + 1e-3


# axis {1,-1} x rank {4,5} x D = 2^{3..6} per spatial dim (fused_instance_norm_test.py:143-155)
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channel_first", [True, False])
@pytest.mark.parametrize("spatial", [(8, 8), (16, 16), (64, 64), (8, 8, 8), (32, 32, 32), (64, 64, 64)])
def test_instance_norm_typical_shapes(dtype, channel_first, spatial):
    x, dy, g, b = rand_in(2, 32, spatial, channel_first, dtype, seed=sum(spatial))
    check_in(x, dy, g, b, 1e-3, channel_first)


# non-typical spatial extents (fused_instance_norm_test.py:157-178)
@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("channel_first", [True, False])
@pytest.mark.parametrize("spatial", [(1, 11), (3, 4), (1, 31), (1, 4001), (61, 82), (113, 145), (198, 331), (179, 2929)])
def test_instance_norm_non_typical_spatial(dtype, channel_first, spatial):
    x, dy, g, b = rand_in(2, 2, spatial, channel_first, dtype, seed=sum(spatial))
    check_in(x, dy, g, b, 1e-3, channel_first)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("channel_first", [True, False])
@pytest.mark.parametrize("N,C,spatial", [(3, 256, (16, 16)), (1, 24, (7, 9)), (5, 3, (5, 5, 5)), (2, 1, (33, 9)),
                                         (4, 520, (6, 6)), (2, 2056, (3, 3)), (7, 8, (1, 1))])
def test_instance_norm_channel_counts(dtype, channel_first, N, C, spatial):
    x, dy, g, b = rand_in(N, C, spatial, channel_first, dtype, seed=C)
    check_in(x, dy, g, b, 1e-5, channel_first)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,C,spatial,fwd_on_chip,bwd_on_chip", [
    (700, 32, (4, 4), True, True),        # small enough for a warp per item
    (700, 32, (8, 16), True, True),       # more items than resident CTAs: the persistent loop
    (5, 64, (16, 16), True, True),
    (3, 512, (8, 8), True, True),         # 64 KB items: one CTA per SM in the backward pass
    (2, 256, (32, 32), False, False),     # 512 KB (fp16) items exceed the slab
    (4, 16, (8, 8, 8), True, True),
    (2, 24, (8, 8), False, False),        # 3 channel vectors do not divide the CTA
])
def test_channels_last_items_that_fit_run_on_chip(lib, dtype, N, C, spatial, fwd_on_chip, bwd_on_chip):
    """N...C items that fit in shared memory take the one-launch on-chip kernels (bulk copy of
    the whole item, per-channel sums over the threads that share a channel vector)."""
    code = {"f32": _lib.NVN_F32, "f16": _lib.NVN_F16, "bf16": _lib.NVN_BF16}[dtype]
    D = int(np.prod(spatial))
    es = 4 if dtype == "f32" else 2
    vec = 16 // es
    fits = lambda tensors: D * C * es * tensors <= 192 * 1024
    divides = C % vec == 0 and C <= 512 and 256 % (C // vec) == 0
    small = C <= 32 and D * C <= 2048   # these go to the warp-per-item kernels instead
    for op, want, tensors in ((2, fwd_on_chip, 1), (3, bwd_on_chip, 2)):
        plan = _lib.describe_plan(op, code, N, C, D, 0)
        expect = want and divides and fits(tensors) and not small
        assert plan.startswith("nlc on-chip") == expect, (plan, expect)
        assert plan.startswith("nlc warp-per-item") == small, plan
    x, dy, g, b = rand_in(N, C, spatial, False, dtype, seed=N + C)
    check_in(x, dy, g, b, 1e-3, False)
    assert lib.nvn_device_status() == _lib.NVN_OK


@pytest.mark.parametrize("channel_first", [True, False])
@pytest.mark.parametrize("N,C,spatial", [(9000, 3, (4, 4)), (70000, 3, (2, 2)), (5000, 8, (2, 4))])
def test_instance_norm_over_many_items(lib, channel_first, N, C, spatial):
    """Thousands of batch items: the parameter-gradient reduction runs over one partial row per
    item (split into slabs when there are few channels), and the channels-last two-phase
    kernels launch in groups of at most 65535 items."""
    x, dy, g, b = rand_in(N, C, spatial, channel_first, "f16", seed=N + C)
    check_in(x, dy, g, b, 1e-3, channel_first)
    assert lib.nvn_device_status() == _lib.NVN_OK


def test_empty_inputs_launch_nothing_and_zero_the_param_grads():
    # fused_layer_norm_test.py:153-179, fused_instance_norm_test.py:181-214
    g = torch.ones(8, device=DEV)
    x = torch.zeros(0, 8, device=DEV)
    before = _lib.load().nvn_launch_count()
    y, m, s = A.fused_layer_norm_op(x, g, g)
    assert y.shape == (0, 8) and m.shape == (0,) and s.shape == (0,)
    dx, dg, db = A.fused_layer_norm_grad_op(x, x, g, m, s)
    torch.cuda.synchronize()
    assert _lib.load().nvn_launch_count() == before
    assert dx.shape == (0, 8) and torch.all(dg == 0) and torch.all(db == 0)
    for fmt, shape in (("NC...", (0, 8, 4, 4)), ("N...C", (0, 4, 4, 8)), ("NC...", (2, 8, 0, 4))):
        xi = torch.zeros(shape, device=DEV, dtype=torch.float16)
        y, m, s = A.fused_instance_norm_op(xi, g, g, data_format=fmt)
        assert y.shape == shape and m.shape == (shape[0], 8)
        dx, dg, db = A.fused_instance_norm_grad_op(xi, xi, g, m, s, data_format=fmt)
        torch.cuda.synchronize()
        assert dx.shape == shape and torch.all(dg == 0) and torch.all(db == 0)


@pytest.mark.parametrize("case", ["ln_cta", "ln_cluster", "ln_twophase", "in_nc", "in_nlc"])
def test_in_place_forward_matches_out_of_place(case):
    if case.startswith("ln"):
        D = {"ln_cta": 4096, "ln_cluster": 65536, "ln_twophase": 2 ** 20}[case]
        x, _, g, b = rand_ln(3, D, "bf16", seed=5)
        xd = x.to(DEV)
        y0, m0, s0 = A.fused_layer_norm_op(xd, g.to(DEV), b.to(DEV))
        buf = xd.clone()
        y1, m1, s1 = A.fused_layer_norm_op(buf, g.to(DEV), b.to(DEV), out=buf)
    else:
        cf = case == "in_nc"
        x, _, g, b = rand_in(2, 16, (24, 24), cf, "f16", seed=6)
        fmt = "NC..." if cf else "N...C"
        xd = x.to(DEV)
        y0, m0, s0 = A.fused_instance_norm_op(xd, g.to(DEV), b.to(DEV), data_format=fmt)
        buf = xd.clone()
        y1, m1, s1 = A.fused_instance_norm_op(buf, g.to(DEV), b.to(DEV), data_format=fmt, out=buf)
    torch.cuda.synchronize()
    assert y1.data_ptr() == buf.data_ptr()
    assert torch.equal(y0, y1) and torch.equal(m0, m1) and torch.equal(s0, s1)


@pytest.mark.parametrize("dtype", DTYPES)
def test_results_are_bitwise_repeatable(dtype):
    """Two runs give identical bits: the dgamma/dbeta reduction order is fixed, and a
    shared-memory race would show up as run-to-run differences."""
    for (N, D) in [(4099, 128), (700, 4096), (64, 65536), (3, 2 ** 20)]:
        x, dy, g, b = rand_ln(N, D, dtype, seed=N)
        xd, dyd, gd, bd = x.to(DEV), dy.to(DEV), g.to(DEV), b.to(DEV)
        outs = []
        for _ in range(2):
            y, m, s = A.fused_layer_norm_op(xd, gd, bd)
            dx, dg, db = A.fused_layer_norm_grad_op(dyd, xd, gd, m, s)
            outs.append((y, m, s, dx, dg, db))
        torch.cuda.synchronize()
        for a, c in zip(*outs):
            assert torch.equal(a, c)
    for cf in (True, False):
        x, dy, g, b = rand_in(3, 32, (40, 40), cf, dtype, seed=9)
        fmt = "NC..." if cf else "N...C"
        xd, dyd, gd, bd = x.to(DEV), dy.to(DEV), g.to(DEV), b.to(DEV)
        outs = []
        for _ in range(2):
            y, m, s = A.fused_instance_norm_op(xd, gd, bd, data_format=fmt)
            dx, dg, db = A.fused_instance_norm_grad_op(dyd, xd, gd, m, s, data_format=fmt)
            outs.append((y, m, s, dx, dg, db))
        torch.cuda.synchronize()
        for a, c in zip(*outs):
            assert torch.equal(a, c)


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_misaligned_buffers_take_the_scalar_path_and_stay_correct(dtype):
    """Views that start one element into an allocation are only element-aligned; canaries
    around the outputs catch any vector store that ignores that."""
    dt = T.TORCH_DTYPE[dtype]
    N, D = 37, 1024
    x, dy, g, b = rand_ln(N, D, dtype, seed=21)
    big = torch.full((N * D + 2,), 7.0, device=DEV, dtype=dt)
    xv = big[1:1 + N * D].view(N, D)
    xv.copy_(x.to(DEV))
    assert xv.data_ptr() % 16 != 0
    outbuf = torch.full((N * D + 2,), -3.0, device=DEV, dtype=dt)
    yv = outbuf[1:1 + N * D].view(N, D)
    y, m, s = A.fused_layer_norm_op(xv, g.to(DEV), b.to(DEV), out=yv)
    y_ref, m_ref, s_ref = A.fused_layer_norm_op(x.to(DEV), g.to(DEV), b.to(DEV))
    torch.cuda.synchronize()
    assert outbuf[0].item() == -3.0 and outbuf[-1].item() == -3.0
    assert T.activation_error(y, T.to_float64(y_ref), dtype)[0] <= 1.0
    # misaligned gamma / beta
    gb = torch.zeros(2 * D + 2, device=DEV)
    gv, bv = gb[1:1 + D], gb[D + 1:2 * D + 1]
    gv.copy_(g.to(DEV))
    bv.copy_(b.to(DEV))
    y2, _, _ = A.fused_layer_norm_op(x.to(DEV), gv, bv)
    dx2, dg2, db2 = A.fused_layer_norm_grad_op(dy.to(DEV), x.to(DEV), gv, m_ref, s_ref)
    dx1, dg1, db1 = A.fused_layer_norm_grad_op(dy.to(DEV), x.to(DEV), g.to(DEV), m_ref, s_ref)
    torch.cuda.synchronize()
    assert T.activation_error(y2, T.to_float64(y_ref), dtype)[0] <= 1.0
    assert T.activation_error(dx2, T.to_float64(dx1), dtype)[0] <= 1.0
    assert T.grad_param_error(dg2, T.to_float64(dg1))[0] <= 1.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,D", [(300, 100), (1000, 12), (64, 1028), (9, 36868), (257, 50), (33, 1026),
                                 (5, 6), (3, 70002)])
def test_widths_that_only_allow_narrower_accesses(dtype, N, D):
    """Widths that are a multiple of half or a quarter of the 128-bit vector, but not of the
    vector itself, run with 64- / 32-bit accesses instead of element by element."""
    code = {"f32": _lib.NVN_F32, "f16": _lib.NVN_F16, "bf16": _lib.NVN_BF16}[dtype]
    full = 4 if dtype == "f32" else 8
    want = next((e for e in (full, full // 2, full // 4) if e >= 2 and D % e == 0), 1)
    for op in (0, 1):
        plan = _lib.describe_plan(op, code, N, 1, D, 0)
        assert f"epv={want} " in plan, plan
    x, dy, g, b = rand_ln(N, D, dtype, seed=N + D)
    check_ln(x, dy, g, b, 1e-3)


@pytest.mark.parametrize("dtype", ["f16", "f32"])
def test_half_aligned_buffers_use_half_width_accesses_and_stay_in_bounds(dtype):
    """Buffers aligned to 8 bytes only: canaries catch a 16-byte store that ignores it."""
    dt = T.TORCH_DTYPE[dtype]
    N, D = 53, 512
    shift = 8 // torch.empty((), dtype=dt).element_size()
    x, dy, g, b = rand_ln(N, D, dtype, seed=5)
    big = torch.full((N * D + 2 * shift,), 7.0, device=DEV, dtype=dt)
    xv = big[shift:shift + N * D].view(N, D)
    xv.copy_(x.to(DEV))
    assert xv.data_ptr() % 16 == 8
    outbuf = torch.full((N * D + 2 * shift,), -3.0, device=DEV, dtype=dt)
    yv = outbuf[shift:shift + N * D].view(N, D)
    y, m, s = A.fused_layer_norm_op(xv, g.to(DEV), b.to(DEV), out=yv)
    y_ref, m_ref, s_ref = A.fused_layer_norm_op(x.to(DEV), g.to(DEV), b.to(DEV))
    dx, dg, db = A.fused_layer_norm_grad_op(dy.to(DEV), xv, g.to(DEV), m_ref, s_ref)
    dx1, dg1, db1 = A.fused_layer_norm_grad_op(dy.to(DEV), x.to(DEV), g.to(DEV), m_ref, s_ref)
    torch.cuda.synchronize()
    assert (outbuf[:shift] == -3.0).all().item() and (outbuf[-shift:] == -3.0).all().item()
    assert T.activation_error(y, T.to_float64(y_ref), dtype)[0] <= 1.0
    assert T.activation_error(dx, T.to_float64(dx1), dtype)[0] <= 1.0
    assert T.grad_param_error(dg, T.to_float64(dg1))[0] <= 1.0
    assert T.grad_param_error(db, T.to_float64(db1))[0] <= 1.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,D", [(300, 32768), (70, 33000), (129, 65536), (33, 98304), (1, 40000),
                                 (75, 16384), (9, 131072)])
def test_wide_rows(lib, dtype, N, D):
    """Rows that a single CTA cannot hold: cluster shapes whose CTAs meet over distributed
    shared memory (widths that fill a shape), two-phase kernels otherwise.  Row counts that
    do not fill the last wave of clusters and the bounded waits (device status word) are
    covered here."""
    x, dy, g, b = rand_ln(N, D, dtype, seed=N + D)
    check_ln(x, dy, g, b, 1e-3)
    assert lib.nvn_device_status() == _lib.NVN_OK


def test_backward_uses_the_statistics_it_is_given():
    """The gradient op must consume the passed-in mean / inverse std, not recompute them
    (the reference's tests feed statistics computed elsewhere, fused_layer_norm_test.py:97-108)."""
    x, dy, g, b = rand_ln(16, 512, "f32", seed=2)
    xd, dyd, gd = x.to(DEV), dy.to(DEV), g.to(DEV)
    fake_mean = torch.full((16,), 0.25, device=DEV)
    fake_istd = torch.full((16,), 2.0, device=DEV)
    dx, dg, db = A.fused_layer_norm_grad_op(dyd, xd, gd, fake_mean, fake_istd)
    torch.cuda.synchronize()
    from oracle import oracle
    dx64, dg64, db64 = oracle.ln_bwd(dy.numpy(), x.numpy(), g.numpy(), fake_mean.cpu().numpy(), fake_istd.cpu().numpy(), "f32")
    assert T.activation_error(dx, dx64, "f32")[0] <= 1.0
    assert T.grad_param_error(dg, dg64)[0] <= 1.0


def test_autograd_wrappers_and_layers():
    """Layer-level check: gradients through the wrapper layers equal the raw gradient op,
    and agree with PyTorch's own composite ops in fp32."""
    torch.manual_seed(0)
    x = torch.randn(6, 5, 64, device=DEV, requires_grad=True)
    layer = A.LayerNormalization(axis=[1, 2], epsilon=1e-3)
    y = layer(x)
    w = torch.randn_like(y)
    (y * w).sum().backward()
    ref_x = x.detach().clone().requires_grad_(True)
    gam = layer.gamma.detach().clone().requires_grad_(True)
    bet = layer.beta.detach().clone().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(ref_x, (5, 64), gam, bet, eps=1e-3)
    (yr * w).sum().backward()
    assert torch.allclose(y, yr, atol=1e-5)
    assert torch.allclose(x.grad, ref_x.grad, atol=1e-5)
    assert torch.allclose(layer.gamma.grad, gam.grad, rtol=1e-4, atol=1e-4)
    assert torch.allclose(layer.beta.grad, bet.grad, rtol=1e-4, atol=1e-4)

    for axis, shape in ((1, (3, 8, 10, 10)), (-1, (3, 10, 10, 8))):
        xi = torch.randn(shape, device=DEV, requires_grad=True)
        inn = A.InstanceNormalization(axis=axis, epsilon=1e-3)
        yi = inn(xi)
        wi = torch.randn_like(yi)
        (yi * wi).sum().backward()
        xr = xi.detach().clone().requires_grad_(True)
        xr_cf = xr if axis == 1 else xr.permute(0, 3, 1, 2)
        gi = inn.gamma.detach().clone().requires_grad_(True)
        bi = inn.beta.detach().clone().requires_grad_(True)
        yr = torch.nn.functional.instance_norm(xr_cf, weight=gi, bias=bi, eps=1e-3)
        yr = yr if axis == 1 else yr.permute(0, 2, 3, 1)
        (yr * wi).sum().backward()
        assert torch.allclose(yi, yr, atol=1e-5)
        assert torch.allclose(xi.grad, xr.grad, atol=1e-5)
        assert torch.allclose(inn.gamma.grad, gi.grad, rtol=1e-4, atol=1e-4)


def test_mixed_precision_layer_keeps_fp32_weights():
    xi = torch.randn(2, 12, 12, 16, device=DEV, dtype=torch.float16)
    inn = A.InstanceNormalization(axis=-1)
    y = inn(xi)
    assert y.dtype == torch.float16 and inn.gamma.dtype == torch.float32


def test_tma_ring_path_is_used_and_no_bounded_wait_ever_gave_up(lib):
    """The benchmark shape runs its forward through the cp.async.bulk ring; its waits are
    bounded and report through the device status word, which must still be clean after
    everything this process has launched so far."""
    plan = _lib.describe_plan(0, _lib.NVN_BF16, 32768, 1, 4096, 0)
    assert "load=tma" in plan, plan
    for (N, D, dtype) in [(3001, 4096, "bf16"), (70000, 128, "f16"), (513, 1024, "f32"), (37, 3072, "bf16")]:
        x, dy, g, b = rand_ln(N, D, dtype, seed=N)
        check_ln(x, dy, g, b, 1e-5)
    assert lib.nvn_device_status() == _lib.NVN_OK
