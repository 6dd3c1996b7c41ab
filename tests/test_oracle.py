"""The oracle against the reference's own expected values, and against itself.

tests/golden/reference_grads.npz holds outputs of the reference's NumPy gradient
functions (layer_norm_grad_np, instance_norm_grad_np) executed on seeded inputs by
tests/golden/make_golden.py.  Both restatements of the oracle (NumPy float64 and C)
must reproduce them, which pins the backward formulas to the reference.
"""
import numpy as np
import pytest

from oracle import oracle, oracle_np


def _ln_case(golden, k):
    p = f"ln{k}_"
    x, dy, gamma = golden[p + "x"], golden[p + "dy"], golden[p + "gamma"]
    ax = tuple(int(a) for a in golden[p + "axis"])
    D = int(np.prod([x.shape[a] for a in ax]))
    N = x.size // D
    return p, x.reshape(N, D), dy.reshape(N, D), gamma.reshape(D), N, D


def test_numpy_oracle_reproduces_reference_layer_norm_grads(golden):
    for k in range(int(golden["ln_count"])):
        p, x, dy, gamma, N, D = _ln_case(golden, k)
        dx, dg, db = oracle_np.ln_bwd(dy, x, gamma, golden[p + "mean"], golden[p + "istd"])
        np.testing.assert_allclose(dx, golden[p + "dx"].reshape(N, D), rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(dg, golden[p + "dgamma"].reshape(D), rtol=1e-12, atol=1e-12)
        np.testing.assert_allclose(db, golden[p + "dbeta"].reshape(D), rtol=1e-12, atol=1e-12)


def test_c_oracle_reproduces_reference_layer_norm_grads(golden):
    for k in range(int(golden["ln_count"])):
        p, x, dy, gamma, N, D = _ln_case(golden, k)
        dx, dg, db = oracle.ln_bwd(dy, x, gamma, golden[p + "mean"], golden[p + "istd"], "f32")
        np.testing.assert_allclose(dx, golden[p + "dx"].reshape(N, D), rtol=1e-11, atol=1e-11)
        np.testing.assert_allclose(dg, golden[p + "dgamma"].reshape(D), rtol=1e-11, atol=1e-11)
        np.testing.assert_allclose(db, golden[p + "dbeta"].reshape(D), rtol=1e-11, atol=1e-11)


def _in_case(golden, k):
    p = f"in{k}_"
    x, dy, gamma = golden[p + "x"], golden[p + "dy"], golden[p + "gamma"]
    cf = bool(golden[p + "cf"])
    N = x.shape[0]
    C = x.shape[1] if cf else x.shape[-1]
    D = x.size // (N * C)
    shape3 = (N, C, D) if cf else (N, D, C)
    return p, x.reshape(shape3), dy.reshape(shape3), gamma, cf, shape3


@pytest.mark.parametrize("impl", ["numpy", "c"])
def test_oracle_reproduces_reference_instance_norm_grads(golden, impl):
    # the reference accumulates its sums in float32 (dtype=np.float32), hence 1e-5
    for k in range(int(golden["in_count"])):
        p, x, dy, gamma, cf, shape3 = _in_case(golden, k)
        if impl == "numpy":
            dx, dg, db = oracle_np.in_bwd(dy, x, gamma, golden[p + "mean"], golden[p + "istd"], cf)
        else:
            dx, dg, db = oracle.in_bwd(dy, x, gamma, golden[p + "mean"], golden[p + "istd"], cf, "f32")
        scale = np.abs(golden[p + "dx"]).max()
        np.testing.assert_allclose(dx, golden[p + "dx"].reshape(shape3), rtol=0, atol=2e-6 * scale)
        np.testing.assert_allclose(dg, golden[p + "dgamma"], rtol=2e-5, atol=2e-5 * np.abs(dg).max())
        np.testing.assert_allclose(db, golden[p + "dbeta"], rtol=2e-5, atol=2e-5 * np.abs(db).max())


def test_forward_statistics_match_the_saved_ones_in_the_fixtures(golden):
    # The fixtures' mean / istd are float64 moments rounded to float32: the oracle's
    # forward must agree with them to float32 rounding.
    for k in range(int(golden["ln_count"])):
        p, x, dy, gamma, N, D = _ln_case(golden, k)
        _, mean, istd = oracle_np.ln_fwd(x, gamma, np.zeros(D), 1e-3)
        np.testing.assert_allclose(mean, golden[p + "mean"], rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(istd, golden[p + "istd"], rtol=1e-6)
    for k in range(int(golden["in_count"])):
        p, x, dy, gamma, cf, shape3 = _in_case(golden, k)
        _, mean, istd = oracle.in_fwd(x, gamma, np.zeros_like(gamma), 1e-3, cf, "f32")
        np.testing.assert_allclose(mean, golden[p + "mean"], rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(istd, golden[p + "istd"], rtol=1e-6)


@pytest.mark.parametrize("dtype", ["f32", "f16", "bf16"])
def test_c_and_numpy_oracles_agree(dtype):
    rng = np.random.default_rng(7)

    def act(shape):
        a = rng.normal(loc=1.0, scale=3.0, size=shape).astype(np.float32)
        if dtype == "f16":
            return a.astype(np.float16), a.astype(np.float16).astype(np.float64)
        if dtype == "bf16":
            bits = oracle_np.f32_to_bf16_bits(a)
            return bits, oracle_np.bf16_bits_to_f32(bits).astype(np.float64)
        return a, a.astype(np.float64)

    x, x64 = act((6, 37))
    dy, dy64 = act((6, 37))
    g = rng.normal(size=37).astype(np.float32)
    b = rng.normal(size=37).astype(np.float32)
    y, m, s = oracle.ln_fwd(x, g, b, 1e-5, dtype)
    y2, m2, s2 = oracle_np.ln_fwd(x64, g, b, 1e-5)
    np.testing.assert_allclose(y, y2, rtol=1e-12, atol=1e-12)
    np.testing.assert_allclose(s, s2, rtol=1e-13)
    m32, s32 = m.astype(np.float32), s.astype(np.float32)
    dx, dg, db = oracle.ln_bwd(dy, x, g, m32, s32, dtype)
    dx2, dg2, db2 = oracle_np.ln_bwd(dy64, x64, g, m32, s32)
    np.testing.assert_allclose(dx, dx2, rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(dg, dg2, rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(db, db2, rtol=1e-11, atol=1e-12)
    for cf in (True, False):
        shape = (3, 5, 23) if cf else (3, 23, 5)
        x, x64 = act(shape)
        dy, dy64 = act(shape)
        g = rng.normal(size=5).astype(np.float32)
        b = rng.normal(size=5).astype(np.float32)
        y, m, s = oracle.in_fwd(x, g, b, 1e-3, cf, dtype)
        y2, m2, s2 = oracle_np.in_fwd(x64, g, b, 1e-3, cf)
        np.testing.assert_allclose(y, y2, rtol=1e-12, atol=1e-12)
        m32, s32 = m.astype(np.float32), s.astype(np.float32)
        dx, dg, db = oracle.in_bwd(dy, x, g, m32, s32, cf, dtype)
        dx2, dg2, db2 = oracle_np.in_bwd(dy64, x64, g, m32, s32, cf)
        np.testing.assert_allclose(dx, dx2, rtol=1e-11, atol=1e-12)
        np.testing.assert_allclose(dg, dg2, rtol=1e-11, atol=1e-12)
        np.testing.assert_allclose(db, db2, rtol=1e-11, atol=1e-12)


def test_fp32_port_is_close_to_the_float64_checker():
    rng = np.random.default_rng(3)
    x = rng.normal(size=(9, 64)).astype(np.float16)
    g = rng.normal(size=64).astype(np.float32)
    b = rng.normal(size=64).astype(np.float32)
    y64, m64, s64 = oracle.ln_fwd(x, g, b, 1e-3, "f16")
    y16, m32, s32 = oracle.ln_fwd(x, g, b, 1e-3, "f16", fp32_port=True)
    assert y16.dtype == np.float16
    np.testing.assert_allclose(y16.astype(np.float64), y64, rtol=2e-3, atol=2e-3)
    np.testing.assert_allclose(m32, m64, rtol=1e-5, atol=1e-6)
    np.testing.assert_allclose(s32, s64, rtol=1e-5)


def test_half_and_bfloat16_conversions_of_the_c_oracle():
    L = oracle.lib()
    h = np.arange(0, 65536, 257, dtype=np.uint16)
    ref = h.view(np.float16).astype(np.float32)
    got = np.array([L.oracle_half_to_f32(int(v)) for v in h], dtype=np.float32)
    ok = ~np.isnan(ref)
    assert np.array_equal(ref.view(np.uint32)[ok], got.view(np.uint32)[ok])
    rng = np.random.default_rng(1)
    f = (rng.normal(size=4000) * 10.0 ** rng.integers(-9, 6, size=4000)).astype(np.float32)
    with np.errstate(over="ignore"):
        ref16 = f.astype(np.float16).view(np.uint16)
    got16 = np.array([L.oracle_f32_to_half(float(v)) for v in f], dtype=np.uint16)
    assert np.array_equal(got16, ref16)
    gotb = np.array([L.oracle_f32_to_bf16(float(v)) for v in f], dtype=np.uint16)
    assert np.array_equal(gotb, oracle_np.f32_to_bf16_bits(f))
