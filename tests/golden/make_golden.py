"""Generates tests/golden/*.npz by executing the reference's own NumPy gradient
functions on seeded inputs.

The reference's tests define ``layer_norm_grad_np``
(atex/nv_norms/tests/fused_layer_norm_test.py:20-62) and ``instance_norm_grad_np``
(atex/nv_norms/tests/fused_instance_norm_test.py:21-65) as the expected values of
its fused gradient ops.  The test modules import TensorFlow at the top, which is
not installed, so the two function definitions are pulled out of the source with
``ast`` and executed with NumPy alone; nothing is copied into this repository.

Run from the repository root, giving the path of a checkout of the reference:

    python tests/golden/make_golden.py <path-to-atex-checkout>

Shapes are taken from the reference's test matrix (typical, odd, rank-3/4 inputs,
both InstanceNorm layouts).  The saved statistics fed to the gradient functions are
float32 roundings of float64 moments of the inputs, which is what a forward op
would have saved.
"""
from __future__ import annotations

import ast
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def extract_function(path: str, name: str):
    with open(path) as f:
        tree = ast.parse(f.read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == name:
            mod = ast.Module(body=[node], type_ignores=[])
            ns = {"np": np}
            exec(compile(mod, path, "exec"), ns)
            return ns[name]
    raise KeyError(name)


class _TensorLike:
    """Stands in for the tf.Tensor entries of the LayerNorm test's cache dict."""

    def __init__(self, a):
        self._a = a

    def numpy(self):
        return self._a


def moments64(x64, axes, eps):
    mean = x64.mean(axis=axes)
    var = x64.var(axis=axes)
    return mean.astype(np.float32), (1.0 / np.sqrt(var + eps)).astype(np.float32)


def main(ref_root: str) -> None:
    ln_grad = extract_function(
        os.path.join(ref_root, "atex/nv_norms/tests/fused_layer_norm_test.py"), "layer_norm_grad_np")
    in_grad = extract_function(
        os.path.join(ref_root, "atex/nv_norms/tests/fused_instance_norm_test.py"), "instance_norm_grad_np")

    rng = np.random.default_rng(20221)
    out = {}
    # LayerNorm: (x_shape, axis) from testFusedLayerNormOp / NonTypical / Brittle shape lists
    ln_cases = [
        ((2, 16), (1,)), ((5, 256), (1,)), ((4, 1024), (-1,)), ((2, 11), (1,)), ((2, 31), (1,)),
        ((2, 2003), (1,)), ((2, 3, 16), (2,)), ((12, 4, 2, 2), (1, 2, 3)), ((1, 4001), (1,)),
    ]
    for k, (shape, axis) in enumerate(ln_cases):
        eps = 1e-3
        x = rng.normal(scale=10.0, size=shape).astype(np.float32)
        dy = rng.normal(size=shape).astype(np.float32)
        ax = tuple(sorted(a % len(shape) for a in axis))
        gshape = tuple(shape[a] for a in ax)
        gamma = rng.normal(size=gshape).astype(np.float32)
        mean, istd = moments64(x.astype(np.float64), ax, eps)
        # float32-rounded statistics, promoted so the reference function works in float64
        cache = {"mean": _TensorLike(mean.reshape(-1).astype(np.float64)),
                 "istd": _TensorLike(istd.reshape(-1).astype(np.float64))}
        dgamma, dbeta, dx = ln_grad(x.astype(np.float64), dy.astype(np.float64),
                                    gamma.astype(np.float64), cache, ax)
        p = f"ln{k}_"
        out.update({p + "x": x, p + "dy": dy, p + "gamma": gamma, p + "axis": np.array(ax),
                    p + "mean": mean.reshape(-1), p + "istd": istd.reshape(-1),
                    p + "dx": dx, p + "dgamma": dgamma, p + "dbeta": dbeta})
    out["ln_count"] = np.array(len(ln_cases))

    # InstanceNorm: (N, C, spatial dims, channel_first)
    in_cases = [
        (2, 32, (8, 8), True), (2, 32, (8, 8), False), (2, 32, (4, 4, 4), True),
        (2, 32, (4, 4, 4), False), (2, 3, (1, 11), True), (2, 3, (1, 11), False),
        (2, 5, (3, 4), False), (1, 3, (61, 82), True), (1, 8, (1, 31), False),
    ]
    for k, (N, C, sp, cf) in enumerate(in_cases):
        eps = 1e-3
        shape = (N, C) + sp if cf else (N,) + sp + (C,)
        x = rng.normal(loc=1.0, scale=3.0, size=shape).astype(np.float32)
        dy = rng.normal(size=shape).astype(np.float32)
        gamma = rng.normal(size=(C,)).astype(np.float32)
        sp_axes = tuple(range(2, len(shape))) if cf else tuple(range(1, len(shape) - 1))
        mean, istd = moments64(x.astype(np.float64), sp_axes, eps)  # [N, C]
        cache = {"mean": mean.astype(np.float64), "istd": istd.astype(np.float64)}
        dgamma, dbeta, dx = in_grad(x.astype(np.float64), dy.astype(np.float64),
                                    gamma.astype(np.float64), cache, cf)
        p = f"in{k}_"
        out.update({p + "x": x, p + "dy": dy, p + "gamma": gamma, p + "cf": np.array(cf),
                    p + "mean": mean, p + "istd": istd, p + "dx": dx, p + "dgamma": dgamma,
                    p + "dbeta": dbeta})
    out["in_count"] = np.array(len(in_cases))
    np.savez_compressed(os.path.join(HERE, "reference_grads.npz"), **out)
    print("wrote", os.path.join(HERE, "reference_grads.npz"), len(out), "arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <path-to-atex-checkout>")
    main(sys.argv[1])
