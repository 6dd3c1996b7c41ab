"""Seeded synthetic workloads and tolerance helpers shared by the tests, the
benchmark and the smoke check.

The reference benchmarks on random tensors (atex/nv_norms/benchmarks/
benchmark_layer_norm.py:39, benchmark_instance_norm.py:36-41); the workloads here
are the seven named configurations this build is measured on, generated from
NumPy ``default_rng`` streams.  Every tensor is generated in independent blocks
(a fixed number of rows, or one batch item) whose stream is keyed by
(config, tensor, block), so a rank of a sharded run generates exactly the slice
of the global tensor it owns and a 1-GPU run sees the same data.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Tuple

import numpy as np
import torch

TORCH_DTYPE = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}
ELEM_SIZE = {"f32": 4, "f16": 2, "bf16": 2}


@dataclass(frozen=True)
class Workload:
    name: str
    op: str            # "ln" or "in"
    dtype: str         # "f32" | "f16" | "bf16"
    N: int             # LayerNorm rows / InstanceNorm batch
    D: int             # reduced extent (features, or product of spatial dims)
    C: int = 1         # InstanceNorm channels
    channel_first: bool = False
    eps: float = 1e-3
    spatial: Tuple[int, ...] = ()
    x_kind: str = "normal"      # distribution of x, see _gen_x
    gamma_kind: str = "uniform"  # "uniform": U(0.5, 1.5), beta N(0, 0.1); "near_one": 1+N(0, .02), beta N(0, .02)
    index: int = 0

    @property
    def elements(self) -> int:
        return self.N * self.D * self.C

    @property
    def features(self) -> int:
        return self.D if self.op == "ln" else self.C

    @property
    def stat_rows(self) -> int:
        return self.N if self.op == "ln" else self.N * self.C

    def shape(self, n: int | None = None) -> Tuple[int, ...]:
        n = self.N if n is None else n
        if self.op == "ln":
            return (n, self.D)
        sp = self.spatial if self.spatial else (self.D,)
        return (n, self.C) + tuple(sp) if self.channel_first else (n,) + tuple(sp) + (self.C,)

    @property
    def data_format(self) -> str:
        return "NC..." if self.channel_first else "N...C"

    def algorithmic_bytes(self, n: int | None = None) -> int:
        """Minimal bytes moved by forward + backward: x read and y written, then x and dy
        read and dx written, plus parameters, their gradients and the saved statistics."""
        n = self.N if n is None else n
        E = n * self.D * self.C
        s = ELEM_SIZE[self.dtype]
        F = self.features
        R = n if self.op == "ln" else n * self.C
        fwd = 2 * E * s + 2 * F * 4 + 2 * R * 4
        bwd = 3 * E * s + 3 * F * 4 + 2 * R * 4
        return fwd + bwd


WORKLOADS: Dict[str, Workload] = {
    "c1": Workload("c1", "ln", "f32", 4096, 1024, eps=1e-3, index=1),
    "c2": Workload("c2", "ln", "bf16", 32768, 4096, eps=1e-5, x_kind="row_offset", index=2),
    "c3a": Workload("c3a", "ln", "f16", 1048576, 128, eps=1e-6, gamma_kind="near_one", index=3),
    "c3b": Workload("c3b", "ln", "f16", 65536, 1024, eps=1e-6, gamma_kind="near_one", index=4),
    "c3c": Workload("c3c", "ln", "f16", 256, 65536, eps=1e-6, gamma_kind="near_one", index=5),
    "c4": Workload("c4", "in", "f16", 8, 128 * 128 * 128, C=32, channel_first=False, eps=1e-3,
                   spatial=(128, 128, 128), x_kind="mean2_std3", index=6),
    "c5": Workload("c5", "in", "bf16", 64, 128 * 128, C=256, channel_first=True, eps=1e-5,
                   spatial=(128, 128), x_kind="channel_scale", index=7),
}

_BLOCK_ROWS = 1024  # LayerNorm rows per independently seeded block


def scaled(w: Workload, N: int) -> Workload:
    """The same workload with a different batch extent (for sharding and small tests)."""
    return Workload(w.name, w.op, w.dtype, N, w.D, w.C, w.channel_first, w.eps, w.spatial,
                    w.x_kind, w.gamma_kind, w.index)


def workload_from_spec(spec: str) -> Workload:
    """A benchmark configuration by name ("c2"), or a problem of any shape:
    "ln:N:D:dtype" or "in:N:C:S1xS2x...:dtype:nlc|nc" (dtype f32 | f16 | bf16)."""
    if spec in WORKLOADS:
        return WORKLOADS[spec]
    f = spec.split(":")
    if f[0] == "ln" and len(f) == 4:
        return Workload(spec, "ln", f[3], int(f[1]), int(f[2]), eps=1e-5, index=8)
    if f[0] == "in" and len(f) == 6:
        sp = tuple(int(v) for v in f[3].split("x"))
        return Workload(spec, "in", f[4], int(f[1]), math.prod(sp), C=int(f[2]), channel_first=(f[5] == "nc"),
                        eps=1e-3, spatial=sp, index=9)
    raise ValueError(f"unknown workload {spec!r}")


def _rng(w: Workload, tensor: int, block: int) -> np.random.Generator:
    return np.random.default_rng([1000 * w.index + tensor, block])


def make_params(w: Workload):
    """gamma, beta as float32 CPU tensors (identical on every rank)."""
    F = w.features
    rg, rb = _rng(w, 2, 0), _rng(w, 3, 0)
    if w.gamma_kind == "near_one":
        gamma = 1.0 + 0.02 * rg.standard_normal(F, dtype=np.float32)
        beta = 0.02 * rb.standard_normal(F, dtype=np.float32)
    else:
        gamma = rg.uniform(0.5, 1.5, F).astype(np.float32)
        beta = 0.1 * rb.standard_normal(F, dtype=np.float32)
    return torch.from_numpy(gamma.astype(np.float32)), torch.from_numpy(beta.astype(np.float32))


def _gen_block(w: Workload, tensor: int, block: int, shape) -> np.ndarray:
    r = _rng(w, tensor, block)
    a = r.standard_normal(shape, dtype=np.float32)
    if tensor == 0:  # x
        if w.x_kind == "row_offset":
            a *= np.float32(4.0)
            a += r.standard_normal((shape[0], 1), dtype=np.float32)
        elif w.x_kind == "mean2_std3":
            a *= np.float32(3.0)
            a += np.float32(2.0)
        elif w.x_kind == "channel_scale":
            s = _rng(w, 4, 0).uniform(0.5, 2.0, w.C).astype(np.float32)
            a *= s.reshape((1, w.C) + (1,) * (len(shape) - 2)) if w.channel_first else s
    return a


def make_activations(w: Workload, start: int = 0, stop: int | None = None, pin: bool = False):
    """x and dy for batch entries [start, stop) as CPU tensors of the workload's dtype."""
    stop = w.N if stop is None else stop
    n = stop - start
    shape = w.shape(n)
    dt = TORCH_DTYPE[w.dtype]
    out = []
    for tensor in (0, 1):
        t = torch.empty(shape, dtype=dt, pin_memory=pin)
        if w.op == "ln":
            b0 = start // _BLOCK_ROWS
            b1 = (stop + _BLOCK_ROWS - 1) // _BLOCK_ROWS
            for b in range(b0, b1):
                lo, hi = max(b * _BLOCK_ROWS, start), min((b + 1) * _BLOCK_ROWS, stop)
                blk = _gen_block(w, tensor, b, (_BLOCK_ROWS, w.D))
                t[lo - start:hi - start] = torch.from_numpy(
                    blk[lo - b * _BLOCK_ROWS:hi - b * _BLOCK_ROWS]).to(dt)
        else:
            for i in range(start, stop):
                t[i - start] = torch.from_numpy(_gen_block(w, tensor, i, w.shape(1))[0]).to(dt)
        out.append(t)
    return out[0], out[1]


# ---------------------------------------------------------------------------
# NumPy views of torch tensors for the oracle
# ---------------------------------------------------------------------------
def to_numpy(t: torch.Tensor) -> np.ndarray:
    """CPU ndarray for the oracle: float32 / float16 as such, bfloat16 as uint16 bit patterns."""
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:
        return t.view(torch.int16).numpy().view(np.uint16)
    return t.numpy()


def to_float64(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().to(torch.float64).numpy()


def dtype_name(t: torch.Tensor) -> str:
    return {torch.float32: "f32", torch.float16: "f16", torch.bfloat16: "bf16"}[t.dtype]


# ---------------------------------------------------------------------------
# tolerances
# ---------------------------------------------------------------------------
_MANT = {"f16": 10, "bf16": 7}
_EMIN = {"f16": -14, "bf16": -126}


def ulp(ref: np.ndarray, dtype: str) -> np.ndarray:
    """Spacing of `dtype` at the magnitude of each reference value."""
    a = np.abs(ref)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(np.where(a > 0, a, 1.0)))
    e = np.where(a > 0, np.maximum(e, _EMIN[dtype]), _EMIN[dtype])
    return np.exp2(e - _MANT[dtype])


def activation_error(got: torch.Tensor, ref64: np.ndarray, dtype: str) -> Tuple[float, str]:
    """Worst error of y / dx in units of the allowance; <= 1.0 passes.

    fp32: max-abs error against 1e-5 (scaled by the tensor's magnitude when that
    exceeds 1).  fp16 / bf16: 2 ulp of the output type at the reference value's
    magnitude, plus an fp32 round-off floor of 2^-20 times the tensor's largest
    magnitude - the kernels (like the reference's) compute in fp32, so elements whose
    terms cancel to nearly zero cannot be resolved below the round-off of the terms.
    """
    g = to_float64(got).reshape(ref64.shape)
    err = np.abs(g - ref64)
    scale = max(1.0, float(np.abs(ref64).max())) if ref64.size else 1.0
    if dtype == "f32":
        worst = float(err.max()) if err.size else 0.0
        return worst / (1e-5 * scale), f"max-abs {worst:.3e} (allow {1e-5 * scale:.1e})"
    allow = 2.0 * ulp(ref64, dtype) + scale * 2.0 ** -20
    ratio = err / allow
    worst = float(ratio.max()) if ratio.size else 0.0
    raw = float((err / ulp(ref64, dtype)).max()) if err.size else 0.0
    return worst, f"worst {worst:.3f} of allowance, {raw:.2f} raw ulp"


def grad_param_error(got: torch.Tensor, ref64: np.ndarray) -> Tuple[float, str]:
    """dgamma / dbeta: max |delta| / max |ref| against 1e-4."""
    g = to_float64(got).reshape(ref64.shape)
    denom = float(np.abs(ref64).max()) if ref64.size else 1.0
    denom = denom if denom > 0 else 1.0
    rel = float(np.abs(g - ref64).max()) / denom if ref64.size else 0.0
    return rel / 1e-4, f"norm-wise rel {rel:.3e}"


def stats_error(mean: torch.Tensor, inv_std: torch.Tensor, mean64: np.ndarray,
                inv_std64: np.ndarray) -> Tuple[float, str]:
    """Saved statistics: inverse std to 1e-5 relative; mean to 1e-5 of (|mean| + std)."""
    m = to_float64(mean).reshape(mean64.shape)
    s = to_float64(inv_std).reshape(inv_std64.shape)
    e_s = float((np.abs(s - inv_std64) / np.abs(inv_std64)).max()) if s.size else 0.0
    e_m = float((np.abs(m - mean64) / (np.abs(mean64) + 1.0 / inv_std64)).max()) if m.size else 0.0
    return max(e_s, e_m) / 1e-5, f"mean rel {e_m:.2e}, inv_std rel {e_s:.2e}"
