"""Host-side mirror of the reference's Python surface for the fused norm ops.

The reference (atex/nv_norms/python/ops/nv_norm_ops.py) loads a TensorFlow op
library and exposes four raw ops, two registered gradient functions and two
Keras wrapper layers.  TensorFlow is not part of this build's environment, so
the same surface is offered over PyTorch tensors, which only supply device
memory and streams; all arithmetic happens in libnvnorms.so through the C ABI
of include/nvnorms.h - the ABI a TensorFlow OpKernel would bind as well.

  fused_layer_norm_op / fused_layer_norm_grad_op
  fused_instance_norm_op / fused_instance_norm_grad_op      nv_norm_ops.py:22-25
  _layer_norm_grad / _instance_norm_grad                    nv_norm_ops.py:27-67
  LayerNormalization / InstanceNormalization                nv_norm_ops.py:69-184

Argument names, defaults, output order, shape rules and error messages follow
the op registrations (atex/nv_norms/cc/ops/norm_ops.cc:148-202) and the OpKernel
checks (atex/nv_norms/cc/kernels/fused_layer_norm_op.cc:295-458,
atex/nv_norms/cc/kernels/fused_instance_norm_op.cc:328-534).  `T` additionally
accepts bfloat16.
"""
from __future__ import annotations

import contextlib
import ctypes
from typing import Iterable, List, Sequence, Tuple

import torch

from . import _lib

__all__ = [
    "InvalidArgumentError",
    "fused_layer_norm_op", "fused_layer_norm_grad_op", "fused_layer_norm_residual_op",
    "fused_instance_norm_op", "fused_instance_norm_grad_op",
    "_layer_norm_grad", "_instance_norm_grad",
    "LayerNormalization", "InstanceNormalization",
    "layer_norm", "instance_norm",
]


class InvalidArgumentError(ValueError):
    """Counterpart of tf.errors.InvalidArgumentError raised by OP_REQUIRES."""


_DTYPE_CODE = {torch.float32: _lib.NVN_F32, torch.float16: _lib.NVN_F16,
               torch.bfloat16: _lib.NVN_BF16}

# One scratch tensor per (device, stream), grown on demand: the analogue of the
# OpKernelContext::allocate_temp calls in the reference functors.  Work on one
# stream is ordered, so consecutive ops can share it.
_workspaces = {}


def _workspace(device: torch.device, stream: int, nbytes: int) -> Tuple[int, int]:
    if nbytes == 0:
        return 0, 0
    key = (device.index, stream)
    ws = _workspaces.get(key)
    if ws is None or ws[1] < nbytes:
        t = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        ws = (t.data_ptr(), t.numel(), t)
        _workspaces[key] = ws
    return ws[0], ws[1]


# Shape bookkeeping and workspace sizes are pure functions of the problem; a training loop
# asks for the same few on every step, so they are remembered (bounded, see _remember).
_dims_cache = {}
_ws_bytes_cache = {}


def _remember(cache: dict, key, value):
    if len(cache) >= 4096:
        cache.clear()
    cache[key] = value
    return value


def _ws_bytes(fn_name: str, *args) -> int:
    key = (fn_name,) + args
    v = _ws_bytes_cache.get(key)
    if v is None:
        v = _remember(_ws_bytes_cache, key, int(getattr(_lib.load(), fn_name)(*args)))
    return v


def _device_guard(device: torch.device):
    """Makes `device` current for the C-ABI call (it works on the calling thread's current
    device); free when it already is."""
    if torch.cuda.current_device() == device.index:
        return contextlib.nullcontext()
    return torch.cuda.device(device)


def _require(cond: bool, *msg) -> None:
    """OP_REQUIRES: tensors among `msg` are rendered as their shape, and only on failure."""
    if not cond:
        raise InvalidArgumentError("".join(
            _shape_str(m) if isinstance(m, torch.Tensor) else str(m) for m in msg))


def _check(status: int, what: str) -> None:
    if status == _lib.NVN_OK:
        return
    text = _lib.status_string(status)
    if status == _lib.NVN_ERR_CUDA:
        raise RuntimeError(f"{what}: {text} (cudaError {_lib.load().nvn_last_cuda_error()})")
    if status in (_lib.NVN_ERR_WORKSPACE, _lib.NVN_ERR_UNSUPPORTED, _lib.NVN_ERR_LIMIT):
        raise RuntimeError(f"{what}: {text}")
    raise InvalidArgumentError(text)


def _dtype_code(t: torch.Tensor, name: str) -> int:
    if t.dtype not in _DTYPE_CODE:
        raise TypeError(f"{name} must be float32, float16 or bfloat16, got {t.dtype}")
    return _DTYPE_CODE[t.dtype]


def _cuda_contig(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(
            f"{name} is on {t.device}: the fused norm ops only run on a CUDA device "
            "(there is no CPU implementation)")
    return t if t.is_contiguous() else t.contiguous()


def _param(t: torch.Tensor, name: str) -> torch.Tensor:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor")
    if t.dtype != torch.float32:
        raise TypeError(f"{name} must be float32 (attr U), got {t.dtype}")
    return t


def _on_device(*named):
    """Shape validation needs no GPU; this runs after it and insists on CUDA memory."""
    return [_cuda_contig(t, name) for t, name in named]


def _shape_str(t: torch.Tensor) -> str:
    return "[" + ",".join(str(int(s)) for s in t.shape) + "]"


def _ln_dims(x: torch.Tensor, axis: Sequence[int]) -> Tuple[int, int]:
    """GetBatchAndFeatureSizes (fused_layer_norm_op.cc:252-282) through the C ABI."""
    key = (tuple(x.shape), tuple(axis))
    hit = _dims_cache.get(key)
    if hit is not None:
        return hit
    rank = x.dim()
    dims = (ctypes.c_int64 * max(rank, 1))(*[int(s) for s in x.shape])
    ax = (ctypes.c_int * max(len(axis), 1))(*[int(a) for a in axis])
    N, D = ctypes.c_int64(), ctypes.c_int64()
    st = _lib.load().nvn_ln_dims(rank, dims, len(axis), ax, ctypes.byref(N), ctypes.byref(D))
    if st == _lib.NVN_ERR_AXIS_RANGE:
        bad = [a for a in axis if not (0 <= (a + rank if a < 0 else a) < rank)]
        raise InvalidArgumentError(f"axis contains invalid value: {bad[0] if bad else axis}")
    _check(st, "nvn_ln_dims")
    return _remember(_dims_cache, key, (N.value, D.value))


def _in_dims(x: torch.Tensor, data_format: str) -> Tuple[int, int, int, bool]:
    key = (tuple(x.shape), str(data_format))
    hit = _dims_cache.get(key)
    if hit is not None:
        return hit
    rank = x.dim()
    dims = (ctypes.c_int64 * max(rank, 1))(*[int(s) for s in x.shape])
    N, C, D, cf = ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int64(), ctypes.c_int()
    st = _lib.load().nvn_in_dims(rank, dims, str(data_format).encode(), ctypes.byref(N),
                                 ctypes.byref(C), ctypes.byref(D), ctypes.byref(cf))
    if st == _lib.NVN_ERR_DATA_FORMAT:
        raise InvalidArgumentError(
            f"We only accept 'NC...' or 'N...C' data format, but got{data_format}")
    if st == _lib.NVN_ERR_RANK:
        raise InvalidArgumentError(f"input must be at least 4-dimensional{_shape_str(x)}")
    _check(st, "nvn_in_dims")
    return _remember(_dims_cache, key, (N.value, C.value, D.value, bool(cf.value)))


def _axis_list(axis) -> List[int]:
    if isinstance(axis, int):
        return [axis]
    return [int(a) for a in axis]


def _stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


# ---------------------------------------------------------------------------
# raw ops
# ---------------------------------------------------------------------------
def _stats_outputs(shape, device, out_stats):
    """mean / inv_std buffers: fresh, or the caller's pair of contiguous float32 tensors."""
    if out_stats is None:
        return (torch.empty(shape, dtype=torch.float32, device=device),
                torch.empty(shape, dtype=torch.float32, device=device))
    mean, inv_std = out_stats
    n = 1
    for s_ in (shape if isinstance(shape, tuple) else (shape,)):
        n *= s_
    for t in (mean, inv_std):
        if (t.dtype != torch.float32 or t.numel() != n or not t.is_contiguous()
                or t.device != device):
            raise ValueError("out_stats must be two contiguous float32 tensors of the statistics' size")
    return mean, inv_std


def _like_output(x, out, name):
    if out is None:
        return torch.empty_like(x)
    if out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous() or out.device != x.device:
        raise ValueError(f"{name} must be a contiguous tensor like x")
    return out


def fused_layer_norm_op(x, scale, offset, axis: Iterable[int] = (-1,), epsilon: float = 0.001,
                        out: torch.Tensor | None = None, out_stats=None):
    """FusedLayerNorm (norm_ops.cc:148-159): returns (y, reserve_space_1, reserve_space_2).

    reserve_space_1 is the per-row mean and reserve_space_2 the per-row
    1/sqrt(var + epsilon), both float32 of shape [N] with N the product of the
    non-normalised leading dims.  `out` may be `x` itself to normalise in place
    (the reference forwards its input buffer the same way); `out_stats` optionally supplies
    the (reserve_space_1, reserve_space_2) buffers, so that a steady-state loop allocates
    nothing.
    """
    _require(isinstance(x, torch.Tensor) and x.dim() > 0, "input must be at least 1-dimensional",
             x if isinstance(x, torch.Tensor) else "")
    code = _dtype_code(x, "x")
    scale, offset = _param(scale, "scale"), _param(offset, "offset")
    axis = _axis_list(axis)
    N, D = _ln_dims(x, axis)
    _require(scale.numel() == D, "scale must have the same number of elements as the features "
             "of x, got ", scale.numel(), " and ", D)
    _require(offset.numel() == D, "offset must have the same number of elements as the features "
             "of x, got ", offset.numel(), " and ", D)
    x, scale, offset = _on_device((x, "x"), (scale, "scale"), (offset, "offset"))
    y = _like_output(x, out, "out")
    mean, inv_std = _stats_outputs(N, x.device, out_stats)
    with _device_guard(x.device):
        lib = _lib.load()
        stream = _stream(x.device)
        ws_ptr, ws_bytes = _workspace(x.device, stream, _ws_bytes("nvn_ln_fwd_workspace_bytes", code, N, D))
        st = lib.nvn_ln_fwd(code, x.data_ptr(), scale.data_ptr(), offset.data_ptr(), N, D,
                            float(epsilon), y.data_ptr(), mean.data_ptr(), inv_std.data_ptr(),
                            ws_ptr, ws_bytes, stream)
    _check(st, "nvn_ln_fwd")
    return y, mean, inv_std


def fused_layer_norm_residual_op(x, residual, scale, offset, axis: Iterable[int] = (-1,),
                                 epsilon: float = 0.001, out: torch.Tensor | None = None,
                                 out_sum: torch.Tensor | None = None, out_stats=None):
    """Residual add + FusedLayerNorm in one pass: returns (y, s, reserve_space_1,
    reserve_space_2) with s = (x + residual) rounded to x's dtype and y = LayerNorm(s).

    The step in front of every LayerNorm of a pre-norm transformer block; the gradient op is
    fused_layer_norm_grad_op on s (its x_backprop is the gradient of x and of residual).
    `out_sum` may be `x` or `residual` to update the residual stream in place.  The
    reference has no such op (its layer calls the bare norm, nv_norm_ops.py:85-99)."""
    _require(isinstance(x, torch.Tensor) and x.dim() > 0, "input must be at least 1-dimensional",
             x if isinstance(x, torch.Tensor) else "")
    code = _dtype_code(x, "x")
    if not isinstance(residual, torch.Tensor) or residual.shape != x.shape or residual.dtype != x.dtype:
        raise InvalidArgumentError("residual must have the shape and dtype of x")
    scale, offset = _param(scale, "scale"), _param(offset, "offset")
    axis = _axis_list(axis)
    N, D = _ln_dims(x, axis)
    _require(scale.numel() == D, "scale must have the same number of elements as the features "
             "of x, got ", scale.numel(), " and ", D)
    _require(offset.numel() == D, "offset must have the same number of elements as the features "
             "of x, got ", offset.numel(), " and ", D)
    x, residual, scale, offset = _on_device((x, "x"), (residual, "residual"), (scale, "scale"),
                                            (offset, "offset"))
    y = _like_output(x, out, "out")
    s = _like_output(x, out_sum, "out_sum")
    mean, inv_std = _stats_outputs(N, x.device, out_stats)
    with _device_guard(x.device):
        lib = _lib.load()
        stream = _stream(x.device)
        ws_ptr, ws_bytes = _workspace(x.device, stream, _ws_bytes("nvn_ln_fwd_workspace_bytes", code, N, D))
        st = lib.nvn_ln_fwd_residual(code, x.data_ptr(), residual.data_ptr(), scale.data_ptr(),
                                     offset.data_ptr(), N, D, float(epsilon), s.data_ptr(),
                                     y.data_ptr(), mean.data_ptr(), inv_std.data_ptr(), ws_ptr,
                                     ws_bytes, stream)
    _check(st, "nvn_ln_fwd_residual")
    return y, s, mean, inv_std


def _grad_outputs(scale: torch.Tensor, out_grads):
    """dgamma / dbeta buffers: fresh, or the caller's pair (e.g. two halves of one all-reduce
    buffer).  Caller buffers must be contiguous float32 of scale's size on scale's device."""
    if out_grads is None:
        return torch.empty_like(scale), torch.empty_like(scale)
    dgamma, dbeta = out_grads
    for t in (dgamma, dbeta):
        if (t.dtype != torch.float32 or t.numel() != scale.numel() or not t.is_contiguous()
                or t.device != scale.device):
            raise ValueError("out_grads must be two contiguous float32 tensors of scale's size")
    return dgamma, dbeta


def fused_layer_norm_grad_op(y_backprop, x, scale, reserve_space_1, reserve_space_2,
                             axis: Iterable[int] = (-1,), epsilon: float = 0.001, out_grads=None,
                             grad_exchange=None, out: torch.Tensor | None = None):
    """FusedLayerNormGrad (norm_ops.cc:161-174): returns (x_backprop, scale_backprop,
    offset_backprop); the parameter gradients take the shape of `scale`.  `out_grads`
    optionally supplies the (scale_backprop, offset_backprop) buffers and `out` the
    x_backprop buffer.  With
    `grad_exchange` (a sharding.GradExchange) the parameter gradients come back already
    summed over all data-parallel ranks."""
    _require(isinstance(y_backprop, torch.Tensor) and y_backprop.dim() > 0,
             "input must be at least 1-dimensional", y_backprop)
    _require(isinstance(x, torch.Tensor) and x.dim() > 0, "input must be at least 1-dimensional",
             x)
    dy = y_backprop
    code = _dtype_code(x, "x")
    if dy.dtype != x.dtype:
        raise TypeError(f"y_backprop ({dy.dtype}) and x ({x.dtype}) must have the same dtype")
    scale = _param(scale, "scale")
    mean, inv_std = _param(reserve_space_1, "reserve_space_1"), _param(reserve_space_2, "reserve_space_2")
    _require(mean.dim() == 1, "saved mean must be 1-dimensional", mean)
    _require(inv_std.dim() == 1, "saved inverted variance must be 1-dimensional", inv_std)
    _require(x.shape == dy.shape, "x and y_backprop must have same shape, but x has shape ",
             x, " and y_backprop has shape ", dy)
    N, D = _ln_dims(x, _axis_list(axis))
    _require(scale.numel() == D, "scale must have the same number of elements as the features "
             "of x, got ", scale.numel(), " and ", D)
    _require(mean.numel() == N, "reserve_space_1 must have the same number of elements as the "
             "batches of x, got ", mean.numel(), " and ", N)
    _require(inv_std.numel() == N, "reserve_space_2 must have the same number of elements as the "
             "channels of x, got ", inv_std.numel(), " and ", N)
    x, dy, scale, mean, inv_std = _on_device((x, "x"), (dy, "y_backprop"), (scale, "scale"),
                                             (mean, "reserve_space_1"), (inv_std, "reserve_space_2"))
    dx = _like_output(x, out, "out")
    dgamma, dbeta = _grad_outputs(scale, out_grads)
    with _device_guard(x.device):
        lib = _lib.load()
        stream = _stream(x.device)
        ws_ptr, ws_bytes = _workspace(x.device, stream, _ws_bytes("nvn_ln_bwd_workspace_bytes", code, N, D))
        if grad_exchange is None:
            st = lib.nvn_ln_bwd(code, dy.data_ptr(), x.data_ptr(), scale.data_ptr(),
                                mean.data_ptr(), inv_std.data_ptr(), N, D, dx.data_ptr(),
                                dgamma.data_ptr(), dbeta.data_ptr(), ws_ptr, ws_bytes, stream)
        else:
            st = lib.nvn_ln_bwd_dp(code, dy.data_ptr(), x.data_ptr(), scale.data_ptr(),
                                   mean.data_ptr(), inv_std.data_ptr(), N, D, dx.data_ptr(),
                                   dgamma.data_ptr(), dbeta.data_ptr(), ws_ptr, ws_bytes,
                                   grad_exchange.next_comm(D), stream)
    _check(st, "nvn_ln_bwd")
    return dx, dgamma, dbeta


def fused_instance_norm_op(x, scale, offset, data_format: str = "N...C", epsilon: float = 0.001,
                           out: torch.Tensor | None = None, out_stats=None):
    """FusedInstanceNorm (norm_ops.cc:176-187): returns (y, reserve_space_1, reserve_space_2)
    with the statistics of shape [N, C]."""
    _require(isinstance(x, torch.Tensor), "input must be a tensor")
    N, C, D, cf = _in_dims(x, data_format)
    code = _dtype_code(x, "x")
    scale, offset = _param(scale, "scale"), _param(offset, "offset")
    _require(scale.dim() == 1, "scale must be 1-dimensional", scale)
    _require(offset.dim() == 1, "offset must be 1-dimensional", offset)
    _require(scale.numel() == C, "scale must have the same number of elements as the channels "
             "of x, got ", scale.numel(), " and ", C)
    _require(offset.numel() == C, "offset must have the same number of elements as the channels "
             "of x, got ", offset.numel(), " and ", C)
    x, scale, offset = _on_device((x, "x"), (scale, "scale"), (offset, "offset"))
    y = _like_output(x, out, "out")
    mean, inv_std = _stats_outputs((N, C), x.device, out_stats)
    with _device_guard(x.device):
        lib = _lib.load()
        stream = _stream(x.device)
        ws_ptr, ws_bytes = _workspace(
            x.device, stream, _ws_bytes("nvn_in_fwd_workspace_bytes", code, N, C, D, int(cf)))
        st = lib.nvn_in_fwd(code, x.data_ptr(), scale.data_ptr(), offset.data_ptr(), N, C, D, int(cf),
                            float(epsilon), y.data_ptr(), mean.data_ptr(), inv_std.data_ptr(),
                            ws_ptr, ws_bytes, stream)
    _check(st, "nvn_in_fwd")
    return y, mean, inv_std


def fused_instance_norm_grad_op(y_backprop, x, scale, reserve_space_1, reserve_space_2,
                                data_format: str = "N...C", epsilon: float = 0.001, out_grads=None,
                                grad_exchange=None, out: torch.Tensor | None = None):
    """FusedInstanceNormGrad (norm_ops.cc:189-202): returns (x_backprop, scale_backprop,
    offset_backprop).  `out_grads` optionally supplies the two parameter-gradient buffers."""
    _require(isinstance(y_backprop, torch.Tensor) and y_backprop.dim() > 3,
             "input must be at least 4-dimensional", y_backprop)
    _require(isinstance(x, torch.Tensor) and x.dim() > 1, "input must be at least 2-dimensional",
             x)
    dy = y_backprop
    code = _dtype_code(x, "x")
    if dy.dtype != x.dtype:
        raise TypeError(f"y_backprop ({dy.dtype}) and x ({x.dtype}) must have the same dtype")
    scale = _param(scale, "scale")
    mean, inv_std = _param(reserve_space_1, "reserve_space_1"), _param(reserve_space_2, "reserve_space_2")
    _require(scale.dim() == 1, "scale must be 1-dimensional", scale)
    _require(mean.dim() == 2, "saved mean must be 2-dimensional", mean)
    _require(inv_std.dim() == 2, "saved inverted variance must be 2-dimensional", inv_std)
    _require(x.shape == dy.shape, "x and y_backprop must have same shape, but x has shape ",
             x, " and y_backprop has shape ", dy)
    N, C, D, cf = _in_dims(x, data_format)
    _require(scale.numel() == C, "scale must have the same number of elements as the channels "
             "of x, got ", scale.numel(), " and ", C)
    _require(mean.numel() == N * C, "reserve_space_1 must have the same number of elements as "
             "the batches*channels of x, got ", mean.numel(), " and ", N * C)
    _require(inv_std.numel() == N * C, "reserve_space_2 must have the same number of elements as "
             "the batches * channels of x, got ", inv_std.numel(), " and ", N * C)
    x, dy, scale, mean, inv_std = _on_device((x, "x"), (dy, "y_backprop"), (scale, "scale"),
                                             (mean, "reserve_space_1"), (inv_std, "reserve_space_2"))
    dx = _like_output(x, out, "out")
    dgamma, dbeta = _grad_outputs(scale, out_grads)
    with _device_guard(x.device):
        lib = _lib.load()
        stream = _stream(x.device)
        ws_ptr, ws_bytes = _workspace(
            x.device, stream, _ws_bytes("nvn_in_bwd_workspace_bytes", code, N, C, D, int(cf)))
        if grad_exchange is None:
            st = lib.nvn_in_bwd(code, dy.data_ptr(), x.data_ptr(), scale.data_ptr(),
                                mean.data_ptr(), inv_std.data_ptr(), N, C, D, int(cf),
                                dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), ws_ptr,
                                ws_bytes, stream)
        else:
            st = lib.nvn_in_bwd_dp(code, dy.data_ptr(), x.data_ptr(), scale.data_ptr(),
                                   mean.data_ptr(), inv_std.data_ptr(), N, C, D, int(cf),
                                   dx.data_ptr(), dgamma.data_ptr(), dbeta.data_ptr(), ws_ptr,
                                   ws_bytes, grad_exchange.next_comm(C), stream)
    _check(st, "nvn_in_bwd")
    return dx, dgamma, dbeta


# ---------------------------------------------------------------------------
# gradient registration (ops.RegisterGradient in the reference)
# ---------------------------------------------------------------------------
class _layer_norm_grad(torch.autograd.Function):
    """Differentiable FusedLayerNorm: backward calls fused_layer_norm_grad_op with the
    saved statistics, as the reference's registered gradient does (nv_norm_ops.py:48-67)."""

    @staticmethod
    def forward(ctx, x, gamma, beta, axis, epsilon):
        y, mean, inv_std = fused_layer_norm_op(x, gamma, beta, axis=axis, epsilon=epsilon)
        ctx.save_for_backward(x, gamma, mean, inv_std)
        ctx.axis = tuple(axis)
        ctx.mark_non_differentiable(mean, inv_std)
        return y, mean, inv_std

    @staticmethod
    def backward(ctx, grad_y, _gm, _gi):
        x, gamma, mean, inv_std = ctx.saved_tensors
        dx, dgamma, dbeta = fused_layer_norm_grad_op(grad_y, x, gamma, mean, inv_std, axis=ctx.axis)
        return dx, dgamma, dbeta, None, None


class _instance_norm_grad(torch.autograd.Function):
    """Differentiable FusedInstanceNorm (nv_norm_ops.py:27-46)."""

    @staticmethod
    def forward(ctx, x, gamma, beta, data_format, epsilon):
        y, mean, inv_std = fused_instance_norm_op(x, gamma, beta, data_format=data_format,
                                                  epsilon=epsilon)
        ctx.save_for_backward(x, gamma, mean, inv_std)
        ctx.data_format = data_format
        ctx.mark_non_differentiable(mean, inv_std)
        return y, mean, inv_std

    @staticmethod
    def backward(ctx, grad_y, _gm, _gi):
        x, gamma, mean, inv_std = ctx.saved_tensors
        dx, dgamma, dbeta = fused_instance_norm_grad_op(grad_y, x, gamma, mean, inv_std,
                                                        data_format=ctx.data_format)
        return dx, dgamma, dbeta, None, None


def layer_norm(x, gamma, beta, axis=(-1,), epsilon=0.001):
    """Differentiable y = FusedLayerNorm(x)."""
    return _layer_norm_grad.apply(x, gamma, beta, tuple(_axis_list(axis)), float(epsilon))[0]


def instance_norm(x, gamma, beta, data_format="N...C", epsilon=0.001):
    """Differentiable y = FusedInstanceNorm(x)."""
    return _instance_norm_grad.apply(x, gamma, beta, str(data_format), float(epsilon))[0]


# ---------------------------------------------------------------------------
# wrapper layers
# ---------------------------------------------------------------------------
class LayerNormalization(torch.nn.Module):
    """Drop-in for nv_norms.LayerNormalization (nv_norm_ops.py:69-121).

    Takes the tf.keras.layers.LayerNormalization keyword arguments that matter
    to the computation: ``axis`` (int or list, default -1; must be the packed
    trailing dims, sorted and unique), ``epsilon`` (default 1e-3), ``center``
    and ``scale``.  gamma / beta are float32 and are created on the first call
    with the shape of the normalised dims (Keras ``build``).
    """

    def __init__(self, axis=-1, epsilon=1e-3, center=True, scale=True, **kwargs):
        super().__init__()
        self.axis = axis
        self.epsilon = float(epsilon)
        self.center = bool(center)
        self.scale = bool(scale)
        self._extra = dict(kwargs)
        self.gamma = None
        self.beta = None
        self.built = False

    def build(self, input_shape, device=None):
        axis = _axis_list(self.axis)
        rank = len(input_shape)
        norm = [a + rank if a < 0 else a for a in axis]
        for a in norm:
            if not 0 <= a < rank:
                raise ValueError(f"Invalid axis: {self.axis}")
        shape = [int(input_shape[a]) for a in norm]
        g = torch.ones(shape, dtype=torch.float32, device=device)
        b = torch.zeros(shape, dtype=torch.float32, device=device)
        self.gamma = torch.nn.Parameter(g, requires_grad=self.scale)
        self.beta = torch.nn.Parameter(b, requires_grad=self.center)
        self._norm_axis = norm
        self.built = True

    def forward(self, inputs):
        if not self.built:
            self.build(tuple(inputs.shape), device=inputs.device)
        axis = _axis_list(self.axis)
        if axis != sorted(set(axis)):
            raise ValueError("We only support sorted and unique axis to make sure the weights "
                             "have the same data layout with the keras layers.")
        return layer_norm(inputs, self.gamma, self.beta, axis=axis, epsilon=self.epsilon)

    call = forward

    def get_weights(self):
        return [self.gamma.detach().cpu().numpy(), self.beta.detach().cpu().numpy()]

    def set_weights(self, weights):
        g, b = weights
        with torch.no_grad():
            self.gamma.copy_(torch.as_tensor(g, dtype=torch.float32).reshape(self.gamma.shape))
            self.beta.copy_(torch.as_tensor(b, dtype=torch.float32).reshape(self.beta.shape))

    @property
    def variables(self):
        """The layer's weights, [gamma, beta] (alias of ``weights`` in the reference)."""
        return [self.gamma, self.beta]

    weights = variables

    def get_config(self):
        cfg = {"axis": self.axis, "epsilon": self.epsilon, "center": self.center, "scale": self.scale}
        cfg.update(self._extra)
        return {"layer_norm": cfg}


class InstanceNormalization(torch.nn.Module):
    """Drop-in for nv_norms.InstanceNormalization (nv_norm_ops.py:123-184).

    ``axis`` is the channel axis and must be 1 ("NC...") or -1 ("N...C"); the
    remaining tfa.layers.InstanceNormalization keywords that matter are
    ``epsilon`` (default 1e-3), ``center`` and ``scale``.  gamma / beta are always
    float32, also under a mixed-precision policy (nv_norm_ops.py:133-143).
    """

    def __init__(self, axis=-1, epsilon=1e-3, center=True, scale=True, **kwargs):
        super().__init__()
        self.axis = axis
        self.epsilon = float(epsilon)
        self.center = bool(center)
        self.scale = bool(scale)
        self._extra = dict(kwargs)
        self.gamma = None
        self.beta = None
        self.built = False

    def build(self, input_shape, device=None):
        C = int(input_shape[self.axis])
        self.gamma = torch.nn.Parameter(torch.ones(C, dtype=torch.float32, device=device),
                                        requires_grad=self.scale)
        self.beta = torch.nn.Parameter(torch.zeros(C, dtype=torch.float32, device=device),
                                       requires_grad=self.center)
        self.built = True

    def forward(self, inputs):
        if self.axis == 1:
            data_format = "NC..."
        elif self.axis == -1:
            data_format = "N...C"
        else:
            raise ValueError("We only support integer axis of 1 or -1 corresponds to"
                             "channel first or channel last layout.")
        if not self.built:
            self.build(tuple(inputs.shape), device=inputs.device)
        return instance_norm(inputs, self.gamma, self.beta, data_format=data_format,
                             epsilon=self.epsilon)

    call = forward

    def get_weights(self):
        return [self.gamma.detach().cpu().numpy(), self.beta.detach().cpu().numpy()]

    def set_weights(self, weights):
        g, b = weights
        with torch.no_grad():
            self.gamma.copy_(torch.as_tensor(g, dtype=torch.float32).reshape(self.gamma.shape))
            self.beta.copy_(torch.as_tensor(b, dtype=torch.float32).reshape(self.beta.shape))

    @property
    def variables(self):
        return [self.gamma, self.beta]

    weights = variables

    def get_config(self):
        cfg = {"axis": self.axis, "epsilon": self.epsilon, "center": self.center, "scale": self.scale}
        cfg.update(self._extra)
        return {"instance_norm": cfg}
