"""TensorFlow bindings of the fused norm ops: op library loading, gradient
registration and Keras wrapper layers with the interface of the reference's
atex/nv_norms/python/ops/nv_norm_ops.py.

The op library `_fused_nv_norm_ops.so` (atex_b200/csrc/tf) registers
FusedLayerNorm, FusedLayerNormGrad, FusedInstanceNorm and FusedInstanceNormGrad
and forwards to libnvnorms.so.  This module cannot be imported without
TensorFlow; the PyTorch-side mirror in atex_b200/nv_norm_ops.py needs neither.
"""
import os

import tensorflow as tf
from tensorflow.python.framework import load_library, ops

_PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_OP_LIB = os.path.join(_PKG, "_fused_nv_norm_ops.so")
if not os.path.exists(_OP_LIB):
    raise ImportError(
        f"{_OP_LIB} not found: build it with `cmake -S atex_b200/csrc/tf -B build/tf && "
        "cmake --build build/tf --target install` after `python -m atex_b200.build`.")

_ops = load_library.load_op_library(_OP_LIB)
fused_layer_norm_op = _ops.fused_layer_norm
fused_layer_norm_grad_op = _ops.fused_layer_norm_grad
fused_instance_norm_op = _ops.fused_instance_norm
fused_instance_norm_grad_op = _ops.fused_instance_norm_grad


@ops.RegisterGradient("FusedLayerNorm")
def _layer_norm_grad(op, *grad):
    """dL/d(x, gamma, beta) of FusedLayerNorm from the saved mean and inverse std."""
    x, gamma = op.inputs[0], op.inputs[1]
    mean, inv_std = op.outputs[1], op.outputs[2]
    return list(fused_layer_norm_grad_op(grad[0], x, gamma, mean, inv_std,
                                         axis=op.get_attr("axis")))


@ops.RegisterGradient("FusedInstanceNorm")
def _instance_norm_grad(op, *grad):
    """dL/d(x, gamma, beta) of FusedInstanceNorm from the saved mean and inverse std."""
    x, gamma = op.inputs[0], op.inputs[1]
    mean, inv_std = op.outputs[1], op.outputs[2]
    return list(fused_instance_norm_grad_op(grad[0], x, gamma, mean, inv_std,
                                            data_format=op.get_attr("data_format")))


class _WeightsFromInner(tf.keras.layers.Layer):
    """Shared plumbing: weights, config and (de)serialisation live in an inner stock layer,
    exactly as in the reference wrappers, so checkpoints stay interchangeable."""

    _inner_key = "inner"

    def build(self, input_shape):
        self._inner.build(input_shape=input_shape)
        self.built = True

    def get_weights(self):
        return self._inner.get_weights()

    def set_weights(self, weights):
        self._inner.set_weights(weights)

    @property
    def variables(self):
        return self._inner.weights

    def get_config(self):
        config = super().get_config()
        config[self._inner_key] = self._inner
        return config


class LayerNormalization(_WeightsFromInner):
    """tf.keras.layers.LayerNormalization computed by the fused op.  `axis` must be the packed
    trailing dimensions, sorted and unique."""

    _inner_key = "layer_norm"

    def __init__(self, **kwargs):
        super().__init__()
        self._inner = tf.keras.layers.LayerNormalization(**kwargs)
        self.layer_norm = self._inner

    def call(self, inputs):
        axis = self._inner.axis
        axis = [axis] if isinstance(axis, int) else list(axis)
        if axis != sorted(set(axis)):
            raise ValueError("We only support sorted and unique axis to make sure the weights "
                             "have the same data layout with the keras layers.")
        y, _, _ = fused_layer_norm_op(inputs, self._inner.gamma, self._inner.beta, axis=axis,
                                      epsilon=self._inner.epsilon)
        return y


class InstanceNormalization(_WeightsFromInner):
    """tfa.layers.InstanceNormalization computed by the fused op; `axis` is 1 or -1.  The
    weights stay float32 under a mixed-precision policy."""

    _inner_key = "instance_norm"

    def __init__(self, axis, **kwargs):
        super().__init__()
        import tensorflow_addons as tfa
        policy = tf.keras.mixed_precision.global_policy()
        mixed = policy is not None and policy.compute_dtype != policy.variable_dtype
        if mixed:
            tf.keras.mixed_precision.set_global_policy("float32")
        try:
            self._inner = tfa.layers.InstanceNormalization(axis=axis, **kwargs)
        finally:
            if mixed:
                tf.keras.mixed_precision.set_global_policy(policy)
        self.instance_norm = self._inner

    def call(self, inputs):
        axis = self._inner.axis
        if axis == 1:
            data_format = "NC..."
        elif axis == -1:
            data_format = "N...C"
        else:
            raise ValueError("We only support integer axis of 1 or -1 corresponds to"
                             "channel first or channel last layout.")
        y, _, _ = fused_instance_norm_op(inputs, self._inner.weights[0], self._inner.weights[1],
                                         data_format=data_format, epsilon=self._inner.epsilon)
        return y
