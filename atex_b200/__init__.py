"""atex_b200: fused LayerNorm / InstanceNorm forward and gradient ops for NVIDIA
B200, exposing the public names of the reference package
(atex/nv_norms/__init__.py:6-13).
"""
from .nv_norm_ops import (InstanceNormalization, InvalidArgumentError, LayerNormalization,
                          _instance_norm_grad, _layer_norm_grad, fused_instance_norm_grad_op,
                          fused_instance_norm_op, fused_layer_norm_grad_op, fused_layer_norm_op,
                          fused_layer_norm_residual_op, instance_norm, layer_norm)

__all__ = [
    "fused_layer_norm_op", "fused_layer_norm_grad_op", "fused_instance_norm_op",
    "fused_instance_norm_grad_op", "_layer_norm_grad", "_instance_norm_grad",
    "LayerNormalization", "InstanceNormalization", "InvalidArgumentError", "layer_norm",
    "instance_norm", "fused_layer_norm_residual_op",
]
