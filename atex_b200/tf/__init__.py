"""TensorFlow front end (needs TensorFlow and a built _fused_nv_norm_ops.so).

`from atex_b200.tf import LayerNormalization, InstanceNormalization` is the drop-in
for `from atex.nv_norms import ...` in a TensorFlow program.  Importing this
sub-package without TensorFlow raises ImportError; nothing else in atex_b200
depends on it.
"""
from .nv_norm_ops import (InstanceNormalization, LayerNormalization, _instance_norm_grad,  # noqa: F401
                          _layer_norm_grad, fused_instance_norm_grad_op, fused_instance_norm_op,
                          fused_layer_norm_grad_op, fused_layer_norm_op)
