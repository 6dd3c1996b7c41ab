"""Toy model Conv2d -> LayerNormalization; `--nvops` swaps in the fused layer.

Counterpart of atex/nv_norms/examples/sample_layerN.py (a Keras Conv2D followed by
LayerNormalization over axes (1, 2, 3), one training step, gradients of sum(y)) on PyTorch
tensors: the host framework only supplies the convolution, autograd and device memory; the
normalisation runs in libnvnorms through the C ABI.

    python examples/sample_layerN.py [--nvops]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

parser = argparse.ArgumentParser(description="Use --nvops to replace LayerN")
parser.add_argument("--nvops", action="store_true", help="Whether to use the fused LayerNorm.")
args, _ = parser.parse_known_args()

N, H, W, C = (10, 3, 3, 4)
k, c, r, s = (4, C, 2, 2)
dev = torch.device("cuda:0")

conv2d = torch.nn.Conv2d(c, k, (r, s), padding="same").to(dev)
if args.nvops:
    import atex_b200 as nv_norms
    layerN = nv_norms.LayerNormalization(axis=(1, 2, 3))
else:
    layerN = torch.nn.LayerNorm((H, W, k), eps=1e-3).to(dev)


def train_step(x):
    # channels-last activations, as in the Keras original: [N, H, W, C]
    y = conv2d(x.permute(0, 3, 1, 2)).permute(0, 2, 3, 1).contiguous()
    z = layerN(y)
    loss = z.sum()
    params = list(conv2d.parameters()) + [p for p in layerN.parameters()]
    if args.nvops:
        params = list(conv2d.parameters()) + list(layerN.variables)
    return torch.autograd.grad(loss, params)


data = torch.randn(N, H, W, C, device=dev)
g = train_step(data)
_ = g[0].cpu()  # sync GPU
print("Done with", "Fused LayerN" if args.nvops else "torch LayerN")
