"""Toy model Conv3d -> InstanceNormalization; `--nvops` swaps in the fused layer.

Counterpart of atex/nv_norms/examples/sample_instanceN.py (a Keras Conv3D followed by
tfa InstanceNormalization, channels last or first, one training step) on PyTorch tensors.

    python examples/sample_instanceN.py [--nvops] [--channels-first]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

parser = argparse.ArgumentParser(description="Use --nvops to replace InstanceN")
parser.add_argument("--nvops", action="store_true", help="Whether to use the fused InstanceNorm.")
parser.add_argument("--channels-first", action="store_true", help="NC... layout instead of N...C.")
args, _ = parser.parse_known_args()

N, D, H, W, C = (2, 2, 3, 4, 8)
k = 8
dev = torch.device("cuda:0")
axis = 1 if args.channels_first else -1

conv3d = torch.nn.Conv3d(C, k, 2, padding="same").to(dev)
if args.nvops:
    import atex_b200 as nv_norms
    instanceN = nv_norms.InstanceNormalization(axis=axis)
else:
    instanceN = torch.nn.InstanceNorm3d(k, eps=1e-3, affine=True).to(dev)


def train_step(x):
    y = conv3d(x)                                   # [N, k, D, H, W]
    if args.nvops and not args.channels_first:
        y = y.permute(0, 2, 3, 4, 1).contiguous()   # N...C for the fused layer
    z = instanceN(y)
    loss = z.sum()
    params = list(conv3d.parameters())
    params += list(instanceN.variables) if args.nvops else list(instanceN.parameters())
    return torch.autograd.grad(loss, params)


data = torch.randn(N, C, D, H, W, device=dev)
g = train_step(data)
_ = g[0].cpu()  # sync GPU
print("Done with", "Fused InstanceN" if args.nvops else "torch InstanceN")
