"""Batch-axis sharding of the norm ops over the GPUs of one node.

The reference ops are single-device (nothing in atex/nv_norms touches a
communicator); in a data-parallel job every rank normalises its own slice of
the batch and only the parameter gradients need to meet.  Rows (LayerNorm) and
batch items (InstanceNorm) are independent, so forward needs no communication
and backward needs exactly one all-reduce of the concatenated
[dgamma | dbeta] vector.  torch.distributed supplies the process group (NCCL
over NVLink on GPUs, gloo in CPU tests).
"""
from __future__ import annotations

from typing import Tuple

import torch
import torch.distributed as dist


def shard_range(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous [start, stop) slice of `total` batch entries owned by `rank`.

    The first ``total % world`` ranks own one extra entry, so any total works
    and the slices tile the batch in rank order.
    """
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    base, extra = divmod(total, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def allreduce_param_grads(dgamma: torch.Tensor, dbeta: torch.Tensor, group=None,
                          buffer: torch.Tensor | None = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sum dgamma and dbeta over the ranks with ONE collective.

    The two vectors are packed into one contiguous fp32 buffer (pass `buffer`, of
    2 * dgamma.numel() floats, to avoid the allocation), reduced in place and
    returned as views of it.  Without an initialised process group (single GPU)
    the inputs are returned untouched.
    """
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return dgamma, dbeta
    F = dgamma.numel()
    if buffer is None:
        buffer = torch.empty(2 * F, dtype=torch.float32, device=dgamma.device)
    buffer[:F].copy_(dgamma.reshape(-1))
    buffer[F:].copy_(dbeta.reshape(-1))
    dist.all_reduce(buffer, op=dist.ReduceOp.SUM, group=group)
    return buffer[:F].view(dgamma.shape), buffer[F:].view(dbeta.shape)
