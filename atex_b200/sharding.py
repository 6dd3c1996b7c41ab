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

import ctypes
from typing import Tuple

import torch
import torch.distributed as dist

from . import _lib


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


NUM_SLOTS = 4   # receive slots of the fused exchange (epoch mod NUM_SLOTS)
MAX_FINISH_LAG = NUM_SLOTS // 2   # a push of epoch e needs this rank's finish of e - MAX_FINISH_LAG


def slot_of_epoch(epoch: int) -> int:
    """Receive slot that the pushes of `epoch` write (epochs count from 1)."""
    return epoch % NUM_SLOTS


def push_allowed(epoch: int, finished_epoch: int) -> bool:
    """May this rank push `epoch`, given that its own finishes up to `finished_epoch` are
    complete?  The slot that the push overwrites at a peer was last read by that peer's
    finish of epoch - NUM_SLOTS, which is complete once this rank's finish of
    epoch - MAX_FINISH_LAG is (that finish needed the peer's push of the same epoch, which
    the peer issued after its own finish of epoch - 2 * MAX_FINISH_LAG)."""
    return finished_epoch >= epoch - MAX_FINISH_LAG


class GradExchange:
    """Peer-memory buffers for the fused column-reduce + all-reduce of [dgamma | dbeta].

    Pass an instance as ``grad_exchange=`` to ``fused_layer_norm_grad_op`` /
    ``fused_instance_norm_grad_op``: the last kernel of the backward pass then writes this
    rank's parameter-gradient vector into every rank's receive buffer over NVLink and adds
    the ``world`` vectors in rank order, so the op returns the global sums and no separate
    collective runs.  Every rank must make the same sequence of calls (same F).

    The receive buffers come from torch's symmetric memory (one allocation per rank, mapped
    into every peer).  Without a process group (single GPU) plain device
    memory is used and the exchange degenerates to a copy through the rank's own buffer.
    """

    def __init__(self, features: int, device: torch.device, group=None, deferred: bool = False,
                 device_epochs: bool = False):
        """deferred=True: the backward op only pushes this rank's vector; call finish()
        (typically on a side stream, see bench.py) to wait for the peers and obtain the sums.
        Start the backward op of step e only after finish() of step e - 2 has completed on
        this rank: there are four receive slots (slot_of_epoch), and a finish that lags its
        push by L steps needs 2L of them.  An instance is bound to one feature count.
        device_epochs=True: the kernels count the epochs in device memory, which lets the
        calls be captured in a CUDA graph and replayed (every rank must choose the same)."""
        lib = _lib.load()
        self.deferred = bool(deferred)
        self.features = int(features)
        if self.features % 2:
            raise ValueError("the fused exchange needs an even number of features")
        self.device = torch.device(device)
        distributed = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(group) if distributed else 1
        self.rank = dist.get_rank(group) if distributed else 0
        if self.world > _lib.NVN_DP_MAX_RANKS:
            raise ValueError(f"at most {_lib.NVN_DP_MAX_RANKS} ranks")
        recv_bytes = lib.nvn_dp_recv_bytes(self.features, self.world)
        self.epoch = 0
        if self.world > 1:
            import torch.distributed._symmetric_memory as symm_mem
            grp = group if group is not None else dist.group.WORLD
            self._recv = symm_mem.empty(recv_bytes // 4, dtype=torch.int32, device=self.device)
            self._recv.zero_()
            self._h_recv = symm_mem.rendezvous(self._recv, grp)
            recv_ptrs = list(self._h_recv.buffer_ptrs)
            torch.cuda.synchronize(self.device)
            dist.barrier(group)  # every rank's buffer is zero before anyone pushes
        else:
            self._recv = torch.zeros(recv_bytes // 4, dtype=torch.int32, device=self.device)
            recv_ptrs = [self._recv.data_ptr()]
        self._comm = _lib.DpComm()
        self._comm.rank = self.rank
        self._comm.world = self.world
        self._comm.defer = 1 if self.deferred else 0
        self._epochs = torch.zeros(4, dtype=torch.int32, device=self.device) if device_epochs else None
        self._comm.device_epochs = self._epochs.data_ptr() if device_epochs else None
        for i in range(self.world):
            self._comm.recv[i] = recv_ptrs[i]

    def next_comm(self, features: int | None = None):
        """ctypes pointer to the nvn_dp_comm for the next call (advances the epoch).
        `features` is the caller's feature count: the receive buffers are laid out for the
        count given at construction and cannot serve another."""
        if features is not None and int(features) != self.features:
            raise ValueError(f"this GradExchange was built for {self.features} features, "
                             f"the op has {features}: use one exchange per feature count")
        self.epoch += 1
        self._comm.epoch = self.epoch
        return ctypes.byref(self._comm)

    def finish(self, dgamma: torch.Tensor, dbeta: torch.Tensor, stream=None) -> None:
        """Deferred mode: complete the exchange of the most recent backward call into
        dgamma / dbeta on `stream` (default: the current stream)."""
        st = stream if stream is not None else torch.cuda.current_stream(self.device)
        with torch.cuda.device(self.device):
            rc = _lib.load().nvn_dp_finish(self.features, ctypes.byref(self._comm),
                                           dgamma.data_ptr(), dbeta.data_ptr(), st.cuda_stream)
        if rc != _lib.NVN_OK:
            raise RuntimeError(f"nvn_dp_finish: {_lib.status_string(rc)}")
