"""Fused column-reduce + all-reduce over peer memory (nvn_ln_bwd_dp / nvn_in_bwd_dp).

On one GPU the exchange runs with world == 1 through the same kernel (own buffer, own
flags).  With two or more GPUs, two ranks are started as child processes over NCCL; each
compares the fused result with the unsharded gradients.  Nothing here makes a GPU wait for
a peer that is not there: every rank runs the same calls, and the device-side waits are
bounded in any case.
"""
import os
import subprocess
import sys

import pytest
import torch

import atex_b200 as A
from atex_b200 import _lib, sharding
from atex_b200 import testing as T

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_world_one_exchange_equals_the_plain_backward(lib):
    dev = torch.device("cuda:0")
    for (N, D, dtype) in [(1000, 4096, "bf16"), (333, 128, "f16"), (64, 1026, "f32")]:
        g = torch.Generator().manual_seed(N)
        dt = T.TORCH_DTYPE[dtype]
        x = torch.randn(N, D, generator=g).to(dt).to(dev)
        dy = torch.randn(N, D, generator=g).to(dt).to(dev)
        gamma = (torch.rand(D, generator=g) + 0.5).to(dev)
        y, m, s = A.fused_layer_norm_op(x, gamma, torch.zeros_like(gamma))
        ref = A.fused_layer_norm_grad_op(dy, x, gamma, m, s)
        ex = sharding.GradExchange(D, dev)
        for _ in range(5):  # epochs 1..5: every receive slot gets used
            got = A.fused_layer_norm_grad_op(dy, x, gamma, m, s, grad_exchange=ex)
            torch.cuda.synchronize()
            for a, b in zip(got, ref):
                assert torch.equal(a, b)
        # deferred mode: push in the backward op, finish as a second launch
        exd = sharding.GradExchange(D, dev, deferred=True)
        for _ in range(3):
            dx, dg, db = A.fused_layer_norm_grad_op(dy, x, gamma, m, s, grad_exchange=exd)
            exd.finish(dg, db)
            torch.cuda.synchronize()
            assert torch.equal(dx, ref[0]) and torch.equal(dg, ref[1]) and torch.equal(db, ref[2])
    # InstanceNorm, both layouts
    for cf in (True, False):
        shape = (3, 16, 20, 20) if cf else (3, 20, 20, 16)
        fmt = "NC..." if cf else "N...C"
        x = torch.randn(shape, device=dev, dtype=torch.float16)
        dy = torch.randn(shape, device=dev, dtype=torch.float16)
        gamma = torch.rand(16, device=dev) + 0.5
        y, m, s = A.fused_instance_norm_op(x, gamma, torch.zeros_like(gamma), data_format=fmt)
        ref = A.fused_instance_norm_grad_op(dy, x, gamma, m, s, data_format=fmt)
        ex = sharding.GradExchange(16, dev)
        got = A.fused_instance_norm_grad_op(dy, x, gamma, m, s, data_format=fmt, grad_exchange=ex)
        torch.cuda.synchronize()
        for a, b in zip(got, ref):
            assert torch.equal(a, b)
    assert lib.nvn_device_status() == _lib.NVN_OK


def test_device_side_epochs_let_the_exchange_replay_from_a_cuda_graph(lib):
    """With nvn_dp_comm::device_epochs the kernels count the epochs themselves: a CUDA graph
    that holds backward calls with the exchange (whose arguments repeat on every replay) can
    be replayed any number of times.  world == 1: the rank exchanges with itself through the
    same kernels, slots and polls."""
    dev = torch.device("cuda:0")
    N, D = 1500, 2048
    g = torch.Generator().manual_seed(11)
    x = torch.randn(N, D, generator=g).bfloat16().to(dev)
    dy = torch.randn(N, D, generator=g).bfloat16().to(dev)
    gamma = (torch.rand(D, generator=g) + 0.5).to(dev)
    y, m, s = A.fused_layer_norm_op(x, gamma, torch.zeros_like(gamma))
    ref = A.fused_layer_norm_grad_op(dy, x, gamma, m, s)
    for deferred in (False, True):
        ex = sharding.GradExchange(D, dev, deferred=deferred, device_epochs=True)
        dx = torch.empty_like(x)
        grads = (torch.empty_like(gamma), torch.empty_like(gamma))

        def steps(k):
            for _ in range(k):
                A.fused_layer_norm_grad_op(dy, x, gamma, m, s, grad_exchange=ex, out=dx, out_grads=grads)
                if deferred:
                    ex.finish(grads[0], grads[1])
        cap = torch.cuda.Stream()
        with torch.cuda.stream(cap):
            steps(2)                      # eager first: epochs 1, 2
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=cap):
            steps(3)                      # three epochs per replay: slots wrap around
        for _ in range(5):
            grads[0].zero_(); grads[1].zero_(); dx.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(dx, ref[0]) and torch.equal(grads[0], ref[1]) and torch.equal(grads[1], ref[2])
        steps(1)                          # and eager again after the replays
        torch.cuda.synchronize()
        assert torch.equal(grads[0], ref[1])
        assert int(ex._epochs[0].item()) == 2 + 3 * 5 + 1
    assert lib.nvn_device_status() == _lib.NVN_OK


def test_dp_entry_points_validate_their_communicator(lib):
    c = _lib.DpComm()
    c.rank, c.world, c.epoch = 0, 1, 1  # null buffers
    import ctypes
    st = lib.nvn_ln_bwd_dp(0, None, None, None, None, None, 4, 8, None, None, None, None, 0,
                           ctypes.byref(c), None)
    assert st == _lib.NVN_ERR_INVALID_ARGUMENT
    assert lib.nvn_dp_recv_bytes(4096, 8) == 4 * 8 * 8192 * 8
    with pytest.raises(ValueError):
        sharding.GradExchange(7, torch.device("cuda:0"))


_WORKER = r"""
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["NVN_ROOT"])
import atex_b200 as A
from atex_b200 import sharding, testing as T, _lib
rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank); dev = torch.device("cuda", rank)
dist.init_process_group("nccl", device_id=dev)
N, D = 2048, 4096
g = torch.Generator().manual_seed(1)
x = torch.randn(N, D, generator=g).bfloat16(); dy = torch.randn(N, D, generator=g).bfloat16()
gamma = torch.rand(D, generator=g) + 0.5
a, b = sharding.shard_range(N, rank, world)
xs, dys, gd = x[a:b].to(dev), dy[a:b].to(dev), gamma.to(dev)
y, m, s = A.fused_layer_norm_op(xs, gd, torch.zeros_like(gd))
ex = sharding.GradExchange(D, dev)
ok = True
for it in range(4):
    dx, dg, db = A.fused_layer_norm_grad_op(dys, xs, gd, m, s, grad_exchange=ex)
    # reference: local gradients summed with NCCL
    _, dg_l, db_l = A.fused_layer_norm_grad_op(dys, xs, gd, m, s)
    dist.all_reduce(dg_l); dist.all_reduce(db_l)
    torch.cuda.synchronize()
    ok = ok and T.grad_param_error(dg, T.to_float64(dg_l))[0] <= 1.0
    ok = ok and T.grad_param_error(db, T.to_float64(db_l))[0] <= 1.0
    # all ranks hold bit-identical sums
    both = [torch.empty_like(dg) for _ in range(world)]
    dist.all_gather(both, dg)
    ok = ok and all(torch.equal(both[0], t) for t in both)
# deferred mode with the finish on a side stream, pipelined like the benchmark
exd = sharding.GradExchange(D, dev, deferred=True)
side = torch.cuda.Stream()
fin = [torch.cuda.Event() for _ in range(4)]
outs = []
for it in range(9):
    main = torch.cuda.current_stream()
    if it > 1:
        main.wait_event(fin[(it - 2) % 4])
    dx, dg, db = A.fused_layer_norm_grad_op(dys, xs, gd, m, s, grad_exchange=exd)
    pushed = torch.cuda.Event(); pushed.record(main)
    side.wait_event(pushed)
    exd.finish(dg, db, stream=side)
    fin[it % 4].record(side)
    outs.append((dg, db))
torch.cuda.synchronize()
_, dg_l, db_l = A.fused_layer_norm_grad_op(dys, xs, gd, m, s)
dist.all_reduce(dg_l); dist.all_reduce(db_l)
torch.cuda.synchronize()
for dg, db in outs:
    ok = ok and T.grad_param_error(dg, T.to_float64(dg_l))[0] <= 1.0
    ok = ok and T.grad_param_error(db, T.to_float64(db_l))[0] <= 1.0
    ok = ok and torch.equal(dg, outs[0][0])
ok = ok and _lib.load().nvn_device_status() == 0
flag = torch.tensor([1 if ok else 0], device=dev)
dist.all_reduce(flag, op=dist.ReduceOp.MIN)
dist.barrier(); dist.destroy_process_group()
sys.exit(0 if int(flag.item()) == 1 else 3)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_rank_fused_exchange_matches_nccl_allreduce(tmp_path):
    script = tmp_path / "dp_worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, NVN_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    port = 29600 + os.getpid() % 300
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
