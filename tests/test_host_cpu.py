"""Host-side mirror of the reference Python surface: validation, error text, wrapper
layers and the sharding helpers.  Everything here runs without a GPU; the ops must
refuse CPU tensors instead of falling back."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import atex_b200 as A
from atex_b200 import _lib, sharding
from atex_b200 import testing as T


def test_public_names_match_the_reference_package(lib):
    # atex/nv_norms/__init__.py:6-13
    for name in ("fused_layer_norm_op", "fused_layer_norm_grad_op", "fused_instance_norm_op",
                 "fused_instance_norm_grad_op", "_layer_norm_grad", "_instance_norm_grad",
                 "LayerNormalization", "InstanceNormalization"):
        assert hasattr(A, name)


def test_ops_refuse_cpu_tensors_loudly(lib):
    x = torch.zeros(4, 8)
    g = torch.ones(8)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        A.fused_layer_norm_op(x, g, g)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        A.fused_instance_norm_op(torch.zeros(2, 3, 4, 8), g, g)


def test_layer_norm_validation_messages(lib):
    x = torch.zeros(2, 3, 4)
    g4, g12 = torch.ones(4), torch.ones(12)
    with pytest.raises(A.InvalidArgumentError, match="axis is not packed from last dim"):
        A.fused_layer_norm_op(x, g4, g4, axis=[0])
    with pytest.raises(A.InvalidArgumentError, match="axis contains invalid value: 7"):
        A.fused_layer_norm_op(x, g4, g4, axis=[7])
    with pytest.raises(A.InvalidArgumentError, match="scale must have the same number of elements as the features of x, got 12 and 4"):
        A.fused_layer_norm_op(x, g12, g4, axis=[-1])
    with pytest.raises(A.InvalidArgumentError, match="offset must have the same number of elements"):
        A.fused_layer_norm_op(x, g4, g12, axis=[-1])
    with pytest.raises(A.InvalidArgumentError, match="at least 1-dimensional"):
        A.fused_layer_norm_op(torch.zeros(()), g4, g4)
    with pytest.raises(TypeError, match="float32"):
        A.fused_layer_norm_op(x, g4.half(), g4)
    with pytest.raises(TypeError):
        A.fused_layer_norm_op(x.double(), g4, g4)
    m = torch.zeros(6)
    with pytest.raises(A.InvalidArgumentError, match="x and y_backprop must have same shape"):
        A.fused_layer_norm_grad_op(torch.zeros(2, 3, 5), x, g4, m, m)
    with pytest.raises(A.InvalidArgumentError, match="saved mean must be 1-dimensional"):
        A.fused_layer_norm_grad_op(x, x, g4, m.reshape(2, 3), m)
    with pytest.raises(A.InvalidArgumentError, match="reserve_space_1 must have the same number of elements as the batches of x, got 5 and 6"):
        A.fused_layer_norm_grad_op(x, x, g4, torch.zeros(5), m)


def test_instance_norm_validation_messages(lib):
    x = torch.zeros(2, 3, 4, 5)
    g3, g5 = torch.ones(3), torch.ones(5)
    with pytest.raises(A.InvalidArgumentError, match="We only accept 'NC...' or 'N...C' data format"):
        A.fused_instance_norm_op(x, g3, g3, data_format="CHWN")
    with pytest.raises(A.InvalidArgumentError, match="at least 4-dimensional"):
        A.fused_instance_norm_op(torch.zeros(2, 3, 4), g3, g3, data_format="NC...")
    with pytest.raises(A.InvalidArgumentError, match="scale must have the same number of elements as the channels of x, got 5 and 3"):
        A.fused_instance_norm_op(x, g5, g3, data_format="NC...")
    with pytest.raises(A.InvalidArgumentError, match="scale must be 1-dimensional"):
        A.fused_instance_norm_op(x, g3.reshape(1, 3), g3, data_format="NC...")
    with pytest.raises(A.InvalidArgumentError, match="saved mean must be 2-dimensional"):
        A.fused_instance_norm_grad_op(x, x, g3, torch.zeros(6), torch.zeros(2, 3), data_format="NC...")
    with pytest.raises(A.InvalidArgumentError, match="batches\\*channels of x, got 4 and 6"):
        A.fused_instance_norm_grad_op(x, x, g3, torch.zeros(2, 2), torch.zeros(2, 3), data_format="NC...")


def test_wrapper_layers_keep_the_reference_interface(lib):
    ln = A.LayerNormalization(axis=[1, 2], epsilon=1e-5)
    ln.build((4, 3, 5))
    assert [tuple(v.shape) for v in ln.variables] == [(3, 5), (3, 5)]
    w = [np.full((3, 5), 2.0, np.float32), np.full((3, 5), -1.0, np.float32)]
    ln.set_weights(w)
    got = ln.get_weights()
    assert np.array_equal(got[0], w[0]) and np.array_equal(got[1], w[1])
    assert ln.get_config()["layer_norm"]["epsilon"] == 1e-5
    bad = A.LayerNormalization(axis=[2, 1])
    with pytest.raises(ValueError, match="sorted and unique axis"):
        bad(torch.zeros(4, 3, 5))
    inn = A.InstanceNormalization(axis=1)
    inn.build((2, 7, 4, 4))
    assert inn.gamma.shape == (7,) and inn.gamma.dtype == torch.float32
    with pytest.raises(ValueError, match="axis of 1 or -1"):
        A.InstanceNormalization(axis=2)(torch.zeros(2, 3, 4, 5))
    assert A.InstanceNormalization(axis=-1, epsilon=1e-3).get_config()["instance_norm"]["axis"] == -1


def test_shard_range_tiles_the_batch():
    for total in (0, 1, 7, 8, 64, 32768, 1048577):
        for world in (1, 2, 4, 8):
            prev = 0
            for r in range(world):
                a, b = sharding.shard_range(total, r, world)
                assert a == prev and b >= a
                prev = b
            assert prev == total
    with pytest.raises(ValueError):
        sharding.shard_range(8, 2, 2)


def test_workload_shards_are_slices_of_the_global_tensor():
    w = T.scaled(T.WORKLOADS["c2"], 2500)
    x, dy = T.make_activations(w)
    a, b = sharding.shard_range(w.N, 1, 2)
    xs, dys = T.make_activations(w, a, b)
    assert torch.equal(xs, x[a:b]) and torch.equal(dys, dy[a:b])
    w5 = T.scaled(T.WORKLOADS["c5"], 3)
    w5 = T.Workload(w5.name, w5.op, w5.dtype, 3, 64, 8, True, w5.eps, (8, 8), w5.x_kind, w5.gamma_kind, w5.index)
    x, _ = T.make_activations(w5)
    xs, _ = T.make_activations(w5, 1, 3)
    assert torch.equal(xs, x[1:3])
    assert x.shape == (3, 8, 8, 8)


def test_algorithmic_bytes_match_the_published_table():
    expect = {"c1": 83972096, "c2": 1342783488, "c3a": 1358957056, "c3b": 672157696,
              "c3c": 169086976, "c4": 5368713856, "c5": 2684621824}
    for k, v in expect.items():
        assert T.WORKLOADS[k].algorithmic_bytes() == v


def _gloo_worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import oracle_np
        rng = np.random.default_rng(5)
        N, D = 10, 12
        x = rng.normal(size=(N, D)).astype(np.float32)
        dy = rng.normal(size=(N, D)).astype(np.float32)
        g = rng.normal(size=D).astype(np.float32)
        _, mean, istd = oracle_np.ln_fwd(x, g, np.zeros(D), 1e-3)
        a, b = sharding.shard_range(N, rank, world)
        # each rank's local parameter gradients (stand-in for the CUDA op on its shard)
        _, dg, db = oracle_np.ln_bwd(dy[a:b], x[a:b], g, mean[a:b], istd[a:b])
        tg, tb = sharding.allreduce_param_grads(torch.from_numpy(dg.astype(np.float32)),
                                                torch.from_numpy(db.astype(np.float32)))
        _, dg_all, db_all = oracle_np.ln_bwd(dy, x, g, mean, istd)
        ok = np.allclose(tg.numpy(), dg_all, rtol=1e-5, atol=1e-5) and np.allclose(tb.numpy(), db_all, rtol=1e-5, atol=1e-5)
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_allreduce_of_param_grads_equals_the_unsharded_result():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]


def test_allreduce_is_identity_without_a_process_group():
    a, b = torch.ones(4), torch.zeros(4)
    ra, rb = sharding.allreduce_param_grads(a, b)
    assert ra is a and rb is b


# ---------------------------------------------------------------------------
# Receive-slot arithmetic of the deferred exchange (host logic of colreduce_dp.cu).
# A model of the protocol: every rank pushes epoch e into slot e % NUM_SLOTS of every peer
# and later "finishes" e (reads its own slot rows, which needs every rank's push of e).
# The contract: a rank pushes e only after its own finish of e - MAX_FINISH_LAG.  The model
# lets ranks run in random order under that contract and checks that no push ever
# overwrites a slot whose reader has not finished; with a larger lag the check must fail.
# ---------------------------------------------------------------------------
def _simulate_exchange(world, epochs, lag, seed):
    import random
    rnd = random.Random(seed)
    pushed = [0] * world      # highest epoch pushed by rank r
    finished = [0] * world    # highest epoch finished by rank r
    slot = [[[0] * world for _ in range(sharding.NUM_SLOTS)] for _ in range(world)]  # [owner][slot][src]
    while min(finished) < epochs:
        r = rnd.randrange(world)
        can_push = pushed[r] < epochs and finished[r] >= pushed[r] + 1 - lag
        e_fin = finished[r] + 1
        can_finish = e_fin <= pushed[r] and all(pushed[q] >= e_fin for q in range(world))
        choices = [c for c, okc in (("push", can_push), ("finish", can_finish)) if okc]
        if not choices:
            continue
        if rnd.choice(choices) == "push":
            e = pushed[r] + 1
            for owner in range(world):
                # the value being overwritten belongs to epoch e - NUM_SLOTS: its reader must be done
                if finished[owner] < e - sharding.NUM_SLOTS:
                    return False
                slot[owner][sharding.slot_of_epoch(e)][r] = e
            pushed[r] = e
        else:
            if any(slot[r][sharding.slot_of_epoch(e_fin)][q] != e_fin for q in range(world)):
                return False   # a needed value was overwritten before it was read
            finished[r] = e_fin
    return True


def test_documented_finish_lag_keeps_every_receive_slot_safe():
    assert sharding.MAX_FINISH_LAG * 2 == sharding.NUM_SLOTS
    for world in (2, 3, 8):
        for seed in range(40):
            assert _simulate_exchange(world, 40, sharding.MAX_FINISH_LAG, seed)
    assert sharding.push_allowed(3, 1) and not sharding.push_allowed(4, 1)


def test_a_longer_finish_lag_overwrites_unread_slots():
    # lagging the finish by three epochs with four slots is the hazard: some schedule breaks
    broke = any(not _simulate_exchange(2, 40, 3, seed) for seed in range(200))
    assert broke


def test_grad_exchange_is_bound_to_one_feature_count():
    ex = sharding.GradExchange.__new__(sharding.GradExchange)
    ex.features, ex.epoch, ex._comm = 64, 0, _lib.DpComm()
    ex.next_comm(64)
    assert ex.epoch == 1
    with pytest.raises(ValueError):
        ex.next_comm(128)


def test_workloads_from_shape_specs():
    w = T.workload_from_spec("c4")
    assert w is T.WORKLOADS["c4"]
    w = T.workload_from_spec("ln:12:96:bf16")
    assert (w.op, w.N, w.D, w.dtype) == ("ln", 12, 96, "bf16") and w.shape() == (12, 96)
    w = T.workload_from_spec("in:3:16:5x7:f16:nlc")
    assert w.shape() == (3, 5, 7, 16) and w.D == 35 and not w.channel_first
    w = T.workload_from_spec("in:3:16:5x7:f32:nc")
    assert w.shape() == (3, 16, 5, 7) and w.channel_first
    x, dy = T.make_activations(w)
    assert x.shape == (3, 16, 5, 7) and x.dtype == torch.float32
    with pytest.raises(ValueError):
        T.workload_from_spec("conv:1:2:3")
