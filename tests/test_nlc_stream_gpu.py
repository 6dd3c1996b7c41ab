"""The persistent channels-last InstanceNorm kernels (one cooperative launch per direction,
grid barrier per item, item tails kept in shared memory) on shapes far smaller than the
134 MB items they are meant for, so that every corner runs in seconds: items whose vector
count does not fill the last sweep, fewer sweeps than CTAs (some CTAs idle), a single
item, several items (ring hand-over from one item to the next), every dtype, C from one
to sixteen channel vectors; and two shapes with items of ~43 MB, the smallest size at which a
part of the item lies outside every CTA's ring after the first phase, so that the second phase
fetches chunks again on its backward walk.

The dispatcher only sends large items there (or mid-size items that it can spread over CTA
groups); NVN_FORCE_VARIANT=nlc=stream (read when the library is loaded) lifts the size rule
and stream_groups=K fixes the number of CTA groups, so the checks run in a child process.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

_WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["NVN_ROOT"]); sys.path.insert(0, os.path.join(os.environ["NVN_ROOT"], "tests"))
import torch
from atex_b200 import _lib
import _gpu_util as U
lib = _lib.load()
cases = [  # N, C, spatial, dtype
    (1, 32, (64, 64, 16), "f16"),      # 65536 voxels: 512 sweeps over 148 CTAs
    (3, 32, (61, 67), "f16"),          # 4087 voxels: ragged last sweep, fewer sweeps than CTAs
    (2, 8, (130, 129), "bf16"),        # one channel vector per voxel
    (2, 64, (40, 40, 40), "bf16"),     # 8 channel vectors, 64000 voxels
    (2, 16, (99, 101), "f32"),         # fp32: 4 channel vectors of 4
    (4, 128, (50, 31), "f16"),         # 16 channel vectors, C = 128
    (3, 256, (33, 29), "bf16"),        # 32 channel vectors, C = 256: warps share partial slots
    (2, 128, (45, 20), "f32"),         # fp32 at its widest: 32 channel vectors of 4
    (1, 32, (7, 3), "f16"),            # 21 voxels: almost every CTA is idle
    (5, 32, (128, 128), "f32"),        # several items back to back
    (2, 32, (101, 103, 64), "f16"),    # 42.6 MB items: more chunks per CTA than ring stages
    (3, 16, (150, 150, 30), "f32"),    # 43.2 MB items, fp32, odd item count
]
for i, (N, C, sp, dt) in enumerate(cases):
    code = {"f32": 0, "f16": 1, "bf16": 2}[dt]
    D = 1
    for s in sp: D *= s
    for op in (2, 3):
        plan = _lib.describe_plan(op, code, N, C, D, 0)
        assert plan.startswith("nlc persistent"), plan
    x, dy, g, b = U.rand_in(N, C, sp, False, dt, seed=100 + i)
    U.check_in(x, dy, g, b, 1e-3, False)
    # a second pass over the same buffers: bitwise repeatable
    import atex_b200 as A
    xd, gd, bd = x.cuda(), g.cuda(), b.cuda()
    y1, m1, s1 = A.fused_instance_norm_op(xd, gd, bd, data_format="N...C")
    y2, m2, s2 = A.fused_instance_norm_op(xd, gd, bd, data_format="N...C")
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and torch.equal(m1, m2) and torch.equal(s1, s2)
    dyd = dy.cuda()
    dx1, dg1, db1 = A.fused_instance_norm_grad_op(dyd, xd, gd, m1, s1, data_format="N...C")
    dx2, dg2, db2 = A.fused_instance_norm_grad_op(dyd, xd, gd, m1, s1, data_format="N...C")
    torch.cuda.synchronize()
    assert torch.equal(dx1, dx2) and torch.equal(dg1, dg2) and torch.equal(db1, db2)
assert lib.nvn_device_status() == 0
print("stream ok")
"""


@pytest.mark.parametrize("variant", ["nlc=stream", "nlc=stream,stream_block=256",
                                     "nlc=stream,stream_groups=3", "nlc=stream,stream_groups=8"])
def test_persistent_channels_last_kernels_on_small_and_ragged_items(tmp_path, variant):
    script = tmp_path / "stream_worker.py"
    script.write_text(_WORKER)
    env = dict(os.environ, NVN_ROOT=ROOT, NVN_FORCE_VARIANT=variant)
    r = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "stream ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]


def test_mid_size_items_run_in_cta_groups_by_default():
    """Items of a few MB: the dispatcher picks the persistent kernels with several CTA groups
    (each group its own items and its own barrier); parity and repeatability as above."""
    import torch
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import _gpu_util as U
    import atex_b200 as A
    from atex_b200 import _lib
    lib = _lib.load()
    for i, (N, C, sp, dt) in enumerate([(8, 32, (64, 64, 32), "f16"),     # 8.4 MB items
                                        (5, 64, (40, 40, 40), "bf16"),    # 8.2 MB, odd item count
                                        (3, 16, (96, 96, 60), "f32")]):   # 35 MB items, 3 of them
        code = {"f32": 0, "f16": 1, "bf16": 2}[dt]
        D = 1
        for v in sp:
            D *= v
        for op in (2, 3):
            plan = _lib.describe_plan(op, code, N, C, D, 0)
            assert plan.startswith("nlc persistent") and "groups=" in plan, plan
        x, dy, g, b = U.rand_in(N, C, sp, False, dt, seed=300 + i)
        U.check_in(x, dy, g, b, 1e-3, False)
        xd, dyd, gd, bd = x.cuda(), dy.cuda(), g.cuda(), b.cuda()
        y1, m1, s1 = A.fused_instance_norm_op(xd, gd, bd, data_format="N...C")
        y2, m2, s2 = A.fused_instance_norm_op(xd, gd, bd, data_format="N...C")
        d1 = A.fused_instance_norm_grad_op(dyd, xd, gd, m1, s1, data_format="N...C")
        d2 = A.fused_instance_norm_grad_op(dyd, xd, gd, m1, s1, data_format="N...C")
        torch.cuda.synchronize()
        assert torch.equal(y1, y2) and torch.equal(m1, m2) and torch.equal(s1, s2)
        assert all(torch.equal(a, b_) for a, b_ in zip(d1, d2))
    assert lib.nvn_device_status() == 0


_ROW_WORKER = r"""
import os, sys
sys.path.insert(0, os.environ["NVN_ROOT"]); sys.path.insert(0, os.path.join(os.environ["NVN_ROOT"], "tests"))
import torch
from atex_b200 import _lib
import atex_b200 as A
import _gpu_util as U
lib = _lib.load()
cases = [  # N, C, spatial, dtype: channel-first rows wider than the row-cached kernels take
    (2, 4, (100, 101, 64), "f16"),     # 8 rows of 1.29 MB, not a whole number of chunks
    (3, 8, (128, 128, 40), "bf16"),    # 24 rows of 1.31 MB
    (2, 16, (70, 60, 64), "f32"),      # 32 rows of 1.07 MB, fp32
    (1, 3, (90, 90, 90), "f16"),       # 3 rows: fewer rows than CTA groups wanted
]
for i, (N, C, sp, dt) in enumerate(cases):
    code = {"f32": 0, "f16": 1, "bf16": 2}[dt]
    D = 1
    for s in sp: D *= s
    for op in (2, 3):
        plan = _lib.describe_plan(op, code, N, C, D, 1)
        assert plan.startswith("rows persistent"), plan
    x, dy, g, b = U.rand_in(N, C, sp, True, dt, seed=400 + i)
    U.check_in(x, dy, g, b, 1e-3, True)
    xd, dyd, gd, bd = x.cuda(), dy.cuda(), g.cuda(), b.cuda()
    y1, m1, s1 = A.fused_instance_norm_op(xd, gd, bd, data_format="NC...")
    y2, m2, s2 = A.fused_instance_norm_op(xd, gd, bd, data_format="NC...")
    d1 = A.fused_instance_norm_grad_op(dyd, xd, gd, m1, s1, data_format="NC...")
    d2 = A.fused_instance_norm_grad_op(dyd, xd, gd, m1, s1, data_format="NC...")
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and torch.equal(m1, m2) and torch.equal(s1, s2)
    assert all(torch.equal(p, q) for p, q in zip(d1, d2))
assert lib.nvn_device_status() == 0
print("rows ok")
"""


@pytest.mark.parametrize("variant", ["nlc=stream", "nlc=stream,stream_groups=5"])
def test_persistent_kernels_in_row_mode_on_channel_first_rows(tmp_path, variant):
    """InstanceNorm "NC..." rows of a MB and more run the persistent kernels in row mode (a
    row is an item of one channel vector per voxel); forced for every batch size here."""
    script = tmp_path / "row_worker.py"
    script.write_text(_ROW_WORKER)
    env = dict(os.environ, NVN_ROOT=ROOT, NVN_FORCE_VARIANT=variant)
    r = subprocess.run([sys.executable, str(script)], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "rows ok" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
