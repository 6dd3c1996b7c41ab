#!/usr/bin/env python
"""Benchmark of the fused norm hot path: forward + backward HBM GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

One step = one forward + one backward pass of the workload's norm op over one batch
(plus, on N > 1 GPUs, the single all-reduce of [dgamma | dbeta]).  The default workload
is c2: LayerNorm, bf16 activations, [32768, 4096], fp32 gamma / beta.  Every rank owns
one full batch of that shape (weak scaling, the data-parallel training arrangement), so
`value` = N * algorithmic bytes / step time.

Prints ONE JSON line (rank 0).  Keys beyond the basic contract:
  roofline      achieved / peak HBM bandwidth of the dominant op (backward), timed with
                CUDA events inside the timed region
  cpu_baseline  the oracle's fp32 port of the reference CPU functors, timed on the host
  e2e           the same metric through the public API with pinned HOST buffers: each
                step copies x and dy to the device and dgamma / dbeta back
  clocks        nvidia-smi SM clocks and throttle reasons sampled during the timed region

`--impl reference` times the CPU port alone (the reference's own GPU op needs
TensorFlow headers, which this environment does not have).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# DRAM traffic of one backward launch (dram__bytes_read + dram__bytes_write) taken from the
# ncu capture summarised in profiles/rows_c2_ncu_full.md: 370.9 MB for 16384 rows of c2,
# i.e. 22 640 bytes per row (traffic grows in proportion to the rows).  Only known for c2.
NCU_BWD_TRAFFIC_BYTES_PER_ROW = {"c2": 370.93e6 / 16384}

NOMINAL_PEAK_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--workload", default="c2")
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    p.add_argument("--batch", type=int, default=0,
                   help="override the per-GPU batch extent (rows / batch items); used for small "
                        "profiler captures, not for reported numbers")
    p.add_argument("--graph", action="store_true",
                   help="replay the timed steps from a CUDA graph (removes host launch overhead; "
                        "meant for the small workloads c1 / c3c)")
    p.add_argument("--collective", default="fused-async", choices=["fused-async", "fused", "nccl"],
                   help="N > 1: 'fused' exchanges dgamma|dbeta inside the last backward kernel over "
                        "peer memory; 'fused-async' pushes there and completes the exchange on a "
                        "side stream while the next forward runs; 'nccl' is a separate NCCL all-reduce")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--no-e2e", action="store_true")
    return p.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_PEAK_GBS, "fallback"


# ---------------------------------------------------------------------------
# CPU arm: the oracle's fp32 port of the reference CPU functors
# ---------------------------------------------------------------------------
def _cpu_arrays(w, x, dy, gamma, beta):
    from atex_b200 import testing as T
    xn, dyn = T.to_numpy(x), T.to_numpy(dy)
    if w.op == "in":
        s3 = (x.shape[0], w.C, w.D) if w.channel_first else (x.shape[0], w.D, w.C)
        xn, dyn = xn.reshape(s3), dyn.reshape(s3)
    return xn, dyn, gamma.numpy(), beta.numpy()


def cpu_port_once(w, xn, dyn, g, b):
    """Seconds for one forward+backward of the sample on the host, all OpenMP threads."""
    from oracle import oracle
    t0 = time.perf_counter()
    if w.op == "ln":
        _, m, s = oracle.ln_fwd(xn, g, b, w.eps, w.dtype, fp32_port=True)
        oracle.ln_bwd(dyn, xn, g, m, s, w.dtype, fp32_port=True)
    else:
        _, m, s = oracle.in_fwd(xn, g, b, w.eps, w.channel_first, w.dtype, fp32_port=True)
        oracle.in_bwd(dyn, xn, g, m, s, w.channel_first, w.dtype, fp32_port=True)
    return time.perf_counter() - t0


def cpu_port_time(w, x, dy, gamma, beta, budget_s=12.0, max_reps=5):
    """Best-of seconds per forward+backward of the sample, within a time budget."""
    arrs = _cpu_arrays(w, x, dy, gamma, beta)
    cpu_port_once(w, *arrs)  # page in, spin up the OpenMP team
    times = []
    t_start = time.perf_counter()
    while len(times) < max_reps and (time.perf_counter() - t_start < budget_s or not times):
        times.append(cpu_port_once(w, *arrs))
    return min(times), len(times)


def cpu_sample(w, rows_cap_bytes=600e6):
    """A bounded slice of the workload for the CPU arm: whole batch entries, at most
    ~600 MB of activations."""
    from atex_b200 import testing as T
    per_entry = w.D * w.C * T.ELEM_SIZE[w.dtype] if w.op == "in" else w.D * T.ELEM_SIZE[w.dtype]
    n = int(max(1, min(w.N, rows_cap_bytes // (2 * per_entry))))
    return n


def run_reference_arm(args, rank, world):
    """`--impl reference`: the CPU port on rank 0; other ranks exit quietly."""
    if rank != 0:
        return
    from atex_b200 import testing as T
    from oracle import oracle
    oracle.build()
    w = T.WORKLOADS[args.workload]
    if args.batch:
        w = T.scaled(w, args.batch)
    n = cpu_sample(w)
    ws = T.scaled(w, n)
    x, dy = T.make_activations(ws)
    gamma, beta = T.make_params(w)
    # torchrun exports OMP_NUM_THREADS=1: ask for every core explicitly
    cores = oracle.set_num_threads(os.cpu_count() or 1)
    arrs = _cpu_arrays(ws, x, dy, gamma, beta)
    for _ in range(max(1, min(args.warmup, 3))):
        cpu_port_once(ws, *arrs)
    steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_port_once(ws, *arrs)
    per_step = (time.perf_counter() - t0) / steps
    gbs = ws.algorithmic_bytes() / per_step / 1e9
    sample = f"{n} of {w.N} batch entries of {w.name} per step, fwd+bwd, fp32 OpenMP port"
    line = {
        "impl": "reference",
        "metric": "norm_fwd_bwd_hbm_gbps", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": args.scaling,
        "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": workload_config(w, args, 1),
        "gelem_per_s": ws.elements / per_step / 1e9,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own fused op and the Keras/tfa composites need TensorFlow, which is "
                "not installed; this arm is the oracle's fp32 port of the reference CPU functors",
    }
    print(json.dumps(line), flush=True)


def workload_config(w, args, world):
    return {
        "workload": f"{w.name}: {'LayerNorm' if w.op == 'ln' else 'InstanceNorm ' + w.data_format} "
                    f"{w.dtype} {list(w.shape())} per GPU, eps={w.eps}, fwd+bwd",
        "per_gpu_batch": w.N, "global_batch": w.N * (world if args.scaling == "weak" else 1),
        "parallelism": f"dp{world}",
        "collective": ("none" if world == 1 else
                       "all-reduce of dgamma|dbeta fused into the column-reduce kernel (peer memory)"
                       if args.collective == "fused" else
                       "dgamma|dbeta pushed to peers by the column-reduce kernel, summed on a side stream"
                       if args.collective == "fused-async" else "NCCL all_reduce(dgamma|dbeta)"),
        "l2": "inputs larger than L2; buffer sets rotated",
    }


# ---------------------------------------------------------------------------
# clocks sampler
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows = [l for (t, l) in self.lines if t0 - 0.05 <= t <= t1 + 0.15] or [l for (_, l) in self.lines]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for l in rows:
            parts = [p.strip() for p in l.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm)}


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------
def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return

    import torch
    import torch.distributed as dist

    import atex_b200 as A
    from atex_b200 import _lib, sharding
    from atex_b200 import testing as T

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the norm ops have no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()

    w = T.WORKLOADS[args.workload]
    if args.batch:
        w = T.scaled(w, args.batch)
    if args.scaling == "weak":
        a, b = rank * w.N, (rank + 1) * w.N
        wl = w
        x_h, dy_h = T.make_activations(T.scaled(w, world * w.N), a, b, pin=True)
    else:
        a, b = sharding.shard_range(w.N, rank, world)
        wl = T.scaled(w, b - a)
        x_h, dy_h = T.make_activations(w, a, b, pin=True)
    gamma_h, beta_h = T.make_params(w)
    gamma, beta = gamma_h.to(dev), beta_h.to(dev)
    F = w.features

    # Resident inputs: enough rotating sets that consecutive steps never find their
    # inputs in the 126 MB L2.
    set_bytes = 2 * wl.elements * T.ELEM_SIZE[w.dtype]
    nsets = max(1, min(8, int(-(-400e6 // set_bytes))))
    xs = [x_h.to(dev)]
    dys = [dy_h.to(dev)]
    for k in range(1, nsets):
        xs.append(xs[0].roll(k, 0).contiguous())
        dys.append(dys[0].roll(k, 0).contiguous())
    # dgamma and dbeta are written next to each other, so one all-reduce covers both
    grad_buf = torch.empty(2 * F, dtype=torch.float32, device=dev)
    grad_views = (grad_buf[:F], grad_buf[F:])

    exchange = None
    deferred = args.collective == "fused-async"
    if world > 1 and args.collective != "nccl" and F % 2 == 0:
        exchange = sharding.GradExchange(F, dev, deferred=deferred)
    side = torch.cuda.Stream(device=dev) if (exchange is not None and deferred) else None
    fin_ev = [torch.cuda.Event() for _ in range(4)]
    push_ev = [torch.cuda.Event() for _ in range(4)]
    pending = {"n": 0}
    if w.op == "ln":
        def fwd(x):
            return A.fused_layer_norm_op(x, gamma, beta, axis=[-1], epsilon=w.eps)

        def bwd(dy, x, m, s):
            return A.fused_layer_norm_grad_op(dy, x, gamma, m, s, axis=[-1], out_grads=grad_views,
                                              grad_exchange=exchange)
    else:
        def fwd(x):
            return A.fused_instance_norm_op(x, gamma, beta, data_format=w.data_format, epsilon=w.eps)

        def bwd(dy, x, m, s):
            return A.fused_instance_norm_grad_op(dy, x, gamma, m, s, data_format=w.data_format,
                                                 out_grads=grad_views, grad_exchange=exchange)

    def step(i, ev=None):
        x, dy = xs[i % nsets], dys[i % nsets]
        y, m, s = fwd(x)
        if ev is not None:
            ev[0].record()
        main = torch.cuda.current_stream()
        if side is not None and pending["n"] > 1:
            # receive slots are reused every fourth step: staying at most two finishes
            # ahead keeps every slot's readers done before it is overwritten
            main.wait_event(fin_ev[(pending["n"] - 2) % 4])
        dx, dg, db = bwd(dy, x, m, s)
        if ev is not None:
            ev[1].record()
        if side is not None:
            k = pending["n"] % 4
            push_ev[k].record(main)
            side.wait_event(push_ev[k])
            exchange.finish(grad_views[0], grad_views[1], stream=side)
            fin_ev[k].record(side)
            pending["n"] += 1
        if world > 1 and exchange is None:
            dist.all_reduce(grad_buf)
        return y, dx, dg, db

    def drain():
        if side is not None and pending["n"] > 0:
            torch.cuda.current_stream().wait_event(fin_ev[(pending["n"] - 1) % 4])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(args.warmup, 3)):
        step(i)
    barrier()

    K = args.steps
    graph_ms = None
    if args.graph and world == 1:
        # One graph holds `nsets` consecutive steps (one per rotating buffer set).
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            for i in range(nsets):
                step(i)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for i in range(nsets):
                step(i)
        reps = max(1, -(-K // nsets))
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        g0.record()
        for _ in range(reps):
            graph.replay()
        g1.record()
        torch.cuda.synchronize()
        graph_ms = g0.elapsed_time(g1) / (reps * nsets)
    mids = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(K)]
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
        time.sleep(0.3)
    barrier()
    launches0 = lib.nvn_launch_count()
    t_wall0 = time.perf_counter()
    e0.record()
    # per-op events (for the roofline) on every `stride`-th step only: three timed events per
    # step cost a few microseconds of stream time each
    stride = 4 if K >= 16 else 1
    sampled = list(range(stride - 1, K, stride))  # not the first step after the idle barrier
    for i in range(K):
        if i % stride == stride - 1:
            starts[i].record()
            step(i, mids[i])
        else:
            step(i)
    drain()
    e1.record()
    barrier()
    t_wall1 = time.perf_counter()
    launches = lib.nvn_launch_count() - launches0
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None
    ms_total = e0.elapsed_time(e1)
    t_ms = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t_ms, op=dist.ReduceOp.MAX)
    ms_per_step = float(t_ms.item()) / K
    eager_ms_per_step = ms_per_step
    if graph_ms is not None:
        ms_per_step = graph_ms
    fwd_ms = statistics.mean(starts[i].elapsed_time(mids[i][0]) for i in sampled)
    bwd_ms = statistics.mean(mids[i][0].elapsed_time(mids[i][1]) for i in sampled)

    # ---- e2e: pinned host buffers in, parameter gradients out, every step ----
    e2e = None
    if not args.no_e2e:
        xd, dyd = torch.empty_like(xs[0]), torch.empty_like(dys[0])
        out_h = torch.empty(2 * F, dtype=torch.float32).pin_memory()

        def e2e_step():
            xd.copy_(x_h, non_blocking=True)
            dyd.copy_(dy_h, non_blocking=True)
            y, m, s = fwd(xd)
            dx, dg, db = bwd(dyd, xd, m, s)
            if side is not None:
                k = pending["n"] % 4
                push_ev[k].record(torch.cuda.current_stream())
                side.wait_event(push_ev[k])
                exchange.finish(grad_views[0], grad_views[1], stream=side)
                fin_ev[k].record(side)
                pending["n"] += 1
                drain()
            if world > 1 and exchange is None:
                dist.all_reduce(grad_buf)
            out_h.copy_(grad_buf, non_blocking=True)

        Ke = max(3, min(K, 20))
        for _ in range(3):
            e2e_step()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(Ke):
            e2e_step()
        s1.record()
        barrier()
        te = torch.tensor([s0.elapsed_time(s1)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        e2e_ms = float(te.item()) / Ke
        e2e = {"value": world * wl.algorithmic_bytes() / (e2e_ms * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": 2 * wl.elements * T.ELEM_SIZE[w.dtype],
               "d2h_bytes_per_step": 2 * F * 4, "ms_per_step": e2e_ms, "steps": Ke}

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    peak, peak_kind = measured_peak()
    total_bytes = world * wl.algorithmic_bytes()
    value = total_bytes / (ms_per_step * 1e-3) / 1e9
    s = T.ELEM_SIZE[w.dtype]
    R = wl.stat_rows
    bwd_bytes = 3 * wl.elements * s + 3 * F * 4 + 2 * R * 4
    fwd_bytes = 2 * wl.elements * s + 2 * F * 4 + 2 * R * 4
    bwd_gbs = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = fwd_bytes / (fwd_ms * 1e-3) / 1e9
    opn = 0 if w.op == "ln" else 2
    code = {"f32": 0, "f16": 1, "bf16": 2}[w.dtype]
    roofline = {
        "bound": "hbm", "achieved": bwd_gbs, "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak,
        "peak_kind": peak_kind,
        "traffic": (NCU_BWD_TRAFFIC_BYTES_PER_ROW[w.name] * wl.N
                    if w.name in NCU_BWD_TRAFFIC_BYTES_PER_ROW else None),
        "kernel": f"{w.op}_bwd: " + _lib.describe_plan(opn + 1, code, wl.N, w.C, w.D, int(w.channel_first)),
        "algorithmic_bytes_per_launch": bwd_bytes, "ms_per_launch": bwd_ms,
        "launches_timed": len(sampled),
        "forward": {"achieved": fwd_gbs, "frac": fwd_gbs / peak, "ms_per_launch": fwd_ms,
                    "algorithmic_bytes_per_launch": fwd_bytes,
                    "kernel": f"{w.op}_fwd: " + _lib.describe_plan(opn, code, wl.N, w.C, w.D, int(w.channel_first))},
        "step_frac_of_peak": (value / world) / peak,
    }

    cpu_baseline = None
    if not args.no_cpu_baseline and world == 1:
        from oracle import oracle
        oracle.build()
        cores = oracle.set_num_threads(os.cpu_count() or 1)
        n = cpu_sample(w)
        wsamp = T.scaled(w, n)
        sec, reps = cpu_port_time(wsamp, x_h[:n], dy_h[:n], gamma_h, beta_h)
        cpu_baseline = {"value": wsamp.algorithmic_bytes() / sec / 1e9, "unit": "GB/s",
                        "cores": cores, "kind": "port",
                        "sample": f"{n} of {w.N} batch entries of {w.name}, fwd+bwd, best of {reps}, "
                                  "fp32 OpenMP port of the reference CPU functors"}

    line = {
        "metric": "norm_fwd_bwd_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": world,
        "steps": K, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": w.dtype, "data": "synthetic",
        "config": workload_config(w, args, world),
        "gelem_per_s": world * wl.elements / (ms_per_step * 1e-3) / 1e9,
        "pct_of_nominal_8000": 100.0 * (value / world) / NOMINAL_PEAK_GBS,
        "pct_of_measured_peak": 100.0 * (value / world) / peak,
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        "gpu_launches": int(launches) * world, "clocks": clocks,
    }
    if graph_ms is not None:
        line["timing"] = "CUDA-graph replay of the steps; eager launch path: %.4f ms/step" % eager_ms_per_step
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
