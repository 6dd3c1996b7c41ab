#!/usr/bin/env python
"""Benchmark of the fused norm hot path: forward + backward HBM GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl ours|reference]

One step = one forward + one backward pass of the workload's norm op over one batch (plus,
on N > 1 GPUs, the single exchange of [dgamma | dbeta]).  The headline workload is c2:
LayerNorm, bf16 activations, [32768, 4096], fp32 gamma / beta.

Scaling.  On N > 1 GPUs the FIXED global batch is sharded over the ranks by default
("scaling": "strong": c2's 32768 rows become 4096 rows per rank at N = 8); the same line
carries the weak-scaling result (every rank a full batch) as the sub-record `weak`, the
compute / exchange split of a step, and `dp_check`: the exchanged parameter gradients
compared, outside the timed region, with one NCCL all-reduce of the local ones.

Prints ONE JSON line (rank 0).  Keys beyond the basic contract:
  roofline      achieved / peak HBM bandwidth of the dominant op (backward), timed with
                CUDA events inside the timed region
  per_config    (N = 1) every benchmark configuration c1 ... c5 in the same run: eager and
                CUDA-graph-replayed ms per step, GB/s of algorithmic bytes, fraction of the
                measured and of the nominal peak, forward / backward split, the kernel plans;
                `worst_frac` is the smallest fraction of the measured peak among them
  cpu_baseline  the oracle's fp32 port of the reference CPU functors, timed on the host
  e2e           the same metric through the public API with pinned HOST buffers: each step
                copies x and dy to the device and y, dx, dgamma and dbeta back; uploads,
                kernels and downloads run on three streams over two buffer sets, so the
                copies of neighbouring steps overlap (PCIe is full duplex)
  clocks        nvidia-smi SM clocks and throttle reasons sampled during the timed region

`--impl reference` times the CPU port alone (the reference's own fused op and the Keras /
tfa composites need TensorFlow, which this environment does not have).
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

# DRAM traffic (dram__bytes_read + dram__bytes_write) of one launch of the dominant backward
# kernel, per row / batch item, from ncu captures of reduced batches (traffic grows in
# proportion to the batch).  c2: 268.6 MB read + 102.3 MB written for 16384 rows.
NCU_BWD_TRAFFIC_BYTES_PER_ENTRY = {"c2": (268.6e6 + 102.3e6) / 16384}

NOMINAL_PEAK_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0
CONFIGS = ("c1", "c2", "c3a", "c3b", "c3c", "c4", "c5")


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=50)
    p.add_argument("--warmup", type=int, default=5)
    p.add_argument("--workload", default="c2",
                   help="a benchmark configuration (c1 ... c5) or a shape: ln:N:D:dtype, "
                        "in:N:C:S1xS2x..:dtype:nlc|nc")
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--scaling", default="auto", choices=["auto", "weak", "strong"],
                   help="N > 1: 'strong' (default) shards the fixed global batch, 'weak' gives every "
                        "rank a full batch")
    p.add_argument("--batch", type=int, default=0,
                   help="override the global batch extent (rows / batch items); used for small "
                        "profiler captures, not for reported numbers")
    p.add_argument("--launch", default="graph", choices=["graph", "eager"],
                   help="'graph' (default): the K timed steps are replayed from a CUDA graph, as a "
                        "training loop at this granularity would run them (the Python host layer "
                        "costs ~35 us per step, more than a rank's GPU time at 8 GPUs); 'eager': the "
                        "headline is the eager launch loop.  The other one is reported beside it.")
    p.add_argument("--collective", default="fused-async", choices=["fused-async", "fused", "nccl"],
                   help="N > 1: 'fused' exchanges dgamma|dbeta inside the last backward kernel over "
                        "peer memory; 'fused-async' pushes there and completes the exchange on a "
                        "side stream while the next forward runs; 'nccl' is a separate NCCL all-reduce")
    p.add_argument("--configs", default="all",
                   help="N = 1: comma-separated configurations for per_config ('all', 'none', or e.g. c1,c3c)")
    p.add_argument("--ref-shapes", action="store_true",
                   help="N = 1: time forward + backward on the shapes of the reference's own benchmark "
                        "scripts (fp16) and print them beside its published A100 / H100 figures")
    p.add_argument("--residual", action="store_true",
                   help="N = 1: time only the residual-add LayerNorm forward on the c2 shape (--batch rows)")
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


def scaling_mode(args, world):
    if args.scaling != "auto":
        return args.scaling
    return "strong"


def workload_config(w, args, world):
    """The `config` object; a function of the command line only, so that both arms of one
    (N, workload) pair print the same one."""
    mode = scaling_mode(args, world)
    per_gpu = w.N if mode == "weak" else -(-w.N // world)
    return {
        "workload": f"{w.name}: {'LayerNorm' if w.op == 'ln' else 'InstanceNorm ' + w.data_format} "
                    f"{w.dtype} {list(w.shape())} global batch, eps={w.eps}, fwd+bwd",
        "per_gpu_batch": per_gpu, "global_batch": w.N * (world if mode == "weak" else 1),
        "parallelism": f"dp{world}",
        "collective": ("none" if world == 1 else
                       "all-reduce of dgamma|dbeta fused into the column-reduce kernel (peer memory)"
                       if args.collective == "fused" else
                       "dgamma|dbeta pushed to peers by the column-reduce kernel, summed on a side stream"
                       if args.collective == "fused-async" else "NCCL all_reduce(dgamma|dbeta)"),
        "l2": "inputs larger than L2; buffer sets rotated",
    }


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


def cpu_sample(w, cap_bytes=600e6):
    """A bounded slice of the workload for the CPU arm: whole batch entries, at most
    ~600 MB of activations."""
    from atex_b200 import testing as T
    per_entry = w.D * w.C * T.ELEM_SIZE[w.dtype] if w.op == "in" else w.D * T.ELEM_SIZE[w.dtype]
    return int(max(1, min(w.N, cap_bytes // (2 * per_entry))))


def run_reference_arm(args, rank, world):
    """`--impl reference`: the CPU port on rank 0, on the arm's own workload and step count;
    other ranks exit quietly.  Every step is one pass over a bounded sample of the global
    batch, sized from a calibration pass so that warm-up + steps stay within ~90 s."""
    if rank != 0:
        return
    from atex_b200 import testing as T
    from oracle import oracle
    oracle.build()
    w = T.workload_from_spec(args.workload)
    if args.batch:
        w = T.scaled(w, args.batch)
    mode = scaling_mode(args, world)
    gamma, beta = T.make_params(w)
    # torchrun exports OMP_NUM_THREADS=1: ask for every core explicitly
    cores = oracle.set_num_threads(os.cpu_count() or 1)
    steps = max(1, args.steps)
    warmup = max(0, args.warmup)
    # calibration on a small slice -> entries per step that fit the budget
    n0 = max(1, min(w.N, cpu_sample(w, cap_bytes=64e6)))
    w0 = T.scaled(w, n0)
    x0, dy0 = T.make_activations(w0)
    arrs0 = _cpu_arrays(w0, x0, dy0, gamma, beta)
    cpu_port_once(w0, *arrs0)
    per_entry_s = min(cpu_port_once(w0, *arrs0) for _ in range(2)) / n0
    budget_s = 90.0
    n = int(budget_s / ((steps + warmup) * per_entry_s))
    n = max(1, min(n, cpu_sample(w), w.N))
    ws = T.scaled(w, n)
    x, dy = T.make_activations(ws)
    arrs = _cpu_arrays(ws, x, dy, gamma, beta)
    for _ in range(warmup):
        cpu_port_once(ws, *arrs)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_port_once(ws, *arrs)
    per_step = (time.perf_counter() - t0) / steps
    gbs = ws.algorithmic_bytes() / per_step / 1e9
    sample = (f"{n} of {w.N} batch entries of {w.name} per step, fwd+bwd, fp32 OpenMP port of the "
              "reference CPU functors")
    line = {
        "impl": "reference",
        "metric": "norm_fwd_bwd_hbm_gbps", "value": gbs, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": per_step * 1e3, "higher_is_better": True, "scaling": mode,
        "vs_baseline": None, "dtype": w.dtype, "data": "synthetic",
        "config": workload_config(w, args, world),
        "gelem_per_s": ws.elements / per_step / 1e9,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own fused op and the Keras/tfa composites need TensorFlow, which is "
                "not installed; this arm is the oracle's fp32 port of the reference CPU functors",
    }
    print(json.dumps(line), flush=True)


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
class Runner:
    """Forward + backward of one workload on one device over rotating, preallocated buffer
    sets (enough of them that consecutive steps never find their inputs in the 126 MB L2).
    Outputs are preallocated too, so a steady-state step allocates nothing."""

    def __init__(self, w, x0, dy0, gamma, beta, exchange=None, deferred=False, nccl=False):
        import torch
        import atex_b200 as A
        from atex_b200 import testing as T
        self.torch, self.A, self.w = torch, A, w
        self.dev = x0.device
        self.gamma, self.beta = gamma, beta
        n_local = x0.shape[0]
        self.wl = T.scaled(w, n_local)
        F = w.features
        set_bytes = 2 * self.wl.elements * T.ELEM_SIZE[w.dtype]
        self.nsets = max(1, min(8, int(-(-400e6 // max(set_bytes, 1)))))
        self.xs, self.dys = [x0], [dy0]
        for k in range(1, self.nsets):
            self.xs.append(x0.roll(k, 0).contiguous())
            self.dys.append(dy0.roll(k, 0).contiguous())
        self.ys = [torch.empty_like(x0) for _ in range(self.nsets)]
        self.dxs = [torch.empty_like(x0) for _ in range(self.nsets)]
        R = self.wl.stat_rows
        stat_shape = (R,) if w.op == "ln" else (n_local, w.C)
        self.stats = [(torch.empty(stat_shape, dtype=torch.float32, device=self.dev),
                       torch.empty(stat_shape, dtype=torch.float32, device=self.dev))
                      for _ in range(self.nsets)]
        # dgamma and dbeta are written next to each other, so one all-reduce covers both
        self.grad_buf = torch.empty(2 * F, dtype=torch.float32, device=self.dev)
        self.grad_views = (self.grad_buf[:F], self.grad_buf[F:])
        self.exchange, self.deferred, self.nccl = exchange, deferred and exchange is not None, nccl
        self.side = torch.cuda.Stream(device=self.dev) if self.deferred else None
        self.fin_ev = [torch.cuda.Event() for _ in range(4)]
        self.push_ev = [torch.cuda.Event() for _ in range(4)]
        self.pending = 0

    def fwd(self, i, x=None, out=None):
        k = i % self.nsets
        w = self.w
        x = self.xs[k] if x is None else x
        out = self.ys[k] if out is None else out
        if w.op == "ln":
            return self.A.fused_layer_norm_op(x, self.gamma, self.beta, axis=[-1], epsilon=w.eps,
                                              out=out, out_stats=self.stats[k])
        return self.A.fused_instance_norm_op(x, self.gamma, self.beta, data_format=w.data_format,
                                             epsilon=w.eps, out=out, out_stats=self.stats[k])

    def bwd(self, i, x=None, dy=None, exchange=True, out=None):
        k = i % self.nsets
        w = self.w
        x = self.xs[k] if x is None else x
        dy = self.dys[k] if dy is None else dy
        out = self.dxs[k] if out is None else out
        m, s = self.stats[k]
        ex = self.exchange if exchange else None
        if w.op == "ln":
            return self.A.fused_layer_norm_grad_op(dy, x, self.gamma, m, s, axis=[-1],
                                                   out_grads=self.grad_views, grad_exchange=ex,
                                                   out=out)
        return self.A.fused_instance_norm_grad_op(dy, x, self.gamma, m, s, data_format=w.data_format,
                                                  out_grads=self.grad_views, grad_exchange=ex,
                                                  out=out)

    def step(self, i, ev=None, x=None, dy=None, exchange=True, y_out=None, dx_out=None):
        torch = self.torch
        self.fwd(i, x, y_out)
        if ev is not None:
            ev[0].record()
        main = torch.cuda.current_stream()
        deferred = self.deferred and exchange
        if deferred and self.pending > 1:
            # a push of epoch e needs this rank's finish of e - 2 (four receive slots)
            main.wait_event(self.fin_ev[(self.pending - 2) % 4])
        self.bwd(i, x, dy, exchange, dx_out)
        if ev is not None:
            ev[1].record()
        if deferred:
            k = self.pending % 4
            self.push_ev[k].record(main)
            self.side.wait_event(self.push_ev[k])
            self.exchange.finish(self.grad_views[0], self.grad_views[1], stream=self.side)
            self.fin_ev[k].record(self.side)
            self.pending += 1
        if self.nccl and exchange:
            import torch.distributed as dist
            dist.all_reduce(self.grad_buf)

    def drain(self):
        if self.deferred and self.pending > 0:
            self.torch.cuda.current_stream().wait_event(self.fin_ev[(self.pending - 1) % 4])


def _time_loop(torch, fn, n, sync):
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync()
    e0.record()
    for i in range(n):
        fn(i)
    e1.record()
    sync()
    return e0.elapsed_time(e1) / n


def _graph_ms(torch, body, nsets, steps):
    """ms per body(i) when `nsets` consecutive calls are replayed from one CUDA graph."""
    cap = torch.cuda.Stream()
    with torch.cuda.stream(cap):
        for i in range(nsets):
            body(i)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=cap):
        for i in range(nsets):
            body(i)
    reps = max(2, -(-steps // nsets))
    for _ in range(2):
        graph.replay()
    ms = _time_loop(torch, lambda _i: graph.replay(), reps, torch.cuda.synchronize) / nsets
    del graph
    return ms


def device_inputs(w, dev, seed):
    """x, dy of the workload generated on the device (same distributions as the host
    generator of atex_b200.testing; used for the per-configuration sweep, whose inputs never
    leave the GPU)."""
    import torch
    from atex_b200 import testing as T
    g = torch.Generator(device=dev).manual_seed(seed)
    shape = w.shape()
    dt = T.TORCH_DTYPE[w.dtype]
    x = torch.randn(shape, generator=g, device=dev, dtype=torch.float32)
    if w.x_kind == "row_offset":
        x.mul_(4.0).add_(torch.randn((shape[0], 1), generator=g, device=dev))
    elif w.x_kind == "mean2_std3":
        x.mul_(3.0).add_(2.0)
    elif w.x_kind == "channel_scale":
        s = torch.rand(w.C, generator=g, device=dev) * 1.5 + 0.5
        x.mul_(s.reshape((1, w.C) + (1,) * (len(shape) - 2)) if w.channel_first else s)
    xo = x.to(dt)
    del x
    dy = torch.randn(shape, generator=g, device=dev, dtype=torch.float32).to(dt)
    return xo, dy


def measure_config(name, dev, peak, steps=20, host_calls=0):
    """One entry of `per_config`: the workload's forward + backward on one GPU, launched
    eagerly through the public API and replayed from CUDA graphs."""
    import torch
    from atex_b200 import _lib
    from atex_b200 import testing as T
    w = T.workload_from_spec(name)
    gamma_h, beta_h = T.make_params(w)
    gamma, beta = gamma_h.to(dev), beta_h.to(dev)
    x, dy = device_inputs(w, dev, 77 + w.index)
    r = Runner(w, x, dy, gamma, beta)
    sync = torch.cuda.synchronize
    for i in range(3):
        r.step(i)
    eager_ms = _time_loop(torch, r.step, steps, sync)
    graph_ms = _graph_ms(torch, r.step, r.nsets, steps)
    fwd_ms = _graph_ms(torch, r.fwd, r.nsets, steps)
    bwd_ms = _graph_ms(torch, r.bwd, r.nsets, steps)
    s = T.ELEM_SIZE[w.dtype]
    F, R, E = w.features, w.stat_rows, w.elements
    fwd_bytes = 2 * E * s + 2 * F * 4 + 2 * R * 4
    bwd_bytes = 3 * E * s + 3 * F * 4 + 2 * R * 4
    total = w.algorithmic_bytes()
    gbs = total / (graph_ms * 1e-3) / 1e9
    opn = 0 if w.op == "ln" else 2
    code = {"f32": 0, "f16": 1, "bf16": 2}[w.dtype]
    out = {
        "workload": f"{'LayerNorm' if w.op == 'ln' else 'InstanceNorm ' + w.data_format} {w.dtype} {list(w.shape())}",
        "eager_ms_per_step": eager_ms, "graph_ms_per_step": graph_ms,
        "gbps": gbs, "gelem_per_s": E / (graph_ms * 1e-3) / 1e9,
        "frac_of_measured": gbs / peak, "frac_of_nominal_8000": gbs / NOMINAL_PEAK_GBS,
        "eager_frac_of_measured": total / (eager_ms * 1e-3) / 1e9 / peak,
        "fwd": {"graph_ms": fwd_ms, "gbps": fwd_bytes / (fwd_ms * 1e-3) / 1e9,
                "frac_of_measured": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak,
                "plan": _lib.describe_plan(opn, code, w.N, w.C, w.D, int(w.channel_first))},
        "bwd": {"graph_ms": bwd_ms, "gbps": bwd_bytes / (bwd_ms * 1e-3) / 1e9,
                "frac_of_measured": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak,
                "plan": _lib.describe_plan(opn + 1, code, w.N, w.C, w.D, int(w.channel_first))},
        "algorithmic_bytes": total, "buffer_sets": r.nsets,
    }
    if name == "c4":
        # the two-phase channels-last kernels move x twice forward and x, dy twice backward
        # (one batch item exceeds L2): 8 tensor passes for the 5 counted
        moved = 8 * E * s
        out["frac_of_measured_by_bytes_moved_8_passes"] = moved / (graph_ms * 1e-3) / 1e9 / peak
    if host_calls:
        # host cost of one op call through the public API (launches are asynchronous; the
        # problem is small enough that the GPU keeps up with the issue rate)
        sync()
        t0 = time.perf_counter()
        for i in range(host_calls):
            r.fwd(i)
        t1 = time.perf_counter()
        for i in range(host_calls):
            r.bwd(i)
        t2 = time.perf_counter()
        sync()
        out["host_us_per_call"] = {"fwd": (t1 - t0) / host_calls * 1e6, "bwd": (t2 - t1) / host_calls * 1e6,
                                   "calls": host_calls}
    del r, x, dy
    torch.cuda.empty_cache()
    return out


# Shapes of the reference's benchmark scripts (benchmark_layer_norm.py:53-63,
# benchmark_instance_norm.py:58-69) with the "NV" column of its README (ms per training step
# of the fused op under mixed_float16, eager TensorFlow, wall clock: A100, H100).
REF_LN_SHAPES = [((10, 10000000), 3.36, 2.36), ((100, 1000000), 2.78, 1.78), ((1000, 100000), 2.81, 1.95),
                 ((10000, 10000), 4.50, 5.84), ((100000, 1000), 4.32, 4.73), ((1000000, 100), 6.33, 6.26),
                 ((10000000, 10), 13.82, 10.61), ((4, 400001), 0.59, 0.74), ((4, 10000001), 1.69, 1.15)]
REF_IN_SHAPES = [(2, 32, 6), (2, 32, 128), (2, 64, 128), (4, 32, 128), (4, 64, 64), (8, 32, 64), (8, 64, 64),
                 (8, 128, 64), (4, 256, 32), (8, 256, 32)]
REF_IN_NLC_MS = [(0.78, 0.70), (7.51, 6.05), (12.53, 8.69), (12.35, 8.70), (5.36, 4.63), (5.35, 4.66),
                 (7.65, 5.98), (12.33, 8.63), (3.76, 3.57), (5.01, 4.25)]
REF_IN_NC_MS = [(0.77, 0.69), (5.20, 3.85), (10.53, 7.57), (9.27, 6.16), (2.98, 2.17), (3.01, 2.17),
                (5.32, 3.51), (10.37, 6.38), (1.18, 0.91), (2.57, 1.71)]


def run_ref_shapes(dev, peak):
    """fp16 forward + backward on every shape of the reference's benchmark scripts: device time
    per step (eager launches through the public API, CUDA events, 20 steps after 10 warm-up
    steps as the scripts do) next to the published wall-clock figures of the fused TF op."""
    import torch
    import atex_b200 as A
    rows = []
    g = torch.Generator(device=dev).manual_seed(3)

    def time_steps(fn):
        for _ in range(10):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(20):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 20

    for shape, a100, h100 in REF_LN_SHAPES:
        x = torch.randn(shape, generator=g, device=dev, dtype=torch.float32).half()
        dy = torch.ones_like(x)                       # d(sum y)/dy, as in the script
        gamma = torch.ones(shape[1], device=dev)
        beta = torch.zeros(shape[1], device=dev)

        def step():
            y, m, s = A.fused_layer_norm_op(x, gamma, beta, axis=[1])
            A.fused_layer_norm_grad_op(dy, x, gamma, m, s, axis=[1])
        ms = time_steps(step)
        E = x.numel()
        rows.append({"op": "LayerNorm", "shape": list(shape), "ms": ms, "gbps": 10 * E / ms / 1e6,
                     "frac_of_measured": 10 * E / ms / 1e6 / peak, "ref_A100_ms": a100, "ref_H100_ms": h100})
        del x, dy
    for fmt, table in (("N...C", REF_IN_NLC_MS), ("NC...", REF_IN_NC_MS)):
        for (n, c, d), (a100, h100) in zip(REF_IN_SHAPES, table):
            shape = (n, d, d, d, c) if fmt == "N...C" else (n, c, d, d, d)
            x = torch.randn(shape, generator=g, device=dev, dtype=torch.float32).half()
            dy = torch.ones_like(x)
            gamma, beta = torch.ones(c, device=dev), torch.zeros(c, device=dev)

            def step():
                y, m, s = A.fused_instance_norm_op(x, gamma, beta, data_format=fmt)
                A.fused_instance_norm_grad_op(dy, x, gamma, m, s, data_format=fmt)
            ms = time_steps(step)
            E = x.numel()
            rows.append({"op": "InstanceNorm " + fmt, "shape": list(shape), "ms": ms, "gbps": 10 * E / ms / 1e6,
                         "frac_of_measured": 10 * E / ms / 1e6 / peak, "ref_A100_ms": a100, "ref_H100_ms": h100})
            del x, dy
            torch.cuda.empty_cache()
    return rows


def measure_residual(dev, peak, steps=20, rows=0):
    """Forward of the residual-add LayerNorm on the c2 shape: s = x + r and y = LN(s) in one
    pass.  Algorithmic bytes: x and r read, s and y written (4 tensor passes)."""
    import torch
    import atex_b200 as A
    from atex_b200 import testing as T
    w = T.WORKLOADS["c2"] if not rows else T.scaled(T.WORKLOADS["c2"], rows)
    gamma_h, beta_h = T.make_params(w)
    gamma, beta = gamma_h.to(dev), beta_h.to(dev)
    x, r = device_inputs(w, dev, 91)
    y, s_out = torch.empty_like(x), torch.empty_like(x)
    stats = (torch.empty(w.N, dtype=torch.float32, device=dev), torch.empty(w.N, dtype=torch.float32, device=dev))

    def body(_i):
        A.fused_layer_norm_residual_op(x, r, gamma, beta, axis=[-1], epsilon=w.eps, out=y, out_sum=s_out,
                                       out_stats=stats)
    ms = _graph_ms(torch, body, 1, steps)
    nbytes = 4 * w.elements * T.ELEM_SIZE[w.dtype] + 2 * w.D * 4 + 2 * w.N * 4
    del x, r, y, s_out
    torch.cuda.empty_cache()
    return {"workload": f"residual add + LayerNorm forward {w.dtype} {list(w.shape())}", "graph_ms": ms,
            "algorithmic_bytes": nbytes, "gbps": nbytes / ms / 1e6, "frac_of_measured": nbytes / ms / 1e6 / peak}


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
    mode = scaling_mode(args, world)
    peak, peak_kind = measured_peak()

    if args.residual:
        if rank == 0:
            rec = measure_residual(dev, peak, steps=args.steps, rows=args.batch)
            print(json.dumps({"metric": "residual_ln_fwd_hbm_gbps", "value": rec["gbps"], "unit": "GB/s",
                              "n_gpus": 1, "dtype": "bf16", "data": "synthetic", "higher_is_better": True,
                              "ms_per_step": rec["graph_ms"], "detail": rec}), flush=True)
        return
    if args.ref_shapes:
        if rank == 0:
            rows = run_ref_shapes(dev, peak)
            print(json.dumps({
                "metric": "ref_benchmark_shapes_fwd_bwd_ms", "unit": "ms", "n_gpus": 1, "dtype": "f16",
                "data": "synthetic", "higher_is_better": False,
                "value": sum(r["ms"] for r in rows),
                "note": "device time of fwd+bwd through the public API on the shapes of the reference's "
                        "benchmark scripts; ref_*_ms are the README's wall-clock figures of the fused TF op "
                        "on A100 / H100 (they include TensorFlow's eager overhead and a reduce_sum)",
                "shapes": rows}), flush=True)
        return

    w = T.workload_from_spec(args.workload)
    if args.batch:
        w = T.scaled(w, args.batch)
    gamma_h, beta_h = T.make_params(w)
    gamma, beta = gamma_h.to(dev), beta_h.to(dev)
    F = w.features

    def shard_inputs(kind):
        if kind == "weak":
            return T.make_activations(T.scaled(w, world * w.N), rank * w.N, (rank + 1) * w.N, pin=True)
        a, b = sharding.shard_range(w.N, rank, world)
        return T.make_activations(w, a, b, pin=True)

    x_h, dy_h = shard_inputs(mode)

    def make_runner(xh, dyh):
        exchange = None
        deferred = args.collective == "fused-async"
        if world > 1 and args.collective != "nccl" and F % 2 == 0:
            # device-side epochs: the exchange can be replayed from a CUDA graph
            exchange = sharding.GradExchange(F, dev, deferred=deferred, device_epochs=True)
        return Runner(w, xh.to(dev), dyh.to(dev), gamma, beta, exchange=exchange, deferred=deferred,
                      nccl=(world > 1 and exchange is None))

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(r, K, exchange=True):
        """ms per step of K eager steps, max over ranks (barrier + synchronize on both sides)."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(K):
            r.step(i, exchange=exchange)
        if exchange:
            r.drain()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1)) / K

    r = make_runner(x_h, dy_h)
    wl = r.wl
    W = max(args.warmup, 3)
    for i in range(W):
        r.step(i)
    r.drain()
    barrier()

    K = args.steps
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
            r.step(i, mids[i])
        else:
            r.step(i)
    r.drain()
    e1.record()
    barrier()
    t_wall1 = time.perf_counter()
    launches = lib.nvn_launch_count() - launches0
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None
    ms_per_step = max_over_ranks(e0.elapsed_time(e1)) / K
    eager_ms_per_step = ms_per_step
    fwd_ms = statistics.mean(starts[i].elapsed_time(mids[i][0]) for i in sampled)
    bwd_ms = statistics.mean(mids[i][0].elapsed_time(mids[i][1]) for i in sampled)
    # ---- the same K steps replayed from a CUDA graph ----
    def graph_timed(rr, exchange=True):
        """ms per step (max over ranks) of exactly K steps replayed from CUDA graphs - a graph of
        S steps (a whole number of turns through the buffer sets) replayed K // S times, then a
        graph of the K % S steps left over - or None when the steps cannot be captured (NCCL
        collective)."""
        if args.launch != "graph" or (rr.nccl and exchange):
            return None, 0
        S = min(K, rr.nsets * max(1, 32 // rr.nsets))
        reps, rem = divmod(K, S)
        cap = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(cap):
            for i in range(rr.nsets):
                rr.step(i, exchange=exchange)
            rr.drain()
        barrier()

        def capture(n):
            rr.pending = 0      # no wait on events recorded outside the capture
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=cap):
                for i in range(n):
                    rr.step(i, exchange=exchange)
                if exchange:
                    rr.drain()
            rr.pending = 0
            return g

        main = capture(S)
        tail = capture(rem) if rem else None
        for _ in range(2):
            main.replay()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        g0.record()
        for _ in range(reps):
            main.replay()
        if tail is not None:
            tail.replay()
        g1.record()
        barrier()
        ms = max_over_ranks(g0.elapsed_time(g1)) / K
        del main, tail
        return ms, S

    graph_ms, S = graph_timed(r)
    if graph_ms is not None:
        ms_per_step = graph_ms

    # ---- N > 1: compute / exchange split, correctness of the exchange, weak sub-record ----
    split = dp_check = weak = None
    if world > 1:
        # the same shard without any exchange, launched the same way as the headline
        local_ms, _ = graph_timed(r, exchange=False)
        if local_ms is None or graph_ms is None:
            local_ms = timed(r, K, exchange=False)
        split = {"launch": "graph" if graph_ms is not None else "eager", "step_ms": ms_per_step,
                 "compute_ms": local_ms, "exchange_ms": ms_per_step - local_ms,
                 "fwd_interval_ms": max_over_ranks(fwd_ms), "bwd_interval_ms": max_over_ranks(bwd_ms),
                 "note": "compute = the same fwd+bwd on this rank's shard with the local column "
                         "reduction only; exchange = what the step costs on top of it"}
        # exchanged [dgamma | dbeta] against one NCCL all-reduce of the local vectors
        r.step(0)
        r.drain()
        torch.cuda.synchronize()
        got = r.grad_buf.clone()
        r.step(0, exchange=False)
        torch.cuda.synchronize()
        ref = r.grad_buf.clone()
        dist.all_reduce(ref)
        torch.cuda.synchronize()
        denom = float(ref.abs().max().item()) or 1.0
        err = float((got - ref).abs().max().item()) / denom
        same = [torch.empty_like(got) for _ in range(world)]
        dist.all_gather(same, got)
        identical = all(torch.equal(same[0], t) for t in same)
        ok = torch.tensor([1 if (err <= 1e-5 and identical and lib.nvn_device_status() == 0) else 0],
                          device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        dp_check = {"status": "ok" if int(ok.item()) == 1 else "fail", "max_rel_err_vs_nccl": err,
                    "bit_identical_on_all_ranks": identical}

    # ---- e2e: pinned host buffers in; y, dx and the parameter gradients out, every step ----
    # Three streams and two buffer sets: the upload of step i + 1 and the download of step
    # i - 1 run beside the kernels of step i (PCIe is full duplex), as an input pipeline
    # would; every step still brings all its inputs in and takes all its results out inside
    # the timed region.
    e2e = None
    if not args.no_e2e:
        y_h = [torch.empty_like(x_h).pin_memory() for _ in range(2)]
        dx_h = [torch.empty_like(x_h).pin_memory() for _ in range(2)]
        out_h = [torch.empty(2 * F, dtype=torch.float32).pin_memory() for _ in range(2)]
        if r.nsets >= 2:
            xin, dyin = r.xs, r.dys
        else:   # one set only: a second pair of device input buffers for the pipeline
            xin = [r.xs[0], torch.empty_like(r.xs[0])]
            dyin = [r.dys[0], torch.empty_like(r.dys[0])]
        yout = [torch.empty_like(r.xs[0]) for _ in range(2)]
        dxout = [torch.empty_like(r.xs[0]) for _ in range(2)]
        up, down = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        cur = torch.cuda.current_stream(dev)
        ev_up = [torch.cuda.Event() for _ in range(2)]
        ev_comp = [torch.cuda.Event() for _ in range(2)]
        ev_down = [torch.cuda.Event() for _ in range(2)]

        def e2e_step(i):
            k = i % 2
            with torch.cuda.stream(up):
                up.wait_event(ev_comp[k])       # step i - 2 has read these inputs
                xin[k].copy_(x_h, non_blocking=True)
                dyin[k].copy_(dy_h, non_blocking=True)
                ev_up[k].record(up)
            cur.wait_event(ev_up[k])
            cur.wait_event(ev_down[k])          # the results of step i - 2 have left
            r.step(0, x=xin[k], dy=dyin[k], y_out=yout[k], dx_out=dxout[k])
            r.drain()
            out_h[k].copy_(r.grad_buf, non_blocking=True)
            ev_comp[k].record(cur)
            with torch.cuda.stream(down):
                down.wait_event(ev_comp[k])
                y_h[k].copy_(yout[k], non_blocking=True)
                dx_h[k].copy_(dxout[k], non_blocking=True)
                ev_down[k].record(down)

        def e2e_join():
            for k in range(2):
                cur.wait_event(ev_down[k])

        Ke = max(4, min(K, 20))
        for i in range(4):
            e2e_step(i)
        e2e_join()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s0.record()
        for i in range(Ke):
            e2e_step(i)
        e2e_join()
        s1.record()
        barrier()
        e2e_ms = max_over_ranks(s0.elapsed_time(s1)) / Ke
        esz = T.ELEM_SIZE[w.dtype]
        e2e = {"value": (world if mode == "weak" else 1) * w.algorithmic_bytes() / (e2e_ms * 1e-3) / 1e9,
               "unit": "GB/s",
               "h2d_bytes_per_step": 2 * wl.elements * esz,
               "d2h_bytes_per_step": 2 * wl.elements * esz + 2 * F * 4,
               "ms_per_step": e2e_ms, "steps": Ke,
               "copies": "per rank and step: x, dy host->device; y, dx, dgamma|dbeta device->host (pinned); "
                         "uploads, kernels and downloads on three streams over two buffer sets, so the "
                         "copies of neighbouring steps overlap"}
        del yout, dxout

    # ---- N > 1: the weak-scaling arrangement (every rank a full batch) as a sub-record ----
    if world > 1 and mode == "strong" and args.scaling == "auto":
        del r
        torch.cuda.empty_cache()
        xw, dyw = shard_inputs("weak")
        rw = make_runner(xw, dyw)
        for i in range(3):
            rw.step(i)
        rw.drain()
        wms, _ = graph_timed(rw)
        if wms is None:
            wms = timed(rw, K)
        weak = {"scaling": "weak", "per_gpu_batch": w.N, "global_batch": w.N * world,
                "ms_per_step": wms,
                "value": world * w.algorithmic_bytes() / (wms * 1e-3) / 1e9, "unit": "GB/s"}
        del rw
        torch.cuda.empty_cache()
        r = None

    # ---- every configuration in the same run (single GPU only) ----
    per_config = None
    worst = None
    if world == 1 and args.configs != "none" and not args.batch:
        names = CONFIGS if args.configs == "all" else tuple(c for c in args.configs.split(",") if c in CONFIGS)
        del r
        torch.cuda.empty_cache()
        per_config = {}
        for name in names:
            per_config[name] = measure_config(name, dev, peak, steps=20,
                                              host_calls=500 if name == "c1" else 0)
        if per_config:
            worst_name = min(per_config, key=lambda n: per_config[n]["frac_of_measured"])
            worst = {"config": worst_name, "frac_of_measured": per_config[worst_name]["frac_of_measured"]}
            if args.configs == "all":
                per_config["residual_fwd_c2"] = measure_residual(dev, peak)

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return

    global_bytes = (world if mode == "weak" else 1) * w.algorithmic_bytes()
    global_elems = (world if mode == "weak" else 1) * w.elements
    value = global_bytes / (ms_per_step * 1e-3) / 1e9
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
        "traffic": (NCU_BWD_TRAFFIC_BYTES_PER_ENTRY[w.name] * wl.N
                    if w.name in NCU_BWD_TRAFFIC_BYTES_PER_ENTRY else None),
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
        "steps": K, "warmup": W, "ms_per_step": ms_per_step,
        "higher_is_better": True, "scaling": mode, "vs_baseline": None,
        "dtype": w.dtype, "data": "synthetic",
        "config": workload_config(w, args, world),
        "gelem_per_s": global_elems / (ms_per_step * 1e-3) / 1e9,
        "pct_of_nominal_8000": 100.0 * (value / world) / NOMINAL_PEAK_GBS,
        "pct_of_measured_peak": 100.0 * (value / world) / peak,
        "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
        "gpu_launches": int(launches) * world, "clocks": clocks,
    }
    line["eager_ms_per_step"] = eager_ms_per_step
    if graph_ms is not None:
        line["timing"] = ("the %d timed steps replayed from a CUDA graph of %d steps (%d replays, then a graph "
                          "of the %d steps left over); eager launches through the Python layer: %.4f ms/step"
                          % (K, S, K // S, K % S, eager_ms_per_step))
    else:
        line["timing"] = "eager launches through the Python layer"
    if split is not None:
        line["split"] = split
        line["dp_check"] = dp_check["status"]
        line["dp_check_detail"] = dp_check
    if weak is not None:
        line["weak"] = weak
    if per_config is not None:
        line["per_config"] = per_config
        line["worst_frac"] = worst
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
