#!/usr/bin/env python
"""Benchmark of LuxLib's fused-layer hot path on B200.

Headline workload (the configuration the metric is quoted on): one fused dense layer, W 4096x4096, x 4096x8192
(features x batch), bias 4096, bf16 storage / fp32 accumulate, gelu; W ~ glorot_uniform, x ~ N(0,1),
b ~ U(-0.1,0.1), upstream gradient ~ N(0,1), seed 1. A step = forward + dX + dW + db = 6*M*N*K FLOP per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload ...] [--no-secondary]

For N > 1 launch under torchrun: every rank runs the layer on its own batch shard of the same size (weak scaling,
replicated weights) and the parameter gradients dW, db are all-reduced (avg) with NCCL, as Lux's DistributedOptimizer
does per leaf; dW travels in column panels so that a panel's all-reduce runs under the next panel's GEMM.

How a number is taken: the step is captured once into a CUDA graph (so that the host's launch path is outside the
measurement), replayed untimed for a fixed wall time (`ramp_s`; a GPU that was idle when the process started needs
it to reach its running clocks), then W warm-up replays, then exactly K timed replays between two CUDA events
bracketed by barrier + synchronize; max over ranks. Every step is also bracketed by its own events (median / min /
max are reported), SM clocks and throttle reasons are sampled every millisecond during the timed region. The launch
durations of the individual kernels come from an eager replay of the same K steps directly afterwards, with event
pairs around each launch.

The same JSON line carries the other configurations of the path as `secondary` records (conv C3, LayerNorm /
GroupNorm C4, BatchNorm C3, the small MLP C1, one ResNet-18 data-parallel training step), each with its own
roofline and clocks. Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
import re
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "lux.jl_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

M, K, N = 4096, 4096, 8192
ACT = "gelu"
METRIC = "fused dense+bias+act fwd+bwd TFLOP/s"
UNIT = "TFLOP/s"
WORKLOAD = "dense W 4096x4096 * x 4096x8192 + b, gelu(tanh), bf16 storage / fp32 accumulate; fwd + dX + dW + db"
RAMP_S = 1.5
DW_PANELS = 4
DX_RESERVE_SMS = 16       # SMs kept out of the dX GEMM of a multi-rank step: the last dW panel's all-reduce runs beside it
TRAFFIC_PROFILE = os.path.join("profiles", "gemm_tc_kernel_dense_c2_bf16.md")


def flops_per_step() -> float:
    return 6.0 * M * N * K


def make_inputs(seed: int, n_cols: int):
    """Seeded synthetic inputs with the reference initialisers' distributions."""
    rng = np.random.default_rng(seed)
    # glorot_uniform (lib/WeightInitializers/src/initializers.jl:28-36): (rand - 0.5) * sqrt(24 / (fan_in + fan_out))
    W = ((rng.random((M, K), dtype=np.float64) - 0.5) * np.sqrt(24.0 / (M + K))).astype(np.float32)
    x = rng.standard_normal((K, n_cols), dtype=np.float32)
    b = rng.uniform(-0.1, 0.1, M).astype(np.float32)
    dy = rng.standard_normal((M, n_cols), dtype=np.float32)
    return W, x, b, dy


def _peaks_file():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f)
    return None


def measured_peaks():
    d = _peaks_file()
    if d is not None:
        return d.get("bf16_tflops_sustained", 1430.0), d.get("bf16_tflops", 1699.0), "measured"
    return 1400.0, 1590.0, "fallback"


def hbm_peak():
    d = _peaks_file()
    if d is not None:
        return d.get("hbm_gbs", 6552.0), "measured"
    return 6650.0, "fallback"


def recorded_traffic():
    """DRAM bytes of one forward launch as recorded in the committed ncu summary (a line
    `roofline_traffic_bytes: <n>` in profiles/gemm_tc_kernel_dense_c2_bf16.md); None when the file has no such line."""
    path = os.path.join(ROOT, TRAFFIC_PROFILE)
    try:
        with open(path) as f:
            m = re.search(r"roofline_traffic_bytes:\s*([0-9.eE+]+)", f.read())
        return float(m.group(1)) if m else None
    except OSError:
        return None


# ---------------------------------------------------------------------------------------------
# CPU arms (oracle port of LuxLib's CPU path; test/bench infrastructure, never the product path)
# ---------------------------------------------------------------------------------------------
def cpu_step(W, x, b, dy):
    from oracle import luxlib_oracle as O
    y, pb = O.fused_dense_rrule(ACT, W, x, b)
    return y, pb(dy)


def use_all_host_threads() -> int:
    """torchrun exports OMP_NUM_THREADS=1; the CPU arms are meant to use every host core, so the BLAS pool is
    widened again at run time. Returns the thread count in effect."""
    cores = os.cpu_count() or 1
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=cores)
    except Exception:
        pass
    return cores


def cpu_tflops(n_cols: int, reps: int, seed: int = 1):
    from oracle import luxlib_oracle as O
    use_all_host_threads()
    W, x, b, dy = make_inputs(seed, n_cols)
    W, x, b, dy = (O.round_bf16(a) for a in (W, x, b, dy))
    cpu_step(W, x, b, dy)  # warm the BLAS threads
    t0 = time.perf_counter()
    for _ in range(reps):
        cpu_step(W, x, b, dy)
    dt = (time.perf_counter() - t0) / reps
    return 6.0 * M * n_cols * K / dt / 1e12, dt


def run_reference_arm(args):
    """`--impl reference`: the CPU implementation of the path on the host cores. Julia is not available, so this is
    the numpy restatement of LuxLib's CPU code (kind "port"), BLAS-threaded over all host cores. Each step is a
    bounded sample (a column block of the batch)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    cores = os.cpu_count() or 1
    _, t_probe = cpu_tflops(128, 1)
    budget = 120.0 / max(args.steps + args.warmup, 1)     # seconds per step
    n_cols = int(min(N, max(64, 128 * budget / max(t_probe, 1e-6))))
    n_cols = max(64, (n_cols // 64) * 64)
    from oracle import luxlib_oracle as O
    W, x, b, dy = (O.round_bf16(a) for a in make_inputs(1, n_cols))
    for _ in range(args.warmup):
        cpu_step(W, x, b, dy)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step(W, x, b, dy)
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    val = 6.0 * M * n_cols * K / dt / 1e12
    sample = f"{n_cols} of {N} batch columns per step (same W, K, M), numpy/BLAS on all host threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
# clock sampling during the timed region (read-only NVML)
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
        0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x100: "display_clock_setting",
    }

    def __init__(self, index: int, period_s: float = 0.001):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self.period = period_s
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# measurement helpers
# ---------------------------------------------------------------------------------------------
EAGER = False   # --eager: time plain launches (no graph capture, no ramp); used when profiling the launch list


GRAPHS = []      # every captured graph, so that shutdown() can release them before the process group goes


def nccl_defaults():
    """NCCL settings of the multi-rank runs, applied before the communicator exists and only where the launcher's
    environment does not say otherwise. NVLS (in-switch reduction) is switched off: with it, replays of a captured step
    that holds all-reduces were separated by about 1.3 ms of idle time on 4 GPUs (2.26 ms per step against 0.92 ms of
    device time per replay), and its all-reduce of these 8 MB panels is no faster than the ring (0.25 against 0.24 ms
    for the four panels); without it the panels hide completely under the next panel's GEMM."""
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")


def shutdown(dist, torch):
    """Ends a multi-rank run. Captured graphs that hold collectives are released first and the communicator is
    destroyed after a barrier; because a rank must not outlive its result by minutes whatever a library does on
    the way out, the destruction runs beside a 20 s watch that ends the process (the JSON line is out by then)."""
    import gc
    import threading
    torch.cuda.synchronize()
    for g in GRAPHS:
        try:
            g.reset()                # frees the captured graph even while a caller's variable still names the object
        except Exception:            # noqa: BLE001
            pass
    GRAPHS.clear()
    gc.collect()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    if dist is None:
        return

    def watch():
        time.sleep(20.0)
        sys.stderr.write("[bench] process-group shutdown did not return within 20 s; leaving\n")
        sys.stderr.flush()
        os._exit(0)
    threading.Thread(target=watch, daemon=True).start()
    dist.barrier()
    torch.cuda.synchronize()
    dist.destroy_process_group()


def capture(step, torch, device):
    """The step as a CUDA graph replay (None when capture is not possible: the caller then times eager launches)."""
    if EAGER:
        return None, None
    try:
        torch.cuda.synchronize(device)
        g = torch.cuda.CUDAGraph()
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side):
            step()                                   # allocator and library caches warm on the capture stream
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        # thread_local: the NCCL watchdog and the clock sampler are other threads of this process
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            out = step()
        torch.cuda.synchronize(device)
        GRAPHS.append(g)
        return g, out
    except Exception as e:                           # noqa: BLE001 - any capture failure falls back to eager timing
        sys.stderr.write(f"[bench] CUDA graph capture failed ({type(e).__name__}: {e}); timing eager launches\n")
        try:
            torch.cuda.synchronize(device)
        except Exception:
            pass
        return None, None


def ramp(run, torch, seconds: float, barrier=None, dist=None):
    """Untimed repetitions of the step for a fixed wall time (clocks, caches, NCCL first-use set-up). With several
    ranks the decision to stop is shared (an all-reduce of the "time is up" flag after every batch of 8), so that
    every rank runs the same number of steps: a step holds collectives, and ranks that disagreed on the count would
    wait for each other for ever."""
    t0 = time.perf_counter()
    n = 0
    if EAGER:
        return 0.0, 0
    while True:
        for _ in range(8):
            run()
        n += 8
        torch.cuda.synchronize()
        done = time.perf_counter() - t0 >= seconds
        if dist is not None:
            flag = torch.tensor([1.0 if done else 0.0], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            done = bool(flag.item() > 0)
        if done or n >= 100000:
            break
    if barrier is not None:
        barrier()
    return time.perf_counter() - t0, n


def timed(run, torch, steps: int, barrier, device_index: int):
    """Exactly `steps` runs between two events, each run also bracketed by its own event; clocks sampled meanwhile.
    Returns (total ms, per-step ms list, clocks)."""
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    barrier()
    sampler = ClockSampler(device_index).start()
    ev[0].record()
    for i in range(steps):
        run()
        ev[i + 1].record()
    barrier()
    clocks = sampler.stop()
    per = [ev[i].elapsed_time(ev[i + 1]) for i in range(steps)]
    return ev[0].elapsed_time(ev[steps]), per, clocks


def stats(per):
    a = np.asarray(per, dtype=np.float64)
    return {"median": float(np.median(a)), "min": float(a.min()), "max": float(a.max())}


# ---------------------------------------------------------------------------------------------
# GPU arm: the dense layer
# ---------------------------------------------------------------------------------------------
def run_gpu_arm(args):
    import torch
    import luxlib_b200 as L
    from luxlib_b200 import _cabi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback on the product path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        from luxlib_b200 import distributed as D
        nccl_defaults()
        D.initialize(D.NCCLBackend)            # DistributedUtils.initialize: process group from the launcher's environment
        import torch.distributed as dist_mod
        dist = dist_mod
    lib = _cabi.load()

    # every rank holds the same parameters and its own batch shard
    Wn, xn, bn, dyn = make_inputs(1, N)
    if rank > 0:
        r2 = np.random.default_rng(1000 + rank)
        xn = r2.standard_normal((K, N), dtype=np.float32)
        dyn = r2.standard_normal((M, N), dtype=np.float32)
    bf = torch.bfloat16
    W = L.from_numpy(Wn, device, bf)
    b = L.from_numpy(bn, device, bf)
    x = L.from_numpy(xn, device, bf)
    dy = L.from_numpy(dyn, device, bf)
    del Wn, bn

    def reduce_panel(dW_panel, db):
        # DistributedOptimizer's all-reduce(avg) of the parameter-gradient leaves, issued per column panel of dW as soon
        # as the panel exists, so that it runs underneath the next panel's GEMM. A column panel of the column-major dW
        # is contiguous: .T is the contiguous view of the same memory.
        works = [dist.all_reduce(dW_panel.T, op=dist.ReduceOp.AVG, async_op=True)]
        if db is not None:
            works.append(dist.all_reduce(db, op=dist.ReduceOp.AVG, async_op=True))
        return works

    def step_from(x_, dy_, collectives=True):
        y, pullback = L.rrule_fused_dense(ACT, W, x_, b)
        if dist is None or not collectives:
            dW, dx, db = pullback(dy_)
            return y, dW, dx, db
        pending = []
        dW, dx, db = pullback(dy_, on_param_grads=lambda p, d: pending.extend(reduce_panel(p, d)), param_panels=DW_PANELS,
                              dx_reserve_sms=DX_RESERVE_SMS)
        for h in pending:
            h.wait()          # stream-level wait: later work is ordered after the reduced gradients
        return y, dW, dx, db

    def step():
        return step_from(x, dy)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(3):
        step()
    barrier()
    rc = lib.lb2_poll_device_status(None)
    if rc != 0:
        raise SystemExit(f"device status after the first steps: {rc} {lib.lb2_last_error_string()}")

    graph, _ = capture(step, torch, device)
    run = graph.replay if graph is not None else step
    mode = "cuda_graph_replay" if graph is not None else "eager"
    ramp_s, ramp_steps = ramp(run, torch, RAMP_S, barrier, dist)
    warm = max(args.warmup, 3)
    for _ in range(warm):
        run()
    ms_total, per, clocks = timed(run, torch, args.steps, barrier, local)
    t = torch.tensor([ms_total], device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * flops_per_step() / (ms_step * 1e-3) / 1e12
    rc = lib.lb2_poll_device_status(None)
    if rc != 0:
        raise SystemExit(f"device status after the timed region: {rc} {lib.lb2_last_error_string()}")

    # ---- per-launch durations: eager replay of the same K steps, an event pair around every launch
    names = ["forward GEMM (bias+gelu epilogue, pre-activation store)", "g = dy*gelu'(pre) and db partials + db finish",
             "dW GEMM", "dX GEMM"]
    kern = {n_: [] for n_ in names}
    sampler2 = ClockSampler(local).start()
    for _ in range(args.steps):
        e = [torch.cuda.Event(enable_timing=True) for _ in range(5)]
        e[0].record()
        y, pullback = L.rrule_fused_dense(ACT, W, x, b)
        e[1].record()
        marks = []
        pullback(dy, on_param_grads=lambda p, d: None, param_panels=1,
                 mark=lambda: (marks.append(torch.cuda.Event(enable_timing=True)), marks[-1].record()))
        torch.cuda.synchronize()
        kern[names[0]].append(e[0].elapsed_time(e[1]))
        pts = [e[1]] + marks      # marks: after g/db, after dW, after dX
        for nm, a_, b_ in zip(names[1:], pts[:-1], pts[1:]):
            kern[nm].append(a_.elapsed_time(b_))
    clocks2 = sampler2.stop()
    fwd_ms = float(np.median(kern[names[0]]))
    launches = {n_: stats(v) for n_, v in kern.items()}

    # ---- collectives alone and the step without them (N > 1): how much of the all-reduce time is hidden
    comm = None
    if dist is not None:
        dWbuf = L.jl_empty((M, K), bf, device)
        dbbuf = torch.zeros(M, device=device, dtype=bf)
        cols = K // DW_PANELS

        def comm_only():
            hs = []
            for p_ in range(DW_PANELS):
                hs += reduce_panel(dWbuf[:, p_ * cols:(p_ + 1) * cols], dbbuf if p_ == DW_PANELS - 1 else None)
            for h in hs:
                h.wait()
        for _ in range(5):
            comm_only()
        comm_total, _, _ = timed(comm_only, torch, args.steps, barrier, local)
        # the same step without its all-reduces, timed the way the step itself is: a graph replay after an untimed ramp
        nocomm_step = lambda: step_from(x, dy, collectives=False)
        for _ in range(3):
            nocomm_step()
        torch.cuda.synchronize()
        g_nc, _ = capture(nocomm_step, torch, device)
        run_nc = g_nc.replay if g_nc is not None else nocomm_step
        ramp(run_nc, torch, 0.3, barrier, dist)
        nocomm_total, _, _ = timed(run_nc, torch, args.steps, barrier, local)
        tt = torch.tensor([comm_total / args.steps, nocomm_total / args.steps], device=device)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        comm_ms, nocomm_ms = float(tt[0]), float(tt[1])
        exposed = max(0.0, ms_step - nocomm_ms)
        comm = {"comm_ms": comm_ms, "step_without_collectives_ms": nocomm_ms, "exposed_ms": exposed,
                "overlap_frac": max(0.0, min(1.0, 1.0 - exposed / comm_ms)) if comm_ms > 0 else None,
                "payload_bytes": (M * K + M) * 2, "panels": DW_PANELS,
                "nvls": os.environ.get("NCCL_NVLS_ENABLE", "default")}

    # ---- end to end through the public API with HOST buffers (pinned): per step copy this step's inputs (x, dy) to
    # the device, run, and read every result (y, dW, dx, db) back.
    e2e_steps = max(3, min(args.steps, 20))
    hx = torch.from_numpy(np.ascontiguousarray(xn.T)).to(bf).pin_memory()      # column-major bytes of x
    hdy = torch.from_numpy(np.ascontiguousarray(dyn.T)).to(bf).pin_memory()
    # Three streams: uploads, compute, downloads. Device inputs and host outputs are double-buffered so that the
    # upload of step i+1 and the download of step i-1 run under the compute of step i (PCIe is full duplex).
    s_in, s_out = torch.cuda.Stream(device=device), torch.cuda.Stream(device=device)
    in_bufs = [(torch.empty_like(hx, device=device), torch.empty_like(hdy, device=device)) for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    houts = [(torch.empty((N, M), dtype=bf).pin_memory(), torch.empty((K, M), dtype=bf).pin_memory(),
              torch.empty((N, K), dtype=bf).pin_memory(), torch.empty((M,), dtype=bf).pin_memory()) for _ in range(2)]
    hy, hdW, hdx, hdb = houts[0]
    cur = torch.cuda.current_stream(device)
    e2e_count = [0]

    def e2e_step():
        k = e2e_count[0] % 2
        e2e_count[0] += 1
        dxbuf, dybuf = in_bufs[k]
        with torch.cuda.stream(s_in):
            s_in.wait_event(in_free[k])            # the step that last read this buffer pair has finished
            dxbuf.copy_(hx, non_blocking=True)
            dybuf.copy_(hdy, non_blocking=True)
            in_ready[k].record(s_in)
        cur.wait_event(in_ready[k])
        y, dW, dx, db = step_from(dxbuf.T, dybuf.T)
        in_free[k].record(cur)
        done = torch.cuda.Event()
        done.record(cur)
        oy, odW, odx, odb = houts[k]
        with torch.cuda.stream(s_out):
            s_out.wait_event(done)
            oy.copy_(y.T, non_blocking=True)
            odW.copy_(dW.T, non_blocking=True)
            odx.copy_(dx.T, non_blocking=True)
            odb.copy_(db, non_blocking=True)
        for t_ in (y, dW, dx, db):
            t_.record_stream(s_out)                # keep the results alive until their download has run

    for _ in range(3):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    t = torch.tensor([e2e_s], device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_s = float(t.item())
    e2e_val = world * flops_per_step() / e2e_s / 1e12
    h2d = hx.numel() * 2 + hdy.numel() * 2
    d2h = (hy.numel() + hdW.numel() + hdx.numel() + hdb.numel()) * 2
    del in_bufs, houts, hx, hdy

    # ---- the other configurations of the path, in the same line
    secondary = None
    if not args.no_secondary:
        del graph
        torch.cuda.empty_cache()
        secondary = {}
        if world == 1:
            for wl, dts in (("conv", ("bf16", "f32")), ("ln", ("bf16", "f32")), ("gn", ("bf16", "f32")), ("bn", ("bf16", "f32")),
                            ("mlp", ("f32",)), ("pool", ("bf16",))):
                for dt_ in dts:
                    try:
                        secondary[f"{wl}_{dt_}"] = measure_secondary(wl, dt_, steps=max(args.steps, 30), warm=warm, quiet=True)
                    except Exception as e:   # noqa: BLE001 - a failing secondary row must not lose the headline
                        secondary[f"{wl}_{dt_}"] = {"error": f"{type(e).__name__}: {e}"}
                    torch.cuda.empty_cache()
        try:
            secondary["convnet"] = measure_convnet(max(5, min(args.steps, 20)), warm, dist, world, rank, local)
        except Exception as e:               # noqa: BLE001
            secondary["convnet"] = {"error": f"{type(e).__name__}: {e}"}

    if rank == 0:
        sustained, burst, which = measured_peaks()
        achieved = 2.0 * M * N * K / (fwd_ms * 1e-3) / 1e12
        traffic = recorded_traffic()
        roofline = {
            "bound": "tensor", "kernel": "forward GEMM (bias+gelu epilogue, pre-activation store)", "achieved": achieved,
            "peak": sustained, "unit": "TFLOP/s", "frac": achieved / sustained,
            "traffic": traffic, "traffic_unit": "bytes per launch",
            "traffic_source": f"recorded constant: dram__bytes_read.sum + dram__bytes_write.sum of one forward launch in {TRAFFIC_PROFILE}",
            "peak_source": f"{which}: bf16_tflops_sustained (kernel timed inside a long step); burst figure {burst}",
            "launch_ms": fwd_ms,
            "launch_timing": "event pair around each launch, eager replay of the same steps directly after the timed region",
            "launches": launches, "clocks_during_launch_timing": clocks2,
        }
        cpu = None
        if world == 1:
            cores = os.cpu_count() or 1
            n_cols = 512
            val, dt_cpu = cpu_tflops(n_cols, 1)
            reps = int(max(1, min(100, 12.0 / max(dt_cpu, 1e-3))))
            val, dt_cpu = cpu_tflops(n_cols, reps)
            cpu = {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                   "sample": f"{n_cols} of {N} batch columns x {reps} repetitions, numpy/BLAS restatement of LuxLib's CPU path"}
        st = stats(per)
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "M": M, "N_per_gpu": N, "K": K, "gelu": L.ops.GELU_VARIANT,
                       "l2": "inputs larger than L2 (704 MB touched per step vs 126 MB L2)",
                       "parallelism": (f"dp{world}: replicated W, per-GPU batch {N}, NCCL allreduce(avg) of dW in {DW_PANELS} column "
                                       "panels (each under the next panel's GEMM) and of db") if world > 1 else "single GPU"},
            "timing": {"mode": mode, "ramp_s": ramp_s, "ramp_steps": ramp_steps, "step_ms": st,
                       "ms_x_sm_mhz": ms_step * clocks["sm_mhz"] if clocks.get("sm_mhz") else None},
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                    "pipeline": "uploads, compute and downloads on three streams, double-buffered; wall clock over all steps"},
            "gpu_launches": (5 if world == 1 else 4 + DW_PANELS) * args.steps,   # fwd GEMM, g/db pass, db finish, dX GEMM, dW GEMM(s)
            "roofline": roofline,
            "cpu_baseline": cpu,
            "pct_of_measured_peak": {"sustained": value / world / sustained, "burst": value / world / burst},
        }
        if comm is not None:
            line["collectives"] = comm
        if secondary is not None:
            line["secondary"] = secondary
        print(json.dumps(line), flush=True)
    shutdown(dist, torch)
    return 0


# ---------------------------------------------------------------------------------------------
# secondary workloads (the other configurations of the path), single GPU
# ---------------------------------------------------------------------------------------------
def measure_secondary(wl: str, dtype: str, steps: int, warm: int, quiet: bool = False):
    """ln | gn | bn: algorithmic GB/s (5*numel*sizeof(T) per fwd+bwd step) against the measured HBM copy bandwidth;
    conv: TFLOP/s (3 x 2*Wo*Ho*N*Cout*Cin*kW*kH per step) against the measured bf16 tensor peak; mlp: microseconds
    per forward + backward of the small MLP (latency-bound: time, not a fraction)."""
    import torch
    import luxlib_b200 as L
    dev_index = torch.cuda.current_device()
    tdt = torch.float32 if dtype == "f32" else torch.bfloat16
    es = 4 if dtype == "f32" else 2
    g = torch.Generator(device="cuda").manual_seed(3)
    rn = lambda *shape: torch.randn(*shape, device="cuda", generator=g)
    cm = lambda t: t.permute(*reversed(range(t.dim()))) if t.dim() > 1 else t  # row-major bytes -> Julia shape
    if wl == "ln":
        D, R = 4096, 16384
        x = cm((rn(R, D) * 1.3).to(tdt)); dy = cm(rn(R, D).to(tdt))
        gam = (torch.rand(D, device="cuda", generator=g) + 0.5).to(tdt); bet = (rn(D) * 0.1).to(tdt)
        def step():
            y, pb = L.rrule_layernorm(x, gam, bet, "identity", None, 1e-5)
            return pb(dy)
        numel, name = D * R, "LayerNorm 4096x16384 (rows of 4096), affine, fwd+bwd"
    elif wl == "gn":
        shape = (128, 512, 32, 32)  # N, C, H, W row-major == WHCN column-major
        x = cm((rn(*shape) * (torch.rand(1, 512, 1, 1, device="cuda", generator=g) * 1.5 + 0.5)).to(tdt)); dy = cm(rn(*shape).to(tdt))
        gam = (torch.rand(512, device="cuda", generator=g) + 0.5).to(tdt); bet = (rn(512) * 0.1).to(tdt)
        def step():
            y, pb = L.rrule_groupnorm(x, gam, bet, 32, "identity", 1e-5)
            return pb(dy)
        numel, name = 128 * 512 * 32 * 32, "GroupNorm(32 groups) 32x32x512x128, affine, fwd+bwd"
    elif wl == "bn":
        shape = (256, 64, 56, 56)
        x = cm(rn(*shape).to(tdt)); dy = cm(rn(*shape).to(tdt))
        gam = torch.ones(64, device="cuda", dtype=tdt); bet = torch.zeros(64, device="cuda", dtype=tdt)
        rm = torch.zeros(64, device="cuda", dtype=tdt); rv = torch.ones(64, device="cuda", dtype=tdt)
        def step():
            y, st, pb = L.rrule_batchnorm(x, gam, bet, rm, rv, True, "relu", 0.1, 1e-5)
            return pb(dy)
        numel, name = 256 * 64 * 56 * 56, "BatchNorm(64)+relu 56x56x64x256 training, running stats, fwd+bwd"
    elif wl == "conv":
        x = cm(rn(256, 64, 56, 56).to(tdt)); dy = cm(rn(256, 64, 56, 56).to(tdt))
        w = cm((rn(64, 64, 3, 3) * (2.0 / 576) ** 0.5).to(tdt)); b = torch.zeros(64, device="cuda", dtype=tdt)
        cd = L.ConvDims.make(2, 1, 1, 1, 1, False)
        def step():
            y, pb = L.rrule_fused_conv("identity", w, x, b, cd)
            return pb(dy)
        numel, name = 256 * 64 * 56 * 56, "Conv 3x3 64->64 s1 p1 on 56x56x64x256, fwd + dx + dw + db"
    elif wl == "mlp":
        # Dense(784 -> 256, relu) -> Dense(256 -> 10), batch 128, Float32: forward + pullback of the mean-squared error
        W1 = cm(((torch.rand(784, 256, device="cuda", generator=g) - 0.5) * (24.0 / (784 + 256)) ** 0.5))
        W2 = cm(((torch.rand(256, 10, device="cuda", generator=g) - 0.5) * (24.0 / (256 + 10)) ** 0.5))
        b1, b2 = torch.zeros(256, device="cuda"), torch.zeros(10, device="cuda")
        x = cm(rn(128, 784)); tgt = cm(torch.nn.functional.one_hot(torch.randint(0, 10, (128,), device="cuda", generator=g), 10).float())
        def step():
            h, pb1 = L.rrule_fused_dense("relu", W1, x, b1)
            y, pb2 = L.rrule_fused_dense("identity", W2, h, b2)
            loss, pl = L.rrule_mse_loss(y, tgt)
            dW2, dh, db2 = pb2(pl())
            return pb1(dh)
        numel, name = 0, "MLP Dense(784->256, relu) -> Dense(256->10), batch 128, Float32: forward + pullback of MSE"
    elif wl == "pool":
        # the stem's pooling of ResNet-18 at batch 256: MaxPool 3x3, stride 2, SamePad on 112x112x64x256, fwd + pullback
        x = cm(rn(256, 64, 112, 112).to(tdt))
        pd = L.PoolDims.make((3, 3), 2, 1)
        y0, _ = L.rrule_maxpool(x, pd)
        dy = torch.empty_like(y0).normal_(generator=g)       # same (column-major) strides as y: no layout copy in the step
        def step():
            y, pb = L.rrule_maxpool(x, pd)
            return pb(dy)
        numel, name = 256 * 64 * 112 * 112, "MaxPool 3x3 / 2 (pad 1) on 112x112x64x256, forward + pullback"
    else:
        raise SystemExit(f"unknown workload {wl}")
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    graph, _ = capture(step, torch, torch.device("cuda", dev_index))
    run = graph.replay if graph is not None else step
    ramp(run, torch, 0.4)
    for _ in range(warm):
        run()
    total, per, clocks = timed(run, torch, steps, torch.cuda.synchronize, dev_index)
    ms = total / steps
    rc = L._cabi.load().lb2_poll_device_status(None)
    if rc != 0:
        raise SystemExit(f"device status {rc}")
    common = {"ms_per_step": ms, "step_ms": stats(per), "steps": steps, "dtype": dtype, "workload": name, "clocks": clocks,
              "mode": "cuda_graph_replay" if graph is not None else "eager"}
    if wl == "conv":
        flop = 3 * 2.0 * 56 * 56 * 256 * 64 * 64 * 9
        sustained, burst, which = measured_peaks()
        val = flop / (ms * 1e-3) / 1e12
        rec = {"metric": "fused conv+bias+act fwd+bwd TFLOP/s", "value": val, "unit": "TFLOP/s",
               "roofline": {"bound": "tensor", "achieved": val, "peak": sustained, "unit": "TFLOP/s", "frac": val / sustained,
                            "traffic": None, "peak_source": f"{which}: bf16_tflops_sustained; whole step (layout passes, 3 GEMM-like kernels, reductions)"}}
    elif wl == "mlp":
        rec = {"metric": "MLP forward+backward time", "value": ms * 1e3, "unit": "us", "higher_is_better": False,
               "flop": 6.0 * 128 * (784 * 256 + 256 * 10)}
    elif wl == "pool":
        byts = 3.5 * numel * es      # forward: read x, write y (a quarter of x); pullback: read x and dy, write dx
        peak, which = hbm_peak()
        val = byts / (ms * 1e-3) / 1e9
        rec = {"metric": "pooling fwd+bwd HBM GB/s", "value": val, "unit": "GB/s",
               "roofline": {"bound": "hbm", "achieved": val, "peak": peak, "unit": "GB/s", "frac": val / peak, "traffic": None,
                            "peak_source": f"{which}: hbm_gbs; algorithmic bytes 3.5*numel*sizeof(T) over the whole fwd+bwd step"}}
    else:
        byts = 5.0 * numel * es
        peak, which = hbm_peak()
        val = byts / (ms * 1e-3) / 1e9
        rec = {"metric": "norm fwd+bwd HBM GB/s", "value": val, "unit": "GB/s",
               "roofline": {"bound": "hbm", "achieved": val, "peak": peak, "unit": "GB/s", "frac": val / peak, "traffic": None,
                            "peak_source": f"{which}: hbm_gbs; algorithmic bytes 5*numel*sizeof(T) over the whole fwd+bwd step"}}
    rec.update(common)
    return rec


def run_secondary(args):
    import torch
    torch.cuda.set_device(0)
    rec = measure_secondary(args.workload, args.dtype, args.steps, max(args.warmup, 3))
    rec.update({"n_gpus": 1, "warmup": max(args.warmup, 3), "higher_is_better": rec.get("higher_is_better", True), "scaling": "weak",
                "vs_baseline": None, "data": "synthetic", "config": {"workload": rec["workload"]}})
    print(json.dumps(rec), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
# ResNet-18 data-parallel training step (perf/resnet/resnet.jl:9-107)
# ---------------------------------------------------------------------------------------------
def build_resnet18(L, torch, device, rank, batch, dtype):
    """Parameters (identical on every rank) and the training step of ResNet(18) as perf/resnet/resnet.jl builds it:
    7x7/2 stem conv + BatchNorm(relu) + 3x3/2 max pool (SamePad), four stages of two basic blocks (conv3x3-BN(relu)-
    conv3x3-BN(relu, scale initialised to zero), projection conv1x1/2-BN on the first block of stages 2-4, joined
    by relu.(main .+ skip)), global mean pool, Dense 512 -> 1000. Convolutions carry no bias. Loss: mean-squared error
    against one-hot labels."""
    gp = torch.Generator(device="cuda").manual_seed(5)               # parameters: same on every rank
    gd = torch.Generator(device="cuda").manual_seed(100 + rank)      # data: one shard per rank
    cm = lambda t: t.permute(*reversed(range(t.dim()))) if t.dim() > 1 else t   # row-major bytes -> Julia shape
    params, names = [], []

    def conv_w(k, cin, cout):
        w = cm((torch.randn(cout, cin, k, k, device=device, generator=gp) * (2.0 / (k * k * cin)) ** 0.5).to(dtype))   # kaiming_normal
        params.append(w); names.append(f"conv{k}x{k}_{cin}_{cout}")
        return len(params) - 1

    def bn_p(c, zero_scale=False):
        g_ = torch.zeros(c, device=device, dtype=dtype) if zero_scale else torch.ones(c, device=device, dtype=dtype)
        params.append(g_); params.append(torch.zeros(c, device=device, dtype=dtype)); names.extend([f"bn_scale_{c}", f"bn_bias_{c}"])
        return len(params) - 2

    stem = (conv_w(7, 3, 64), bn_p(64))
    blocks = []
    cin = 64
    for stage, cout in enumerate((64, 128, 256, 512)):
        for j in range(2):
            stride = 2 if (stage > 0 and j == 0) else 1
            blk = {"stride": stride, "c1": conv_w(3, cin, cout), "n1": bn_p(cout), "c2": conv_w(3, cout, cout), "n2": bn_p(cout, True)}
            if stride != 1 or cin != cout:
                blk["cp"], blk["np"] = conv_w(1, cin, cout), bn_p(cout)
            blocks.append(blk)
            cin = cout
    lim = (24.0 / (512 + 1000)) ** 0.5
    params.append(cm(((torch.rand(512, 1000, device=device, generator=gp) - 0.5) * lim).to(dtype)))   # (1000, 512) glorot_uniform
    params.append(torch.zeros(1000, device=device, dtype=dtype))
    iWd, ibd = len(params) - 2, len(params) - 1
    n_bn = sum(1 for n_ in names if n_.startswith("bn_scale"))
    rstats = {}

    def conv_bn(ic, ib, h, cdims, act):
        """conv_norm of perf/resnet/resnet.jl:17-22: Conv without bias, then BatchNorm carrying the activation; the
        statistics come from the convolution's epilogue where the general tensor-core path runs it. Pullback
        Δ -> (∂weight, ∂x, ∂scale, ∂bias)."""
        c = params[ib].shape[0]
        if ib not in rstats:    # running mean / variance start at 0 / 1 (created once, not per step)
            rstats[ib] = (torch.zeros(c, device=device, dtype=dtype), torch.ones(c, device=device, dtype=dtype))
        rm, rv = rstats[ib]
        y, new, pb = L.rrule_conv_batchnorm(act, params[ic], h, cdims, params[ib], params[ib + 1], rm, rv, 0.1, 1e-5)
        rstats[ib] = new
        return y, pb

    x = cm(torch.randn(batch, 3, 224, 224, device=device, generator=gd).to(dtype))
    labels = torch.randint(0, 1000, (batch,), device=device, generator=gd)
    target = cm(torch.nn.functional.one_hot(labels, 1000).to(dtype))                            # (1000, B)
    cd = lambda s, p: L.ConvDims.make(2, s, p, 1, 1, False)

    def forward_backward():
        grads = [None] * len(params)
        h, pstem = conv_bn(stem[0], stem[1], x, cd(2, 3), "relu")
        h, pp = L.rrule_maxpool(h, L.PoolDims.make((3, 3), (2, 2), (1, 1, 1, 1)))
        tape = []
        for blk in blocks:
            skip = h
            a, p1 = conv_bn(blk["c1"], blk["n1"], h, cd(blk["stride"], 1), "relu")
            a, p2 = conv_bn(blk["c2"], blk["n2"], a, cd(1, 1), "relu")
            pproj = None
            if "cp" in blk:
                skip, pproj = conv_bn(blk["cp"], blk["np"], h, cd(blk["stride"], 0), "identity")
            h, padd = L.rrule_add_activation("relu", a, skip)
            tape.append((blk, p1, p2, pproj, padd))
        pooled, ppool = L.rrule_meanpool(h, L.PoolDims.global_(h))          # (1, 1, 512, B)
        feat = pooled.reshape(512, batch)                                    # same bytes, Julia shape (512, B)
        y, pdense = L.rrule_fused_dense("identity", params[iWd], feat, params[ibd])
        loss, ploss = L.rrule_mse_loss(y, target)
        grads[iWd], dfeat, grads[ibd] = pdense(ploss())
        dh = ppool(dfeat.reshape(1, 1, 512, batch))
        for blk, p1, p2, pproj, padd in reversed(tape):
            da, dskip = padd(dh)
            grads[blk["c2"]], da, grads[blk["n2"]], grads[blk["n2"] + 1] = p2(da)
            grads[blk["c1"]], dmain, grads[blk["n1"]], grads[blk["n1"] + 1] = p1(da)
            if pproj is not None:
                grads[blk["cp"]], dskip, grads[blk["np"]], grads[blk["np"] + 1] = pproj(dskip)
            dh = L.add_activation("identity", dmain, dskip)
        dh = pp(dh)
        grads[stem[0]], _, grads[stem[1]], grads[stem[1] + 1] = pstem(dh, need_dx=False)
        return loss, grads

    return params, forward_backward, n_bn


def measure_convnet(steps, warm, dist, world, rank, local, batch=256):
    import torch
    import luxlib_b200 as L
    from luxlib_b200 import distributed as D
    device = torch.device("cuda", local)
    bf = torch.bfloat16
    params, forward_backward, n_bn = build_resnet18(L, torch, device, rank, batch, bf)
    opt = D.FusedOptimizer(D.NCCLBackend, "momentum", eta=1e-3, rho=0.9)
    states = opt.init(params)
    n_params = sum(p.numel() for p in params)

    def step():
        loss, grads = forward_backward()
        opt.update(states, params, grads)       # one flat sum all-reduce per bucket + one optimiser launch (1/world folded in)
        return loss

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(2):
        loss = step()
    barrier()
    rc = L._cabi.load().lb2_poll_device_status(None)
    if rc != 0:
        raise SystemExit(f"device status {rc}: {L._cabi.load().lb2_last_error_string()}")
    graph, gloss = capture(step, torch, device)
    run = graph.replay if graph is not None else step
    ramp(run, torch, 0.5, barrier, dist)
    for _ in range(warm):
        run()
    total, per, clocks = timed(run, torch, steps, barrier, local)
    t = torch.tensor([total], device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    rc = L._cabi.load().lb2_poll_device_status(None)
    if rc != 0:
        raise SystemExit(f"device status {rc}")
    flop = 10.88e9 * batch                           # 3 x (3.627 GFLOP conv + 0.001 GFLOP dense) per image
    sustained, burst, which = measured_peaks()
    tf = world * flop / (ms * 1e-3) / 1e12
    final_loss = float(gloss if graph is not None else loss)
    return {"metric": "data-parallel conv-net step samples/s", "value": world * batch / (ms * 1e-3), "unit": "samples/s",
            "n_gpus": world, "steps": steps, "ms_per_step": ms, "step_ms": stats(per), "dtype": "bf16",
            "workload": ("ResNet-18 (7x7/2 stem, 3x3/2 max pool, stages [2,2,2,2] of basic blocks at 64/128/256/512 with 1x1/2 projections, "
                         f"global mean pool, Dense 512->1000), 224x224x3 input, per-GPU batch {batch}, MSE loss, momentum SGD fused with the "
                         "gradient all-reduce bucket"),
            "parameters": n_params, "allreduce_bytes": n_params * 2, "parallelism": f"dp{world}", "final_loss": final_loss,
            "mode": "cuda_graph_replay" if graph is not None else "eager", "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": world * sustained, "unit": "TFLOP/s", "frac": tf / (world * sustained),
                         "traffic": None, "peak_source": f"{which}: bf16_tflops_sustained x n_gpus; 10.88 GFLOP per image (conv + dense, fwd + both gradients)"}}


def run_convnet(args):
    import torch
    from luxlib_b200 import distributed as D
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        nccl_defaults()
        D.initialize(D.NCCLBackend)
        import torch.distributed as dist
    rec = measure_convnet(args.steps, max(args.warmup, 3), dist, world, rank, local, batch=args.batch)
    if rank == 0:
        rec.update({"warmup": max(args.warmup, 3), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "data": "synthetic",
                    "config": {"workload": rec["workload"], "parallelism": rec["parallelism"]}, "gpu_launches": None})
        print(json.dumps(rec), flush=True)
    shutdown(dist, torch)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense", choices=["dense", "ln", "gn", "bn", "conv", "mlp", "pool", "convnet"],
                    help="dense = the headline configuration (default; its line also carries the others as `secondary`); "
                         "ln/gn/bn/conv/mlp/pool print one single-GPU row; convnet = the ResNet-18 data-parallel step (any --gpus, "
                         "under torchrun for N > 1)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"], help="storage type of the secondary workloads")
    ap.add_argument("--batch", type=int, default=256, help="per-GPU batch of the convnet workload")
    ap.add_argument("--no-secondary", action="store_true", help="dense workload only: leave the `secondary` records out")
    ap.add_argument("--eager", action="store_true", help="plain launches, no CUDA graph and no ramp (for kernel-list profiling)")
    args = ap.parse_args()
    global EAGER
    EAGER = args.eager
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "convnet":
        return run_convnet(args)
    if args.workload != "dense":
        return run_secondary(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
