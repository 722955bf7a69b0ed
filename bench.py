#!/usr/bin/env python
"""Benchmark of the fused dense layer hot path (forward + pullback) on B200.

Workload (the configuration the headline metric is quoted on): one fused dense layer,
W 4096x4096, x 4096x8192 (features x batch), bias 4096, bf16 storage / fp32 accumulate, gelu;
W ~ glorot_uniform, x ~ N(0,1), b ~ U(-0.1,0.1), upstream gradient ~ N(0,1), seed 1.
A step = forward + dX + dW + db. Algorithmic work = 6*M*N*K FLOP per step per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

For N > 1 launch under torchrun: every rank runs the layer on its own batch shard of the same
size (weak scaling, replicated weights) and the parameter gradients dW, db are all-reduced (avg)
with NCCL, like Lux's DistributedOptimizer does per leaf.

Prints ONE JSON line (rank 0).
"""
from __future__ import annotations

import argparse
import json
import os
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


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d.get("bf16_tflops_sustained", 1430.0), d.get("bf16_tflops", 1699.0), "measured"
    return 1400.0, 1590.0, "fallback"


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
    """`--impl reference`: the CPU implementation of the path on the host cores. Julia is not
    available, so this is the numpy restatement of LuxLib's CPU code (kind "port"), BLAS-threaded
    over all host cores. Each step is a bounded sample (a column block of the batch)."""
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

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
            time.sleep(0.01)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# GPU arm
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
        # The persistent GEMM kernels occupy every SM; NCCL's in-switch (NVLS) all-reduce kernels compete with them
        # for SMs and measured slower here at 8 GPUs (5.0-5.4 PFLOP/s against 5.9 with plain ring / tree kernels).
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)
    lib = _cabi.load()
    if world > 1:   # leave a few SMs to the NCCL all-reduce that runs under the dX GEMM
        pass

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

    pending = []

    def start_allreduce(dW, db):
        # DistributedOptimizer's all-reduce(avg) of every parameter-gradient leaf, started as soon as the
        # leaves exist so that it runs underneath the dX GEMM. dW is column-major: .T is the contiguous
        # view of the same memory.
        pending.append(dist.all_reduce(dW.T, op=dist.ReduceOp.AVG, async_op=True))
        pending.append(dist.all_reduce(db, op=dist.ReduceOp.AVG, async_op=True))

    overlap = os.environ.get("LB2_BENCH_OVERLAP", "1") != "0"   # experiment switch: 0 = all-reduce after the whole pullback

    def backward(pullback):
        return backward_from(pullback, dy)

    def backward_from(pullback, dy_):
        if dist is None:
            return pullback(dy_)
        if overlap:
            dW, dx, db = pullback(dy_, on_param_grads=start_allreduce)
        else:
            dW, dx, db = pullback(dy_)
            start_allreduce(dW, db)
        for h in pending:
            h.wait()          # stream-level wait: the next step's work is ordered after the reduced gradients
        pending.clear()
        return dW, dx, db

    def step():
        y, pullback = L.rrule_fused_dense(ACT, W, x, b)
        dW, dx, db = backward(pullback)
        return y, dW, dx, db

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    rc = lib.lb2_poll_device_status(None)
    if rc != 0:
        raise SystemExit(f"device status after warm-up: {rc} {lib.lb2_last_error_string()}")

    # ---- timed region: K steps, CUDA events on the launching stream; the forward GEMM launch is
    # additionally bracketed by its own event pair to get the dominant kernel's launch duration.
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    fwd_ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    sampler.start()
    e0.record()
    for i in range(args.steps):
        fwd_ev[i][0].record()
        y, pullback = L.rrule_fused_dense(ACT, W, x, b)
        fwd_ev[i][1].record()
        dW, dx, db = backward(pullback)
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms_total = e0.elapsed_time(e1)
    t = torch.tensor([ms_total], device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * flops_per_step() / (ms_step * 1e-3) / 1e12
    fwd_ms = float(np.mean([a.elapsed_time(b_) for a, b_ in fwd_ev]))
    rc = lib.lb2_poll_device_status(None)
    if rc != 0:
        raise SystemExit(f"device status after the timed region: {rc} {lib.lb2_last_error_string()}")

    # ---- end to end through the public API with HOST buffers (pinned): per step copy this step's
    # inputs (x, dy) to the device, run, and read every result (y, dW, dx, db) back.
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
        y, pullback = L.rrule_fused_dense(ACT, W, dxbuf.T, b)
        dW, dx, db = backward_from(pullback, dybuf.T)
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

    for _ in range(2):
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

    line = None
    if rank == 0:
        sustained, burst, which = measured_peaks()
        achieved = 2.0 * M * N * K / (fwd_ms * 1e-3) / 1e12
        roofline = {
            "bound": "tensor", "kernel": "gemm_tc_kernel (forward GEMM, bias+gelu epilogue)", "achieved": achieved,
            "peak": sustained, "unit": "TFLOP/s", "frac": achieved / sustained,
            # dram__bytes_read.sum + dram__bytes_write.sum of one forward launch, from the ncu launch-list pass
            # (132.1 MB read + 103.3 MB written, Nsight Compute launch-list pass on this workload)
            "traffic": 235.4e6, "traffic_unit": "bytes per launch",
            "peak_source": f"{which}: bf16_tflops_sustained (kernel timed inside a long step); burst figure {burst}",
            "launch_ms": fwd_ms,
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
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "M": M, "N_per_gpu": N, "K": K, "gelu": L.ops.GELU_VARIANT,
                       "l2": "inputs larger than L2 (704 MB touched per step vs 126 MB L2)",
                       "parallelism": f"dp{world}: replicated W, per-GPU batch {N}, NCCL allreduce(avg) of dW and db" if world > 1 else "single GPU"},
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s * 1e3, "steps": e2e_steps,
                    "pipeline": "uploads, compute and downloads on three streams, double-buffered; wall clock over all steps"},
            "gpu_launches": 5 * args.steps,   # fwd GEMM, g = dy*act' (+db partials), db finish, dW GEMM, dX GEMM
            "roofline": roofline,
            "cpu_baseline": cpu,
            "pct_of_measured_peak": {"sustained": value / world / sustained, "burst": value / world / burst},
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


# ---------------------------------------------------------------------------------------------
# secondary workloads (the other configurations of the path): one JSON line each, single GPU
# ---------------------------------------------------------------------------------------------
def hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("hbm_gbs", 6552.0), "measured"
    return 6650.0, "fallback"


def run_secondary(args):
    """--workload ln | gn | bn | conv  [--dtype f32|bf16]: norm rows report algorithmic GB/s
    (5*numel*sizeof(T) per fwd+bwd step) against the measured HBM copy bandwidth; conv reports
    TFLOP/s (3 x 2*Wo*Ho*N*Cout*Cin*kW*kH per step) against the measured bf16 tensor peak."""
    import torch
    import luxlib_b200 as L
    torch.cuda.set_device(0)
    tdt = torch.float32 if args.dtype == "f32" else torch.bfloat16
    es = 4 if args.dtype == "f32" else 2
    g = torch.Generator(device="cuda").manual_seed(3)
    rn = lambda *shape: torch.randn(*shape, device="cuda", generator=g)
    cm = lambda t: t.permute(*reversed(range(t.dim()))) if t.dim() > 1 else t  # row-major bytes -> Julia shape
    wl = args.workload
    if wl == "ln":
        D, R = 4096, 16384
        x = cm((rn(R, D) * 1.3).to(tdt)); dy = cm(rn(R, D).to(tdt))
        gam = (torch.rand(D, device="cuda", generator=g) + 0.5).to(tdt); bet = (rn(D) * 0.1).to(tdt)
        def step():
            y, pb = L.rrule_layernorm(x, gam, bet, "identity", None, 1e-5)
            return pb(dy)
        numel, launches, name = D * R, 3, "LayerNorm 4096x16384 (rows of 4096), affine, fwd+bwd"
    elif wl == "gn":
        shape = (128, 512, 32, 32)  # N, C, H, W row-major == WHCN column-major
        x = cm((rn(*shape) * (torch.rand(1, 512, 1, 1, device="cuda", generator=g) * 1.5 + 0.5)).to(tdt)); dy = cm(rn(*shape).to(tdt))
        gam = (torch.rand(512, device="cuda", generator=g) + 0.5).to(tdt); bet = (rn(512) * 0.1).to(tdt)
        def step():
            y, pb = L.rrule_groupnorm(x, gam, bet, 32, "identity", 1e-5)
            return pb(dy)
        numel, launches, name = 128 * 512 * 32 * 32, 3, "GroupNorm(32 groups) 32x32x512x128, affine, fwd+bwd"
    elif wl == "bn":
        shape = (256, 64, 56, 56)
        x = cm(rn(*shape).to(tdt)); dy = cm(rn(*shape).to(tdt))
        gam = torch.ones(64, device="cuda", dtype=tdt); bet = torch.zeros(64, device="cuda", dtype=tdt)
        rm = torch.zeros(64, device="cuda", dtype=tdt); rv = torch.ones(64, device="cuda", dtype=tdt)
        def step():
            y, st, pb = L.rrule_batchnorm(x, gam, bet, rm, rv, True, "relu", 0.1, 1e-5)
            return pb(dy)
        numel, launches, name = 256 * 64 * 56 * 56, 6, "BatchNorm(64)+relu 56x56x64x256 training, running stats, fwd+bwd"
    elif wl == "conv":
        x = cm(rn(256, 64, 56, 56).to(tdt)); dy = cm(rn(256, 64, 56, 56).to(tdt))
        w = cm((rn(64, 64, 3, 3) * (2.0 / 576) ** 0.5).to(tdt)); b = torch.zeros(64, device="cuda", dtype=tdt)
        cd = L.ConvDims.make(2, 1, 1, 1, 1, False)
        def step():
            y, pb = L.rrule_fused_conv("identity", w, x, b, cd)
            return pb(dy)
        numel, launches, name = 256 * 64 * 56 * 56, 0, "Conv 3x3 64->64 s1 p1 on 56x56x64x256, fwd + dx + dw + db"
    else:
        raise SystemExit(f"unknown workload {wl}")
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    torch.cuda.synchronize()
    sampler = ClockSampler(0)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / args.steps
    rc = L._cabi.load().lb2_poll_device_status(None)
    if rc != 0:
        raise SystemExit(f"device status {rc}")
    if wl == "conv":
        flop = 3 * 2.0 * 56 * 56 * 256 * 64 * 64 * 9
        sustained, burst, which = measured_peaks()
        val = flop / (ms * 1e-3) / 1e12
        line = {"metric": "fused conv+bias+act fwd+bwd TFLOP/s", "value": val, "unit": "TFLOP/s",
                "roofline": {"bound": "tensor", "achieved": val, "peak": sustained, "unit": "TFLOP/s", "frac": val / sustained,
                             "traffic": None, "peak_source": f"{which}: bf16_tflops_sustained; whole step (layout passes, 3 GEMM-like kernels, reductions)"}}
    else:
        byts = 5.0 * numel * es
        peak, which = hbm_peak()
        val = byts / (ms * 1e-3) / 1e9
        line = {"metric": "norm fwd+bwd HBM GB/s", "value": val, "unit": "GB/s",
                "roofline": {"bound": "hbm", "achieved": val, "peak": peak, "unit": "GB/s", "frac": val / peak, "traffic": None,
                             "peak_source": f"{which}: hbm_gbs; algorithmic bytes 5*numel*sizeof(T) over the whole fwd+bwd step"}}
    line.update({"n_gpus": 1, "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
                 "vs_baseline": None, "dtype": args.dtype, "data": "synthetic", "config": {"workload": name}, "clocks": clocks,
                 "gpu_launches": launches * args.steps if launches else None})
    print(json.dumps(line), flush=True)
    return 0


def run_convnet(args):
    """--workload convnet: a data-parallel training step of the stride-1 stage of a ResNet-18-style network
    (two basic blocks of conv3x3-BN-relu / conv3x3-BN / residual-add-relu on 56x56x64, global mean pool,
    Dense 64 -> 1000, mean-squared error against one-hot labels), bf16, per-GPU batch 256, momentum SGD.
    Every rank holds the same parameters and its own synthetic batch; parameter gradients go through one flat
    sum all-reduce per bucket and one lb2_optimizer_step launch (1/world folded in). Reports samples/s over all
    ranks. The strided stages of the full network are not included (their convolutions have no tensor-core
    path yet)."""
    import torch
    import luxlib_b200 as L
    from luxlib_b200 import distributed as D
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        D.initialize(D.NCCLBackend)
        import torch.distributed as dist
    bf = torch.bfloat16
    Bsz, C, H, NCLS = 256, 64, 56, 1000
    gp = torch.Generator(device="cuda").manual_seed(5)               # parameters: same on every rank
    gd = torch.Generator(device="cuda").manual_seed(100 + rank)      # data: one shard per rank
    cm = lambda t: t.permute(*reversed(range(t.dim()))) if t.dim() > 1 else t   # row-major bytes -> Julia shape
    rnp = lambda *sh: torch.randn(*sh, device=device, generator=gp)
    convs = [cm((rnp(C, C, 3, 3) * (2.0 / (9 * C)) ** 0.5).to(bf)) for _ in range(4)]       # kaiming_normal
    cbias = [torch.zeros(C, device=device, dtype=bf) for _ in range(4)]
    gam = [torch.ones(C, device=device, dtype=bf) for _ in range(4)]
    bet = [torch.zeros(C, device=device, dtype=bf) for _ in range(4)]
    rmean = [torch.zeros(C, device=device, dtype=bf) for _ in range(4)]
    rvar = [torch.ones(C, device=device, dtype=bf) for _ in range(4)]
    lim = (24.0 / (C + NCLS)) ** 0.5
    Wd = cm(((torch.rand(C, NCLS, device=device, generator=gp) - 0.5) * lim).to(bf))        # (1000, 64) glorot_uniform
    bd = torch.zeros(NCLS, device=device, dtype=bf)
    x = cm(torch.randn(Bsz, C, H, H, device=device, generator=gd).to(bf))
    labels = torch.randint(0, NCLS, (Bsz,), device=device, generator=gd)
    target = cm(torch.nn.functional.one_hot(labels, NCLS).to(bf))                           # (1000, B)
    params = convs + cbias + gam + bet + [Wd, bd]
    opt = D.FusedOptimizer(D.NCCLBackend, "momentum", eta=1e-3, rho=0.9)
    states = opt.init(params)
    cd = L.ConvDims.make(2, 1, 1, 1, 1, False)

    def step():
        h, tape = x, []
        for blk in range(2):
            skip = h
            i0, i1 = 2 * blk, 2 * blk + 1
            c0, pc0 = L.rrule_fused_conv("identity", convs[i0], h, cbias[i0], cd)
            n0, (rmean[i0], rvar[i0]), pn0 = L.rrule_batchnorm(c0, gam[i0], bet[i0], rmean[i0], rvar[i0], True, "relu", 0.1, 1e-5)
            c1, pc1 = L.rrule_fused_conv("identity", convs[i1], n0, cbias[i1], cd)
            n1, (rmean[i1], rvar[i1]), pn1 = L.rrule_batchnorm(c1, gam[i1], bet[i1], rmean[i1], rvar[i1], True, "identity", 0.1, 1e-5)
            h, padd = L.rrule_add_activation("relu", n1, skip)
            tape.append((pc0, pn0, pc1, pn1, padd))
        pooled, ppool = L.rrule_meanpool(h, L.PoolDims.global_(h))          # (1, 1, 64, B)
        feat = pooled.reshape(C, Bsz)                                        # same bytes, Julia shape (64, B)
        y, pdense = L.rrule_fused_dense("identity", Wd, feat, bd)
        # loss glue (tiny, 1000 x B): mean-squared error and its gradient
        diff = y - target
        loss = (diff.float() ** 2).mean()
        dy = diff * (2.0 / diff.numel())
        grads = [None] * len(params)
        dWd, dfeat, dbd = pdense(dy)
        grads[16], grads[17] = dWd, dbd
        dh = ppool(dfeat.reshape(1, 1, C, Bsz))
        for blk in (1, 0):
            pc0, pn0, pc1, pn1, padd = tape[blk]
            i0, i1 = 2 * blk, 2 * blk + 1
            dn1, dskip = padd(dh)
            dc1, grads[8 + i1], grads[12 + i1] = pn1(dn1)
            grads[i1], dn0, grads[4 + i1] = pc1(dc1)
            dc0, grads[8 + i0], grads[12 + i0] = pn0(dn0)
            grads[i0], dx0, grads[4 + i0] = pc0(dc0)
            dh = L.add_activation("identity", dx0, dskip)
        opt.update(states, params, grads)
        return loss

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    warm = max(args.warmup, 3)
    for _ in range(warm):
        step()
    barrier()
    sampler = ClockSampler(local)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    sampler.start()
    e0.record()
    for _ in range(args.steps):
        loss = step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    t = torch.tensor([e0.elapsed_time(e1)], device=device)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / args.steps
    rc = L._cabi.load().lb2_poll_device_status(None)
    if rc != 0:
        raise SystemExit(f"device status {rc}")
    if rank == 0:
        flop = 4 * 3 * 2.0 * H * H * Bsz * C * C * 9 + 3 * 2.0 * NCLS * C * Bsz
        sustained, burst, which = measured_peaks()
        tf = world * flop / (ms * 1e-3) / 1e12
        line = {"metric": "data-parallel conv-net step samples/s", "value": world * Bsz / (ms * 1e-3), "unit": "samples/s",
                "n_gpus": world, "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": "ResNet-18-style stride-1 stage: 2 basic blocks (conv3x3-BN-relu, conv3x3-BN, add-relu) on "
                                       "56x56x64, global mean pool, Dense 64->1000, MSE; per-GPU batch 256; momentum SGD fused with the "
                                       "gradient all-reduce bucket",
                           "parallelism": f"dp{world}", "final_loss": float(loss)},
                "clocks": clocks, "gpu_launches": None,
                "roofline": {"bound": "tensor", "achieved": tf, "peak": world * sustained, "unit": "TFLOP/s", "frac": tf / (world * sustained),
                             "traffic": None, "peak_source": f"{which}: bf16_tflops_sustained x n_gpus; conv + dense FLOPs of the whole step"}}
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense", choices=["dense", "ln", "gn", "bn", "conv", "convnet"],
                    help="dense = the headline configuration (default); ln/gn/bn/conv are single-GPU secondary rows; "
                         "convnet = data-parallel conv-net stage step (any --gpus, under torchrun for N > 1)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"], help="storage type of the secondary workloads")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.workload == "convnet":
        return run_convnet(args)
    if args.workload != "dense":
        return run_secondary(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
