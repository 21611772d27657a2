#!/usr/bin/env python
"""Benchmark of the dense-contraction path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one training step of the large MLP configuration
(8192 -> 4096 -> 4096 -> 4096 -> 1000 with ReLU, CrossEntropy, Adam, global batch
65536 f32, N(0,1) inputs, labels uniform in [0,1000), He-uniform weights),
batch-sharded by rows over N GPUs (one process per GPU, NCCL all-reduce of the
parameter gradients).  The metric is whole-job training samples per second.
At N = 1 the same line also carries the f32 4096^3 GEMM rate and the CPU
baseline.  All inputs are synthetic and seeded; nothing is read from disk.

`--impl reference` times the CPU restatement of the reference's own training
step (oracle/oracle.cpp, OpenMP over the host cores) on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

DIMS = [8192, 4096, 4096, 4096, 1000]
GLOBAL_BATCH = 65536
METRIC = "mlp_train_samples_per_s"
UNIT = "samples/s"
WORKLOAD = "MLP 8192-4096-4096-4096-1000 ReLU + CrossEntropy + Adam, f32, global batch 65536"


def _traffic(key: str):
    """A record of profiles/dram_traffic.json (DRAM bytes per launch from an ncu capture), or None."""
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        return json.load(open(p)).get(key)
    except (OSError, ValueError):
        return None


def record_traffic(csv_path: str, key: str, kernel_regex: str, command: str):
    """Fold an ncu raw CSV (--page raw --csv, or --csv --log-file) into profiles/dram_traffic.json: mean of
    dram__bytes_read.sum + dram__bytes_write.sum over the captured launches whose kernel name matches.  Several
    expressions joined by " + " record the SUM of their means (a call made of a tensor kernel and its fix-up)."""
    import csv
    import re
    if " + " in kernel_regex:
        total, launches = 0.0, 0
        for part in kernel_regex.split(" + "):
            rec = record_traffic(csv_path, key, part.strip(), command)
            total += rec["dram_bytes_per_launch"]
            launches += rec["launches_captured"]
        p = os.path.join(ROOT, "profiles", "dram_traffic.json")
        data = json.load(open(p))
        data[key].update(dram_bytes_per_launch=total, launches_captured=launches, kernels=kernel_regex)
        json.dump(data, open(p, "w"), indent=2)
        print(json.dumps({key: data[key]}))
        return data[key]
    rows = list(csv.reader(open(csv_path, errors="replace")))
    hdr_i = next(i for i, r in enumerate(rows) if "Kernel Name" in r)
    hdr = rows[hdr_i]
    per_launch = {}
    if "Metric Name" in hdr:        # long form: one row per (launch, metric)
        ki, mi, vi, ui, idi = (hdr.index(c) for c in ("Kernel Name", "Metric Name", "Metric Value", "Metric Unit", "ID"))
        for r in rows[hdr_i + 1:]:
            if len(r) <= vi or not re.search(kernel_regex, r[ki]) or not r[mi].startswith("dram__bytes_"):
                continue
            mult = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(r[ui], 1.0)
            per_launch[r[idi]] = per_launch.get(r[idi], 0.0) + float(r[vi].replace(",", "")) * mult
    else:                           # wide form: one row per launch, a units row after the header
        units = rows[hdr_i + 1]
        ki = hdr.index("Kernel Name")
        cols = [i for i, c in enumerate(hdr) if c in ("dram__bytes_read.sum", "dram__bytes_write.sum")]
        for n, r in enumerate(rows[hdr_i + 2:]):
            if len(r) <= max(cols) or not re.search(kernel_regex, r[ki]):
                continue
            tot = 0.0
            for i in cols:
                mult = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9}.get(units[i], 1.0)
                tot += float(r[i].replace(",", "")) * mult
            per_launch[n] = tot
    if not per_launch:
        raise SystemExit(f"no launch of /{kernel_regex}/ with DRAM byte counters in {csv_path}")
    p = os.path.join(ROOT, "profiles", "dram_traffic.json")
    data = json.load(open(p)) if os.path.exists(p) else {}
    commit = subprocess.run(["git", "-C", ROOT, "rev-parse", "--short", "HEAD"], stdout=subprocess.PIPE, text=True).stdout.strip()
    rec = data.get(key, {})
    rec.update(command=command, commit=commit, launches_captured=len(per_launch),
               dram_bytes_per_launch=sum(per_launch.values()) / len(per_launch))
    data[key] = rec
    json.dump(data, open(p, "w"), indent=2)
    print(json.dumps({key: rec}))
    return rec


def _peaks():
    """Measured peaks of this pool (driver-written file), else the stated fallback."""
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clock / throttle samples taken while the timed region runs."""

    Q = ("timestamp,index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.proc = None
        self.idx = device_index
        self.t0 = self.t1 = None

    def mark_begin(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "20", "-i",
                 str(self.idx)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=10)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        import datetime
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                ts = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                rows.append((ts, float(f[2]), float(f[3]), float(f[4]), f[5:9]))
            except ValueError:
                continue
        # samples taken while the timed region ran (the sampler starts before the warm-up steps); if the
        # region was shorter than the sampling period, fall back to the nearest samples under load
        inside = [r for r in rows if self.t0 is not None and self.t0 - 0.05 <= r[0] <= self.t1 + 0.05]
        if not inside and rows and self.t0 is not None:
            inside = sorted(rows, key=lambda r: abs(r[0] - 0.5 * (self.t0 + self.t1)))[:2]
        for ts, c, m, p, flags in (inside or rows):
            sm.append(c); mx.append(m); power.append(p)
            for n, v in zip(names, flags):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# ---------------------------------------------------------------------- CPU side
def cpu_mlp_samples_per_s(sample_rows: int, steps: int, warmup: int):
    """Times oracle.mlp_train_step (the reference's step restated for the CPU) on `sample_rows` rows."""
    import oracle
    oracle.build()
    from minitensor_b200.mlp import mlp_layout
    rng = np.random.default_rng(1)
    _, _, total = mlp_layout(DIMS)
    params = np.zeros(total, dtype=np.float32)
    w_off, b_off, _ = mlp_layout(DIMS)
    for l in range(len(DIMS) - 1):
        n = DIMS[l] * DIMS[l + 1]
        params[w_off[l]:w_off[l] + n] = rng.uniform(-1, 1, n).astype(np.float32) * np.float32(np.sqrt(6.0 / DIMS[l]))
    m, v = np.zeros_like(params), np.zeros_like(params)
    x = rng.standard_normal((sample_rows, DIMS[0])).astype(np.float32)
    labels = rng.integers(0, DIMS[-1], sample_rows)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        oracle.mlp_train_step(DIMS, x, labels, params, m, v, 1e-3, 0.9, 0.999, 1e-8, i + 1)
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    per_step = sum(times) / len(times)
    return sample_rows / per_step, per_step, oracle.num_threads()


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # the launcher of multi-rank runs pins OMP_NUM_THREADS to 1; this arm is the CPU path on ALL host cores,
    # and the OpenMP runtime reads the variable when the oracle library is first loaded
    if "LOCAL_RANK" in os.environ:
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)) or 1)
    rows = 2048
    value, per_step, cores = cpu_mlp_samples_per_s(rows, max(1, args.steps), max(0, min(args.warmup, 1)))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": min(args.warmup, 1), "ms_per_step": per_step * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": f"{rows} of {GLOBAL_BATCH} rows per step, same layer sizes"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": f"one reference-ordered training step on {rows} rows (of {GLOBAL_BATCH}); "
                                   "the reference itself is Rust and cannot be built on this box"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------- GPU side
def gemm4096(be, torch, peaks):
    """f32 4096^3 through the public GEMM call: whole call (operand splits + tensor kernel) and the
    tensor kernel alone, L2 flushed between iterations."""
    n = 4096
    g = torch.Generator(device="cpu").manual_seed(7)
    a = torch.randn(n, n, generator=g).to(be.device)
    b = torch.randn(n, n, generator=g).to(be.device)
    out = torch.empty(n, n, device=be.device)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=be.device)
    for _ in range(3):
        be.gemm(a, b, out=out)
    torch.cuda.synchronize()
    iters = 10

    def timed_calls():
        total = 0.0
        for _ in range(iters):
            flush.fill_(1)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            be.gemm(a, b, out=out)
            e.record()
            torch.cuda.synchronize()
            total += s.elapsed_time(e)
        return total

    total = timed_calls()                 # the call as a user makes it (launch profiler off)
    be.profile(True)                      # a second pass with an event pair around the tensor kernel
    timed_calls()
    launches, kms, kwork = be.profile_read(0)
    be.profile(False)
    ms = total / iters
    flops = 2.0 * n ** 3
    peak = peaks["bf16_burst"] / 3.0        # this mode's own roofline: three 16-bit tensor products per f32 product
    peak_3xtf32 = peaks["bf16_burst"] / 6.0  # what a 3xTF32 emulation (three TF32 MMAs at half rate) could reach
    tf = flops / ms / 1e9
    ktf = kwork / kms / 1e9 if kms else None
    return {"ms": ms, "tflops": tf, "pct_of_peak": 100.0 * tf / peak,
            "pct_of_3xtf32_emulated_peak": 100.0 * tf / peak_3xtf32,
            "kernel_only_tflops": ktf, "kernel_only_pct_of_peak": 100.0 * ktf / peak if ktf else None,
            "peak_tflops": peak, "peak_3xtf32_emulated_tflops": peak_3xtf32, "f32_mode": "f16x3",
            "peak_def": "measured 16-bit dense tensor burst (cuBLAS bf16) / 3 products per f32 product; the "
                        "3xTF32-emulated peak is the same burst / 6",
            "dram_traffic": _traffic("gemm_f32_4096.whole_call_tensor_kernel_plus_fixup")}



def _time_gpu(torch, fn, flush, iters=5, warm=2):
    """Median device time (ms) of fn() over `iters` calls, event-timed on the current stream, L2 flushed (a buffer
    larger than L2 is rewritten) before every timed call."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        flush.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    return statistics.median(times)


def _norm_err(c, ref, a, b):
    """max |c - ref| / (||a_row|| ||b_col||) over the given rows (a [r,K], b [K,N], float64 arithmetic)."""
    na = np.linalg.norm(a.astype(np.float64), axis=-1)[..., :, None]
    nb = np.linalg.norm(b.astype(np.float64), axis=-2)[..., None, :]
    return float((np.abs(c.astype(np.float64) - ref.astype(np.float64)) / np.maximum(na * nb, 1e-300)).max())


def config_table(be, torch, peaks, with_cpu: bool):
    """Every configuration of the benchmark list beside the headline one, each as one record: whole-call device
    time (operand preparation included, L2 flushed between calls), rate, fraction of the roofline that bounds it,
    and - in the CPU leg - the oracle's time on the host cores with its thread count and the largest
    norm-scaled error of the device result.  Sizes whose CPU time is impractical are timed on the CPU at a
    smaller, stated size and never extrapolated."""
    dev = be.device
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    g = torch.Generator(device="cpu").manual_seed(7)
    orc = None
    if with_cpu:
        import oracle as orc
        orc.build()
    threads = orc.num_threads() if orc else None
    f32_peak = peaks["bf16_burst"] / 3.0          # fp16 two-plane mode: three 16-bit products per f32 product
    i8_peak = peaks["bf16_burst"] * 2.0           # kind::i8 runs at twice the 16-bit rate; entries in [-8,8] need one product
    out = []

    def cpu_time(fn, reps=1):
        best = None
        for _ in range(reps):
            t0 = time.perf_counter()
            r = fn()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        return best * 1e3, r

    # ---- C1: 1024^3 f32 forward + backward (upstream gradient of ones)
    n = 1024
    a, b = torch.randn(n, n, generator=g), torch.randn(n, n, generator=g)
    ad, bd, dy = a.to(dev), b.to(dev), torch.ones(n, n, device=dev)
    c, da, db_ = (torch.empty(n, n, device=dev) for _ in range(3))
    fwd = lambda: be.gemm(ad, bd, out=c)
    bwd = lambda: (be.gemm(dy, bd, trans_b=True, out=da), be.gemm(ad, dy, trans_a=True, out=db_))
    ms_f, ms_b = _time_gpu(torch, fwd, flush), _time_gpu(torch, bwd, flush)
    rec = {"config": "C1 matmul f32 1024^3 forward + backward (dY = ones)", "dtype": "f32", "gpu_ms": ms_f + ms_b,
           "gpu_ms_forward": ms_f, "gpu_ms_backward": ms_b, "tflops": 3 * 2.0 * n ** 3 / (ms_f + ms_b) / 1e9,
           "tflops_forward": 2.0 * n ** 3 / ms_f / 1e9, "bound": "tensor", "peak_tflops": f32_peak}
    rec["roofline_frac"] = rec["tflops"] / f32_peak
    if orc:
        an, bn = a.numpy(), b.numpy()
        ones = np.ones((n, n), np.float32)
        t1, ref = cpu_time(lambda: orc.matmul(an, bn), 2)
        t2, (rda, rdb) = cpu_time(lambda: orc.matmul_backward(an, bn, ones), 2)
        rec.update(cpu_ms=t1 + t2, cpu_threads=threads, cpu_size="same",
                   max_err=max(_norm_err(c.cpu().numpy(), ref, an, bn), _norm_err(da.cpu().numpy(), rda, ones, bn.T),
                               _norm_err(db_.cpu().numpy(), rdb, an.T, ones)))
    out.append(rec)

    # ---- bmm f32 [64,512,512] x [64,512,512]
    a, b = torch.randn(64, 512, 512, generator=g), torch.randn(64, 512, 512, generator=g)
    ad, bd = a.to(dev), b.to(dev)
    c = torch.empty(64, 512, 512, device=dev)
    ms = _time_gpu(torch, lambda: be.gemm(ad, bd, out=c), flush)
    rec = {"config": "bmm f32 [64,512,512] x [64,512,512]", "dtype": "f32", "gpu_ms": ms,
           "tflops": 64 * 2.0 * 512 ** 3 / ms / 1e9, "bound": "tensor", "peak_tflops": f32_peak}
    rec["roofline_frac"] = rec["tflops"] / f32_peak
    if orc:
        an, bn = a.numpy(), b.numpy()
        t1, ref = cpu_time(lambda: orc.matmul(an, bn))
        rec.update(cpu_ms=t1, cpu_threads=threads, cpu_size="same", max_err=_norm_err(c.cpu().numpy(), ref, an, bn))
    out.append(rec)
    del a, b, ad, bd, c

    # ---- square sweep, M = N = K in {256, 1024, 4096, 8192} x {f32, f64, i32}
    # a single CPU timing predicted (from the previous size, by the cube of the size ratio) to exceed this is not
    # run; the prediction is optimistic once the operands leave the caches, hence the margin
    cpu_budget_s = 8.0
    for dt_name, tdt in (("f32", torch.float32), ("f64", torch.float64), ("i32", torch.int32)):
        last_cpu = None     # (size, ms) of the largest CPU run of this dtype
        for n in (256, 1024, 4096, 8192):
            if dt_name == "i32":
                a = torch.randint(-8, 9, (n, n), generator=g, dtype=torch.int32)
                b = torch.randint(-8, 9, (n, n), generator=g, dtype=torch.int32)
            else:
                a, b = torch.randn(n, n, generator=g, dtype=tdt), torch.randn(n, n, generator=g, dtype=tdt)
            ad, bd = a.to(dev), b.to(dev)
            c = torch.empty(n, n, dtype=tdt, device=dev)
            ms = _time_gpu(torch, lambda: be.gemm(ad, bd, out=c), flush, iters=5 if n < 8192 else 3)
            ops = 2.0 * n ** 3
            rec = {"config": f"square {dt_name} {n}^3", "dtype": dt_name, "gpu_ms": ms, "tflops": ops / ms / 1e9}
            algo_bytes = 3.0 * n * n * a.element_size()
            if n == 256:      # launch / HBM-bound: microseconds and bytes are the meaningful figures
                rec.update(bound="hbm", gpu_us=ms * 1e3, gbs=algo_bytes / ms / 1e6, peak_gbs=peaks["hbm_gbs"],
                           roofline_frac=algo_bytes / ms / 1e6 / peaks["hbm_gbs"])
            elif dt_name == "f32":
                rec.update(bound="tensor", peak_tflops=f32_peak, roofline_frac=rec["tflops"] / f32_peak,
                           frac_of_3xtf32_emulated_peak=rec["tflops"] / (peaks["bf16_burst"] / 6.0))
            elif dt_name == "i32":
                rec.update(bound="tensor", pipe="int8 tensor cores (tcgen05 kind::i8), one s8 product per int32 product "
                           "for entries that fit in int8", peak_tflops=i8_peak, roofline_frac=rec["tflops"] / i8_peak,
                           peak_def="2 x measured 16-bit dense tensor burst")
            else:
                # no measured FP64 tensor peak exists for this pool: the anchor is the vendor library's dgemm on
                # the same operands in the same run (measurement only; it is not on the product path)
                cref = torch.empty(n, n, dtype=tdt, device=dev)
                ms_lib = _time_gpu(torch, lambda: torch.matmul(ad, bd, out=cref), flush, iters=5 if n < 8192 else 3)
                rec.update(bound="fp64 tensor (mma.sync)", cublas_dgemm_ms=ms_lib, cublas_dgemm_tflops=ops / ms_lib / 1e9,
                           roofline_frac=ms_lib / ms, peak_def="vendor dgemm measured in the same run")
                del cref
            if orc:
                an, bn = a.numpy(), b.numpy()
                predicted = last_cpu[1] * (n / last_cpu[0]) ** 3 / 1e3 if last_cpu else 0.0
                if predicted <= cpu_budget_s:
                    t1, ref = cpu_time(lambda: orc.matmul(an, bn), 2 if n <= 1024 else 1)
                    last_cpu = (n, t1)
                    rec.update(cpu_ms=t1, cpu_threads=threads, cpu_size="same")
                    got = c.cpu().numpy()
                    rec["max_err"] = 0.0 if dt_name == "i32" and np.array_equal(got, ref) else (
                        _norm_err(got, ref, an, bn) if dt_name != "i32" else float("inf"))
                    if dt_name == "i32":
                        rec["bit_exact"] = bool(np.array_equal(got, ref))
                else:
                    rec.update(cpu_ms=last_cpu[1], cpu_threads=threads,
                               cpu_size=f"{last_cpu[0]}^3 (this size is impractical for the CPU loop; not extrapolated)")
                    rows = np.random.default_rng(n).choice(n, 8, replace=False)
                    ar = np.ascontiguousarray(an[rows])
                    got = c[torch.from_numpy(rows).to(dev)].cpu().numpy()
                    if dt_name == "i32":
                        rec["bit_exact"] = bool(np.array_equal(got, orc.matmul(ar, bn)))
                        rec["max_err"] = 0.0 if rec["bit_exact"] else float("inf")
                    else:
                        rec["max_err"] = _norm_err(got, orc.matmul_acc_wide(ar, bn), ar, bn)
                    rec["err_sample"] = "8 rows, all columns"
            out.append(rec)
            del a, b, ad, bd, c

    # ---- C4: conv2d f32 [128,64,56,56] * [64,64,3,3], stride 1, pad 1, bias: forward, dX, dW, db
    N, C_, H, W_, O = 128, 64, 56, 56, 64
    x = torch.randn(N, C_, H, W_, generator=g)
    w = torch.randn(O, C_, 3, 3, generator=g) * (2.0 / (C_ * 9)) ** 0.5      # Kaiming-normal
    bias = torch.randn(O, generator=g)
    dy = torch.randn(N, O, H, W_, generator=g)
    xd, wd, bd, dyd = x.to(dev), w.to(dev), bias.to(dev), dy.to(dev)
    s1, p1 = (1, 1), (1, 1)
    res = {}
    calls = {"forward": lambda: res.__setitem__("y", be.conv2d_fwd(xd, wd, bd, s1, p1)),
             "dX": lambda: res.__setitem__("dx", be.conv2d_bwd_data(dyd, wd, xd.shape, s1, p1)),
             "dW": lambda: res.__setitem__("dw", be.conv2d_bwd_weight(dyd, xd, wd.shape, s1, p1)),
             "db": lambda: res.__setitem__("db", be.conv2d_bwd_bias(dyd))}
    flops = 2.0 * N * O * H * W_ * C_ * 9
    rec = {"config": "C4 conv2d f32 [128,64,56,56] * [64,64,3,3] s1 p1 + bias: forward, dX, dW, db", "dtype": "f32",
           "bound": "tensor", "peak_tflops": f32_peak, "parts": {}}
    total_ms = 0.0
    for name, fn in calls.items():
        ms = _time_gpu(torch, fn, flush)
        total_ms += ms
        part = {"gpu_ms": ms}
        if name == "db":
            part.update(gbs=4.0 * dy.numel() / ms / 1e6, roofline_frac=4.0 * dy.numel() / ms / 1e6 / peaks["hbm_gbs"], bound="hbm")
        else:
            part.update(tflops=flops / ms / 1e9, roofline_frac=flops / ms / 1e9 / f32_peak)
        rec["parts"][name] = part
    rec["gpu_ms"] = total_ms
    rec["tflops"] = 3 * flops / total_ms / 1e9
    rec["roofline_frac"] = rec["tflops"] / f32_peak
    if orc:
        from oracle import conv_f64
        xn, wn, bn_, dyn = x.numpy(), w.numpy(), bias.numpy(), dy.numpy()
        t1, _ = cpu_time(lambda: orc.conv2d(xn, wn, bn_, s1, p1))
        t2, _ = cpu_time(lambda: orc.conv2d_backward(xn, wn, dyn, s1, p1))
        rec.update(cpu_ms=t1 + t2, cpu_ms_forward=t1, cpu_ms_backward=t2, cpu_threads=threads, cpu_size="same")
        yh, dxh, dwh = res["y"].cpu().numpy(), res["dx"].cpu().numpy(), res["dw"].cpu().numpy()
        pick = np.random.default_rng(11)
        worst = 0.0
        for _ in range(96):
            n_, o_, c_, h_, w_ = (int(pick.integers(k)) for k in (N, O, C_, H, W_))
            v, sc = conv_f64.sample_forward(xn, wn, bn_, p1, n_, o_, h_, w_)
            worst = max(worst, abs(float(yh[n_, o_, h_, w_]) - v) / (sc + abs(float(bn_[o_]))))
            v, sc = conv_f64.sample_grad_input(dyn, wn, p1, n_, c_, h_, w_)
            worst = max(worst, abs(float(dxh[n_, c_, h_, w_]) - v) / sc)
            i_, j_ = int(pick.integers(3)), int(pick.integers(3))
            v, sc = conv_f64.sample_grad_weight(dyn, xn, p1, o_, c_, i_, j_)
            worst = max(worst, abs(float(dwh[o_, c_, i_, j_]) - v) / sc)
        rec.update(max_err=worst, err_sample="96 outputs each of y, dX, dW as float64 dot products")
    out.append(rec)
    return out


def dp_check(torch, dist, world, rank, local, comm):
    """Data-parallel parity on the real collective path, before anything is timed: one training step of a small
    fixed model (512-384-256-100, global batch 2048, the same seeds on every rank) through MLPTrainer(world_size =
    N) with its overlapped schedule and the library's NCCL all-reduce, against a world_size = 1 trainer of the same
    process fed the whole batch.  Reports the largest relative Frobenius distance between a layer's averaged
    gradient and the full-batch gradient, the largest parameter difference after the Adam step, and whether the
    parameter checksums of all ranks agree."""
    from minitensor_b200.mlp import MLPTrainer, mlp_layout, shard_rows
    dims, gbatch = [512, 384, 256, 100], 2048
    g = torch.Generator(device="cpu").manual_seed(4242)
    x = torch.randn(gbatch, dims[0], generator=g)
    y = torch.randint(0, dims[-1], (gbatch,), generator=g, dtype=torch.int64)
    lo, hi = shard_rows(gbatch, world, rank)
    dev = torch.device("cuda", local)
    shard = MLPTrainer(dims, hi - lo, device=local, world_size=world, seed=5, comm=comm)
    full = MLPTrainer(dims, gbatch, device=local, world_size=1, seed=5)
    shard.step(x[lo:hi].to(dev), y[lo:hi].to(dev))
    full.step(x.to(dev), y.to(dev))
    torch.cuda.synchronize()
    w_off, b_off, total = mlp_layout(dims)
    err = 0.0
    for l in range(len(dims) - 1):
        a, b = w_off[l], b_off[l] + dims[l + 1]
        gs, gf = shard.grads[a:b].double() / world, full.grads[a:b].double()
        err = max(err, float((gs - gf).norm() / gf.norm()))
    pdiff = float((shard.params - full.params).abs().max())
    chk = shard.params_checksum()
    lo_t, hi_t = chk.clone(), chk.clone()
    dist.all_reduce(lo_t, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi_t, op=dist.ReduceOp.MAX)
    e = torch.tensor([err, pdiff], dtype=torch.float64, device=dev)
    dist.all_reduce(e, op=dist.ReduceOp.MAX)
    return {"model": "512-384-256-100, global batch 2048, one step", "grad_err_norm_scaled": float(e[0]),
            "grad_err_def": "max over layers and ranks of ||g_allreduced / N - g_full_batch||_F / ||g_full_batch||_F",
            "param_max_abs_diff_after_adam": float(e[1]),
            "params_equal_across_ranks": bool(torch.equal(lo_t, hi_t))}


def run_ours(args):
    # stdout carries exactly one JSON line: whatever libraries print on the way (NCCL's version banner, warnings)
    # goes to stderr; the descriptor is put back just before the line is printed
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)
    try:
        return _run_ours(args, saved_stdout)
    finally:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        os.close(saved_stdout)


def _run_ours(args, saved_stdout):
    import torch
    import torch.distributed as dist
    from minitensor_b200.mlp import MLPTrainer, mlp_flops_per_sample, shard_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            os.dup2(saved_stdout, 1)
            print(json.dumps({"error": f"--gpus {args.gpus} needs torchrun with {args.gpus} processes"}), flush=True)
            return 2
    torch.cuda.set_device(local)
    host_numa = None
    if world > 1:
        # host batches next to the GPU that reads them: with every rank copying at once, buffers on the far socket
        # make the socket interconnect the bound (hostmem.py); N = 1 keeps all cores for the CPU baseline
        from minitensor_b200.hostmem import bind_host_to_gpu
        host_numa = bind_host_to_gpu(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = _peaks()
    comm = None
    if world > 1:   # one NCCL communicator of the library for every trainer of this process
        from minitensor_b200.comm import Communicator
        comm = Communicator.from_process_group(local)
    dp = dp_check(torch, dist, world, rank, local, comm) if world > 1 else None
    lo, hi = shard_rows(GLOBAL_BATCH, world, rank)
    rows = hi - lo
    trainer = MLPTrainer(DIMS, rows, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, device=local, world_size=world, seed=0,
                         fused_dense=not args.per_product, comm=comm)
    be = trainer.be
    dev = be.device

    # synthetic shard, generated on the host (seeded per rank) and staged in pinned memory
    g = torch.Generator(device="cpu").manual_seed(1000 + rank)
    host_x = [torch.randn(rows, DIMS[0], generator=g).pin_memory() for _ in range(2)]
    host_y = [torch.randint(0, DIMS[-1], (rows,), generator=g, dtype=torch.int64).pin_memory() for _ in range(2)]
    x = host_x[0].to(dev)
    y = host_y[0].to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident steps (inputs already in HBM)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        trainer.step(x, y)
    barrier()
    sampler.mark_begin()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # Blocks of exactly `steps` steps, each bracketed by barrier + synchronize and timed with events (max over
    # ranks), repeated until the region has run for MIN_REGION_S so that clocks and power have settled; the
    # reported figure is the median block.  The launch profiler brackets the last block only.
    blocks_ms, loss = [], None
    region_t0 = time.time()
    while True:
        last = (time.time() - region_t0) >= args.min_region_s or len(blocks_ms) + 1 >= args.max_blocks
        if world > 1:   # every rank must take the same decision
            flag = torch.tensor([1 if last else 0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            last = bool(flag.item())
        if last:
            be.profile(True)
            launches0 = be.launches
        barrier()
        s.record()
        for _ in range(args.steps):
            loss = trainer.step(x, y)
        e.record()
        barrier()
        blocks_ms.append(max_over_ranks(s.elapsed_time(e)))
        if last:
            break
    sampler.mark_end()
    ms_last = blocks_ms[-1]
    ms_total = statistics.median(blocks_ms)
    clocks = sampler.stop() if rank == 0 else None
    gpu_launches = be.launches - launches0
    k_launches, k_ms, k_flops = be.profile_read(0)
    s_launches, s_ms, s_bytes = be.profile_read(1)
    be.profile(False)
    be.sync()
    mean_loss = loss.clone()
    if world > 1:
        dist.all_reduce(mean_loss, op=dist.ReduceOp.SUM)
        mean_loss /= world
    final_loss = float(mean_loss.item())
    ms_per_step = ms_total / args.steps
    value = GLOBAL_BATCH / (ms_per_step * 1e-3)
    chk = trainer.params_checksum()
    replicas_equal = True
    if world > 1:
        lo_t, hi_t = chk.clone(), chk.clone()
        dist.all_reduce(lo_t, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi_t, op=dist.ReduceOp.MAX)
        replicas_equal = bool(torch.equal(lo_t, hi_t))

    # ---- end to end: every step copies its batch from pinned host memory and reads the loss back
    slot = trainer.prefetch(host_x[0], host_y[0])
    for i in range(2):
        nxt = trainer.prefetch(host_x[(i + 1) % 2], host_y[(i + 1) % 2])
        float(trainer.step_slot(slot).item())
        slot = nxt
    barrier()
    s.record()
    for i in range(args.steps):
        nxt = trainer.prefetch(host_x[(i + 1) % 2], host_y[(i + 1) % 2])   # next batch: overlaps this step
        float(trainer.step_slot(slot).item())                            # loss read back every step
        slot = nxt
    e.record()
    barrier()
    e2e_ms = max_over_ranks(s.elapsed_time(e)) / args.steps
    e2e_value = GLOBAL_BATCH / (e2e_ms * 1e-3)
    h2d = rows * DIMS[0] * 4 + rows * 8
    # what the host link gives this rank while every rank copies at once and nothing else runs: the ceiling of
    # the end-to-end figure when the copy cannot hide behind the step any more
    stage = torch.empty(rows, DIMS[0], dtype=torch.float32, device=dev)
    barrier()
    s.record()
    for i in range(4):
        stage.copy_(host_x[i % 2], non_blocking=True)
    e.record()
    barrier()
    copy_ms = max_over_ranks(s.elapsed_time(e)) / 4
    h2d_ceiling_gbs = rows * DIMS[0] * 4 / copy_ms / 1e6
    del stage

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    peak_f32 = peaks["bf16_sustained"] / 3.0
    tall = _traffic("gemm_split_umma2_kernel.tall_16384x4096x4096")
    achieved = k_flops / k_ms / 1e9 if k_ms else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "rows_per_gpu": rows,
                   "parallelism": f"dp{world}", "f32_mode": "f16x3: two fp16 planes per operand after exact power-of-two row/column "
                               "scaling, three tensor products per f32 product (3xTF32-class accuracy)",
                   "l2": "inputs larger than L2 (2.1 GB batch, 1 GB activations per layer)",
                   "flops_per_sample": mlp_flops_per_sample(DIMS),
                   "mean_loss_over_ranks_after_timed_steps": final_loss,
                   "timed_region": f"{len(blocks_ms)} blocks of {args.steps} steps, median block reported"},
        "blocks_ms": blocks_ms,
        "clocks": clocks,
        "ms_per_step_x_sm_mhz": (ms_per_step * clocks["sm_mhz"]) if clocks and clocks.get("sm_mhz") else None,
        "params_equal_across_ranks_after_timed_steps": replicas_equal,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4, "note": "next batch's host->device copy overlaps the current step",
                "h2d_gbs_per_rank_needed": h2d / (ms_per_step * 1e6),
                "h2d_gbs_per_rank_bare_copy_all_ranks_at_once": h2d_ceiling_gbs,
                "floor_ms_per_step_from_host_link": copy_ms,
                "host_cpus_bound_to_gpu_numa_node": host_numa},
        "gpu_launches": gpu_launches,
        "roofline": {
            "kernel": "gemm_split_umma2_kernel", "bound": "tensor", "achieved": achieved, "peak": peak_f32,
            "unit": "TFLOP/s", "frac": (achieved / peak_f32) if achieved else None,
            "peak_def": f"{peaks['source']} 16-bit dense tensor sustained {peaks['bf16_sustained']} TFLOP/s / 3 "
                        "(three fp16 tensor products per f32 product); a 3xTF32 emulation's roofline is half of this",
            "launches": k_launches, "avg_launch_ms": k_ms / k_launches if k_launches else None,
            "share_of_step": k_ms / ms_last if ms_last else None,
            # DRAM bytes per launch: the step's GEMMs hold 3-6 GB each, above the ncu capture size rule, so the
            # figure is the ncu capture of the same kernel on 16384x4096x4096 scaled by the flops of an average
            # launch of this step (traffic per flop is set by the tile shape and the walk order, which are the same)
            "traffic": (tall["dram_bytes_per_launch"] * (k_flops / max(k_launches, 1)) / tall["flops_per_launch"]) if tall else None,
            "traffic_note": "bytes per average launch of this step, scaled by flops from the recorded ncu capture of the "
                            "same kernel on 16384x4096x4096",
            "traffic_capture": tall,
            "split_kernels": {"launches": s_launches, "ms": s_ms, "gbs": s_bytes / s_ms / 1e6 if s_ms else None,
                              "share_of_step": s_ms / ms_last if ms_last else None},
        },
        "step_tflops": mlp_flops_per_sample(DIMS) * value / 1e12,
    }
    if dp is not None:
        line["dp_check"] = dp
    if world == 1:
        line["gemm_f32_4096"] = gemm4096(be, torch, peaks)
        if not args.no_configs:
            line["configs"] = config_table(be, torch, peaks, with_cpu=not args.no_cpu)
        if not args.no_cpu:
            rows_cpu = 2048
            v, per_step, cores = cpu_mlp_samples_per_s(rows_cpu, 1, 1)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"one reference-ordered training step on {rows_cpu} rows (of "
                                              f"{GLOBAL_BATCH}), {per_step:.2f} s"}
    sys.stdout.flush()
    os.dup2(saved_stdout, 1)
    print(json.dumps(line), flush=True)
    os.dup2(2, 1)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_case(args):
    """Runs one small, fixed workload a few times and prints nothing but a line of timings: the
    command ncu is pointed at for the per-kernel summaries under profiles/ (sizes above L2 where
    the kernel is memory-bound, a few GB at most)."""
    import torch
    from minitensor_b200.backend import get_backend
    be = get_backend(0)
    dev = be.device
    g = torch.Generator(device="cpu").manual_seed(7)
    rnd = lambda *shape, dtype=torch.float32: torch.randn(*shape, generator=g, dtype=dtype).to(dev)
    name = args.case
    if name == "gemm_f32_4096":
        a, b = rnd(4096, 4096), rnd(4096, 4096)
        out = torch.empty(4096, 4096, device=dev)
        fn = lambda: be.gemm(a, b, out=out)
    elif name == "gemm_f32_tall":       # a dense layer's shape at 1/4 of the large MLP's batch: 13.8 waves of tiles
        a, b = rnd(16384, 4096), rnd(4096, 4096)
        out = torch.empty(16384, 4096, device=dev)
        fn = lambda: be.gemm(a, b, trans_b=True, out=out)
    elif name == "dense_pair":          # dense layer forward + backward with shared operand preparation
        x, w, b, dy = rnd(16384, 4096), rnd(4096, 4096), rnd(4096), rnd(16384, 4096)
        saved = torch.empty(be.dense_saved_bytes(16384, 4096, 4096), dtype=torch.uint8, device=dev)
        y, dx = torch.empty(16384, 4096, device=dev), torch.empty(16384, 4096, device=dev)
        dw, db = torch.empty(4096, 4096, device=dev), torch.empty(4096, device=dev)
        fn = lambda: (be.dense_forward(x, w, b, 1, out=y, saved=saved),
                      be.dense_backward(x, w, dy, saved, dx=dx, dx_epilogue=4, dx_aux=x, dw=dw, db=db))
    elif name == "gemm_f32_mid":        # plain products at 512, 1024 and 2048: the launch-bound middle of the range
        mats = [(rnd(n, n), rnd(n, n), torch.empty(n, n, device=dev)) for n in (512, 1024, 2048)]
        fn = lambda: [be.gemm(a, b, out=o) for (a, b, o) in mats]
    elif name == "gemm_f32_nt_tn":      # the two products of MatMulBackward at 2048
        a, b, dy = rnd(2048, 2048), rnd(2048, 2048), rnd(2048, 2048)
        fn = lambda: (be.gemm(dy, b, trans_b=True), be.gemm(a, dy, trans_a=True))
    elif name == "gemm_f64_2048":
        a, b = rnd(2048, 2048, dtype=torch.float64), rnd(2048, 2048, dtype=torch.float64)
        fn = lambda: be.gemm(a, b)
    elif name == "gemm_i32_2048":
        a = torch.randint(-8, 9, (2048, 2048), generator=g, dtype=torch.int32).to(dev)
        b = torch.randint(-8, 9, (2048, 2048), generator=g, dtype=torch.int32).to(dev)
        fn = lambda: be.gemm(a, b)
    elif name == "colsum":              # bias gradient of a [65536, 4096] activation gradient (1.07 GB)
        x = rnd(65536, 4096)
        fn = lambda: be.colsum(x)
    elif name == "cross_entropy":       # [65536, 1000] logits (262 MB)
        x = rnd(65536, 1000)
        y = torch.randint(0, 1000, (65536,), generator=g).to(dev)
        fn = lambda: be.cross_entropy(x, y)
    elif name == "adam":                # 71.2 M parameters (the large MLP): 2.0 GB of traffic
        n = 71_218_152
        p, gr = rnd(n), rnd(n)
        m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        fn = lambda: be.adam_step(p, gr, m, v, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, step=1)
    elif name == "optimizers":          # SGD (momentum), RMSprop (centered, momentum), norm clipping on 71.2 M parameters
        n = 71_218_152
        p, gr = rnd(n), rnd(n)
        bufs = [torch.zeros(n, device=dev) for _ in range(4)]
        fn = lambda: (be.sgd_step(p, gr, bufs[0], lr=1e-3, momentum=0.9, weight_decay=1e-4),
                      be.rmsprop_step(p, gr, bufs[1], bufs[2], bufs[3], lr=1e-3, momentum=0.9),
                      be.clip_grad_norm([gr], 1.0))
    elif name == "batch_norm":          # [65536, 4096] f32 (1.07 GB): forward with batch statistics, then backward
        x, dy = rnd(65536, 4096), rnd(65536, 4096)
        w, b = rnd(4096), rnd(4096)
        rm, rv = torch.zeros(4096, device=dev), torch.ones(4096, device=dev)

        def fn():
            y, mean, inv, bs = be.batch_norm_fwd(x, w, b, rm, rv, training=True)
            be.batch_norm_bwd(x, dy, w, mean, inv, batch_stats=bs)
    elif name == "dropout":             # x * mask on [65536, 4096] f32, mask generated on the fly
        x = rnd(65536, 4096)
        fn = lambda: be.dropout_apply(x, 0.3, 42)
    elif name == "cross_entropy_soft":  # probability targets, per-sample losses: [65536, 1000]
        x = rnd(65536, 1000)
        t = torch.softmax(rnd(65536, 1000), dim=1)
        fn = lambda: be.cross_entropy_ex(x, t, reduction="none")
    elif name == "dense_small":         # the small MLP's layers: launch / HBM-bound shapes
        x, w1, b1 = rnd(32, 784), rnd(128, 784), rnd(128)
        w2, b2 = rnd(10, 128), rnd(10)
        fn = lambda: be.gemm(be.gemm(x, w1, trans_b=True, bias=b1, epilogue=1), w2, trans_b=True, bias=b2)
    elif name == "conv":                # the conv config at batch 32 (forward + the three gradients)
        x, w, b = rnd(32, 64, 56, 56), rnd(64, 64, 3, 3), rnd(64)
        dy = rnd(32, 64, 56, 56)
        fn = lambda: (be.conv2d_fwd(x, w, b, (1, 1), (1, 1)), be.conv2d_bwd_data(dy, w, x.shape, (1, 1), (1, 1)),
                      be.conv2d_bwd_weight(dy, x, w.shape, (1, 1), (1, 1)), be.conv2d_bwd_bias(dy))
    else:
        print(json.dumps({"error": f"unknown case {name}"}))
        return 2
    times = []
    for _ in range(args.reps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    be.sync()
    print(json.dumps({"case": name, "ms": times}), flush=True)
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU-baseline leg")
    ap.add_argument("--no-configs", action="store_true", help="skip the per-configuration table of the N = 1 line")
    ap.add_argument("--per-product", action="store_true",
                    help="one GEMM call per product (as the reference's autograd issues them) instead of the dense-layer pair")
    ap.add_argument("--min-region-s", type=float, default=2.0,
                    help="repeat the block of --steps timed steps until the timed region has run this long")
    ap.add_argument("--max-blocks", type=int, default=40)
    ap.add_argument("--case", default=None, help="run one small fixed workload (profiling target) and exit")
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--record-traffic", default=None, metavar="NCU_CSV",
                    help="fold an ncu CSV's DRAM byte counters into profiles/dram_traffic.json and exit")
    ap.add_argument("--traffic-key", default=None)
    ap.add_argument("--traffic-kernel", default=".", help="regular expression the kernel name must match")
    ap.add_argument("--traffic-command", default="", help="the ncu command line that made the CSV")
    args = ap.parse_args()
    if args.record_traffic:
        if not args.traffic_key:
            ap.error("--record-traffic needs --traffic-key")
        record_traffic(args.record_traffic, args.traffic_key, args.traffic_kernel, args.traffic_command)
        return 0
    if args.case:
        return run_case(args)
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
