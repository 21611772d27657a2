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
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i",
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
            "dram_traffic_mb_per_launch": 361.9, "algorithmic_mb_per_launch": 201.3}


def run_ours(args):
    import torch
    import torch.distributed as dist
    from minitensor_b200.mlp import MLPTrainer, mlp_flops_per_sample, shard_rows

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(json.dumps({"error": f"--gpus {args.gpus} needs torchrun with {args.gpus} processes"}))
            return 2
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # keep NCCL's version banner off stdout: one JSON line only
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    peaks = _peaks()
    lo, hi = shard_rows(GLOBAL_BATCH, world, rank)
    rows = hi - lo
    trainer = MLPTrainer(DIMS, rows, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, device=local, world_size=world, seed=0,
                         fused_dense=not args.per_product)
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
    be.profile(True)
    launches0 = be.launches
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    loss = None
    for _ in range(args.steps):
        loss = trainer.step(x, y)
    e.record()
    barrier()
    sampler.mark_end()
    ms_total = max_over_ranks(s.elapsed_time(e))
    clocks = sampler.stop() if rank == 0 else None
    gpu_launches = be.launches - launches0
    k_launches, k_ms, k_flops = be.profile_read(0)
    s_launches, s_ms, s_bytes = be.profile_read(1)
    be.profile(False)
    be.sync()
    final_loss = float(loss.item())
    ms_per_step = ms_total / args.steps
    value = GLOBAL_BATCH / (ms_per_step * 1e-3)

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

    if rank != 0:
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return 0

    peak_f32 = peaks["bf16_sustained"] / 3.0
    achieved = k_flops / k_ms / 1e9 if k_ms else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": GLOBAL_BATCH, "rows_per_gpu": rows,
                   "parallelism": f"dp{world}", "f32_mode": "f16x3: two fp16 planes per operand after exact power-of-two row/column "
                               "scaling, three tensor products per f32 product (3xTF32-class accuracy)",
                   "l2": "inputs larger than L2 (2.1 GB batch, 1 GB activations per layer)",
                   "flops_per_sample": mlp_flops_per_sample(DIMS), "final_loss": final_loss},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4, "note": "next batch's host->device copy overlaps the current step"},
        "gpu_launches": gpu_launches,
        "roofline": {
            "kernel": "gemm_split_umma2_kernel", "bound": "tensor", "achieved": achieved, "peak": peak_f32,
            "unit": "TFLOP/s", "frac": (achieved / peak_f32) if achieved else None,
            "peak_def": f"{peaks['source']} 16-bit dense tensor sustained {peaks['bf16_sustained']} TFLOP/s / 3 "
                        "(three fp16 tensor products per f32 product); a 3xTF32 emulation's roofline is half of this",
            "launches": k_launches, "avg_launch_ms": k_ms / k_launches if k_launches else None,
            "share_of_step": k_ms / ms_total if ms_total else None,
            # DRAM bytes per launch: the step's GEMMs hold 3-6 GB each, above the ncu capture size rule, so the
            # figure is the ncu capture of the same kernel on 16384x4096x4096 (1.511 GB read + written for
            # 549.8 GFLOP) scaled by the flops of an average launch of this step (traffic per flop is set by the
            # tile shape and the walk order, which are the same)
            "traffic": (1.511e9 * (mlp_flops_per_sample(DIMS) * rows / 11) / 549.8e9),
            "traffic_note": "bytes per average launch, scaled by flops from the ncu capture of the same kernel on "
                            "16384x4096x4096 (profiles/gemm_split_umma2_f32_4096.md)",
            "split_kernels": {"launches": s_launches, "ms": s_ms, "gbs": s_bytes / s_ms / 1e6 if s_ms else None,
                              "share_of_step": s_ms / ms_total if ms_total else None},
        },
        "step_tflops": mlp_flops_per_sample(DIMS) * value / 1e12,
    }
    if world == 1:
        line["gemm_f32_4096"] = gemm4096(be, torch, peaks)
        if not args.no_cpu:
            rows_cpu = 2048
            v, per_step, cores = cpu_mlp_samples_per_s(rows_cpu, 1, 1)
            line["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cores, "kind": "port",
                                    "sample": f"one reference-ordered training step on {rows_cpu} rows (of "
                                              f"{GLOBAL_BATCH}), {per_step:.2f} s"}
    print(json.dumps(line), flush=True)
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
    ap.add_argument("--per-product", action="store_true",
                    help="one GEMM call per product (as the reference's autograd issues them) instead of the dense-layer pair")
    ap.add_argument("--case", default=None, help="run one small fixed workload (profiling target) and exit")
    ap.add_argument("--reps", type=int, default=3)
    args = ap.parse_args()
    if args.case:
        return run_case(args)
    if args.impl == "reference":
        return run_reference(args)
    args.warmup = max(args.warmup, 3)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
