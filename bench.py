#!/usr/bin/env python
"""Benchmark of the operator hot path on B200.

    python bench.py --gpus N --steps K --warmup W            # this backend
    python bench.py --impl reference --gpus N --steps K ...   # the reference's CPU kernels

A "step" is one pass of the hot path over one batch of synthetic input. The headline workload
is benchmark configuration 2: Z = log(X) + Y*Y - exp(X) on float16 X[8192,8192] (uniform[0.1,4]) and
Y[1,8192] (uniform[-2,2], row-broadcast), seed 1, evaluated by ONE fused kernel that streams HBM
once. With N GPUs every rank owns its own [8192,8192] row shard of a [8192*N, 8192] problem (weak
scaling, no collective on the data path; Y is replicated). The metric is algorithmic HBM bytes
(read X + read Y + write Z) per second, summed over ranks, timed with CUDA events and taken as the
max over ranks.

The same JSON line carries, under "workloads", device-timed figures for the other benchmark
configurations (int32 broadcast add, the Llama-3-8B MLP GEMM, the ResNet-50 convolutions, the ViT score
path) on rank 0's GPU.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

ROWS, COLS = 8192, 8192
ALGO_BYTES = 2 * ROWS * COLS * 2 + COLS * 2  # read X + write Z + read Y = 268,451,840
METRIC = "fused broadcast elementwise HBM GB/s (Z = log(X) + Y*Y - exp(X), float16)"
WORKLOAD = "config 2: float16 X[8192,8192] U[0.1,4], Y[1,8192] U[-2,2] row-broadcast, seed 1, per GPU"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            p = json.loads(path.read_text())
            return float(p["hbm_gbs"]), float(p.get("bf16_tflops", FALLBACK_BF16_TFLOPS)), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CPU kernels (oracle/_ref) or the C port
def cpu_expression(rows: int, threads: int):
    """Evaluates the config-2 expression on `rows` rows with the reference's CPU kernels, the rows
    split over `threads` host threads (the reference itself is single-threaded; its kernels are
    pure functions, so independent row blocks can run side by side). Returns (seconds, kind)."""
    import torch
    import oracle
    kind = "reference" if oracle.ref() is not None else "port"
    impl = "ref" if kind == "reference" else "port"
    x = oracle.fill((rows, COLS), torch.float16, 1, "uniform", 0.1, 4.0)
    y = oracle.fill((1, COLS), torch.float16, 2, "uniform", -2.0, 2.0)
    blocks = [x[i::threads] if False else x[(rows * i) // threads:(rows * (i + 1)) // threads] for i in range(threads)]

    def run(block):
        if block.shape[0] == 0:
            return None
        t0 = oracle.unary("log", block, impl=impl)
        t1 = oracle.binary("mul", y, y, impl=impl)
        t2 = oracle.binary("add", t0, t1, impl=impl)
        t3 = oracle.unary("exp", block, impl=impl)
        return oracle.binary("sub", t2, t3, impl=impl)

    start = time.perf_counter()
    if threads == 1:
        run(blocks[0])
    else:
        with ThreadPoolExecutor(max_workers=threads) as pool:
            list(pool.map(run, blocks))
    return time.perf_counter() - start, kind


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = max(1, min(os.cpu_count() or 1, 64))
    rows = min(ROWS, 64 * threads)
    sample_bytes = 2 * rows * COLS * 2 + COLS * 2
    for _ in range(max(0, args.warmup)):
        cpu_expression(rows, threads)
    total = 0.0
    kind = "port"
    for _ in range(args.steps):
        dt, kind = cpu_expression(rows, threads)
        total += dt
    ms = 1e3 * total / args.steps
    value = sample_bytes / (total / args.steps) / 1e9
    sample = f"{rows} of {ROWS} rows per step, five node kernels, {threads} host threads over independent row blocks"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic", "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------------------
def time_device(fn, steps, warmup, torch):
    """Average milliseconds per call of `fn` on the current stream (CUDA events)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def secondary_workloads(torch, tb, A, hbm_peak, tf_peak, only=None, small=False):
    """Device-timed figures for the other benchmark configurations (rank 0 only). Inputs are seeded
    synthetic tensors of the named shapes and distributions, created on the device. `only` runs a
    single workload (used for profiling); `small` shrinks the leading dimension so that a
    profiler capture stays short (inputs still exceed L2 where the workload is HBM-bound)."""
    out = {}
    g = torch.Generator(device="cuda")
    iters, warm = (2, 1) if small else (10, 3)

    def record(name, ms, bytes_=None, flops=None, bound="hbm", note=None):
        e = {"ms": ms, "bound": bound}
        if bytes_ is not None:
            e["GB/s"] = bytes_ / ms / 1e6
        if flops is not None:
            e["TFLOP/s"] = flops / ms / 1e9
        if bound == "hbm" and bytes_ is not None:
            e["frac_of_peak"] = e["GB/s"] / hbm_peak
        if bound == "tensor" and flops is not None:
            e["frac_of_peak"] = e["TFLOP/s"] / tf_peak
        if note:
            e["note"] = note
        out[name] = e

    def config2b():
        g.manual_seed(1)
        a = torch.randint(-1000, 1001, (8192, 8192), dtype=torch.int32, device="cuda", generator=g)
        b = torch.randint(-1000, 1001, (8192, 1), dtype=torch.int32, device="cuda", generator=g)
        ms = time_device(lambda: tb.add(a, b), iters, warm, torch)
        record("config2b_int32_add_colbroadcast", ms, bytes_=2 * 8192 * 8192 * 4 + 8192 * 4)

    def config2c():
        # the same expression as the headline with its nodes listed in another order, so that it
        # misses the compiled programs and runs through the in-kernel interpreter
        g.manual_seed(1)
        x = (torch.rand((8192, 8192), device="cuda", generator=g) * 3.9 + 0.1).to(torch.float16)
        y = (torch.rand((1, 8192), device="cuda", generator=g) * 4.0 - 2.0).to(torch.float16)
        z = torch.empty_like(x)
        nodes = [(A.OP_EXP, 0, 0), (A.OP_LOG, 0, 0), (A.OP_MUL, 1, 1), (A.OP_ADD, 5, 6), (A.OP_SUB, 7, 4)]
        ms = time_device(lambda: tb.program([x, y], nodes, out=z), iters, warm, torch)
        record("config2c_interpreted_expression_fp16", ms, bytes_=2 * 8192 * 8192 * 2 + 8192 * 2, note="log(X)+Y*Y-exp(X), nodes reordered")

    def config1():
        # the reference's own CPU-runnable case, on the device for information
        g.manual_seed(0)
        a = torch.rand((512, 1024), device="cuda", generator=g) * 2 - 1
        b = torch.rand((1024, 512), device="cuda", generator=g) * 2 - 1
        ms = time_device(lambda: tb.matmul(a, b), iters, warm, torch)
        record("config1_matmul_f32_512x1024x512", ms, flops=2 * 512 * 512 * 1024, bound="fp32", note="float32 as three bfloat16 parts on the tensor cores, float32 accumulate")

    def config3():
        batch = 2 if small else 8
        g.manual_seed(2)
        x = torch.randn((batch, 2048, 4096), device="cuda", generator=g).to(torch.bfloat16)
        w = (torch.randn((14336, 4096), device="cuda", generator=g) * 0.02).to(torch.bfloat16)
        ms = time_device(lambda: tb.matmul(x, w.transpose(-1, -2)), iters, warm, torch)
        record("config3_llama_mlp_gemm_bf16", ms, flops=2 * batch * 2048 * 14336 * 4096, bound="tensor",
               note=f"X[{batch},2048,4096] . W[14336,4096]^T")

    def config5():
        batch = 64 if small else 256
        g.manual_seed(4)
        q = torch.randn((batch, 12, 197, 64), device="cuda", generator=g).to(torch.bfloat16)
        k = torch.randn((batch, 12, 197, 64), device="cuda", generator=g).to(torch.bfloat16)
        ms = time_device(lambda: tb.matmul(q, k.transpose(-1, -2), scale_by=0.125), iters, warm, torch)
        s_bytes = batch * 12 * 197 * 197 * 2
        record("config5_vit_scores_gemm_scaled_bf16", ms, bytes_=2 * q.numel() * 2 + s_bytes, flops=2 * batch * 12 * 197 * 197 * 64,
               note=f"Q,K[{batch},12,197,64]")
        s = tb.matmul(q, k.transpose(-1, -2), scale_by=0.125)
        ms = time_device(lambda: tb.reduce_stats(s, -1), iters, warm, torch)
        record("config5_row_max_sum_argmax_bf16", ms, bytes_=s_bytes + batch * 12 * 197 * (8 + 2 + 2))

    def config4():
        n = 16 if small else 128
        g.manual_seed(3)
        xin = torch.randn((n, 256, 56, 56), device="cuda", generator=g).to(torch.float16)
        w1 = (torch.randn((1024, 256, 1, 1), device="cuda", generator=g) * (2.0 / 256) ** 0.5).to(torch.float16)
        ms = time_device(lambda: tb.convolve2D(xin, w1, 1, 0), max(2, iters // 2), max(1, warm - 1), torch)
        record("config4b_conv1x1_fp16", ms, bytes_=xin.numel() * 2 + w1.numel() * 2 + n * 1024 * 3136 * 2,
               flops=2 * n * 1024 * 3136 * 256, note=f"x[{n},256,56,56]")
        del w1
        w3 = (torch.randn((256, 256, 3, 3), device="cuda", generator=g) * (2.0 / 2304) ** 0.5).to(torch.float16)
        ms = time_device(lambda: tb.convolve2D(xin, w3, 1, 1), max(2, iters // 2), max(1, warm - 1), torch)
        record("config4a_conv3x3_fp16", ms, flops=2 * n * 256 * 3136 * 256 * 9, bound="tensor", note=f"x[{n},256,56,56]")

    table = {"config1": config1, "config2b": config2b, "config2c": config2c, "config3": config3, "config5": config5, "config4": config4}
    for name, fn in table.items():
        if only is not None and only != name:
            continue
        try:
            fn()
        except Exception as exc:  # a failing secondary workload must not hide the headline number
            out[name + "_error"] = f"{type(exc).__name__}: {exc}"
        torch.cuda.empty_cache()
    return out


def ours(args):
    import torch
    import torch.distributed as dist
    from tannic_b200 import _abi as A
    from tannic_b200 import ops as tb
    from tannic_b200 import shard

    A.lib()  # raises if the CUDA extension is missing: there is no fallback
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local)
    if world > 1:
        # stdout carries the one JSON line and nothing else: NCCL's own messages (its version banner
        # under NCCL_DEBUG=VERSION, for one) go to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        if os.environ.get("NCCL_DEBUG", "").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"  # the banner is written to stdout whatever the debug file is
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    hbm_peak, tf_peak, peak_kind = peaks()
    if args.only:
        # a single secondary workload, for profiling (one GPU; prints its own JSON line)
        if rank == 0:
            print(json.dumps({"workloads": secondary_workloads(torch, tb, A, hbm_peak, tf_peak, only=args.only, small=args.small),
                              "device_errors": tb.device_errors()}), flush=True)
        return 0

    import oracle  # input generator only (seeded, shared with the tests)
    x_host = oracle.fill((ROWS, COLS), torch.float16, 1 + 7919 * rank, "uniform", 0.1, 4.0).pin_memory()
    y_host = oracle.fill((1, COLS), torch.float16, 2, "uniform", -2.0, 2.0).pin_memory()
    z_host = torch.empty((ROWS, COLS), dtype=torch.float16).pin_memory()
    x, y = x_host.cuda(non_blocking=True), y_host.cuda(non_blocking=True)
    z = torch.empty_like(x)
    nodes = [(A.OP_LOG, 0, 0), (A.OP_MUL, 1, 1), (A.OP_ADD, 4, 5), (A.OP_EXP, 0, 0), (A.OP_SUB, 6, 7)]

    # the step: one fused kernel through the C ABI, writing into a preallocated result
    dx, dy, dz = tb.desc(x), tb.desc(y), tb.desc(z)
    ptrs = (C.POINTER(A.TensorT) * 2)(C.pointer(dx), C.pointer(dy))
    arr = (A.EltwiseNode * len(nodes))()
    for i, nd in enumerate(nodes):
        arr[i].opcode, arr[i].lhs, arr[i].rhs, arr[i].imm = nd[0], nd[1], nd[2], 0.0
    stream = tb.current_stream(x)
    lib = A.lib()

    def step():
        A.check(lib.tn_eltwise_program(ptrs, 2, arr, len(nodes), C.byref(dz), stream))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    time.sleep(0.15)
    launches0 = tb.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    elapsed_ms = start.elapsed_time(stop)
    launches = tb.launch_count() - launches0
    # keep the load up long enough for the sampler to see clocks under load
    t_end = time.time() + 0.6
    while time.time() < t_end:
        step()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    elapsed_ms = shard.max_over_ranks(elapsed_ms, device="cuda")
    ms_per_step = elapsed_ms / args.steps
    value = world * ALGO_BYTES / ms_per_step / 1e6

    # ---- end to end: host buffers in, host buffer out, through the same entry point
    d = A.DeviceT(local)

    # the public host-to-host call: rows in chunks, copy-in / kernel / copy-out overlapped on three
    # streams; every step copies all of X and Y in and all of Z out
    pipe = tb.HostPipeline(device=local, chunks=int(os.environ.get("TN_E2E_CHUNKS", "8")))

    def e2e_step():
        pipe.program([x_host, y_host], nodes, z_host)
        torch.cuda.current_stream().synchronize()

    for _ in range(2):
        e2e_step()
    barrier()
    t0 = time.perf_counter()
    e2e_steps = max(3, min(args.steps, 10))
    for _ in range(e2e_steps):
        e2e_step()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    e2e_s = shard.max_over_ranks(e2e_s, device="cuda")
    e2e_value = world * ALGO_BYTES / e2e_s / 1e9

    # parity spot-check of what was just timed: the first rows of Z against the oracle's node chain
    xs, zs = x_host[:4], z_host[:4]
    want = oracle.binary("sub", oracle.binary("add", oracle.unary("log", xs), oracle.binary("mul", y_host, y_host)), oracle.unary("exp", xs))
    parity_ok = bool(((zs.double() - want.double()).abs() <= 1e-2 + 1e-2 * want.double().abs()).all())
    errors = tb.device_errors()

    if rank == 0:
        achieved = ALGO_BYTES / ms_per_step / 1e6
        line = {
            "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": WORKLOAD, "kernel": "ew_program_rows<half, log+square+exp>", "l2": "inputs larger than L2: 256 MiB touched per step vs 126 MB L2",
                       "parallelism": f"rows sharded over {world} GPU(s), Y replicated, no collective"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH, "peak_kind": peak_kind},
            "e2e": {"value": e2e_value, "unit": "GB/s", "h2d_bytes_per_step": ROWS * COLS * 2 + COLS * 2, "d2h_bytes_per_step": ROWS * COLS * 2},
            "gpu_launches": launches, "clocks": clocks, "device_errors": errors, "parity_spot_check": parity_ok,
        }
        if world == 1 and not args.no_cpu_baseline:
            rows = 1024
            dt, kind = cpu_expression(rows, 1)
            line["cpu_baseline"] = {"value": (2 * rows * COLS * 2 + COLS * 2) / dt / 1e9, "unit": "GB/s", "cores": 1, "kind": kind,
                                    "sample": f"{rows} of {ROWS} rows, five node kernels of the reference CPU path, 1 thread (the reference has no threading)"}
        if not args.headline_only:
            line["workloads"] = secondary_workloads(torch, tb, A, hbm_peak, tf_peak)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


# DRAM bytes read + written by one launch of the headline kernel, from the ncu capture summarised in
# profiles/ew_program_rows_config2_fp16.md (dram__bytes_read.sum 134.25 MB + dram__bytes_write.sum
# 85.51 MB; the write side is below the 134.2 MB of Z because L2 still holds its tail at kernel end).
TRAFFIC_BYTES_PER_LAUNCH = 219_758_080


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--headline-only", action="store_true", help="skip the secondary workloads")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--only", default=None, choices=["config1", "config2b", "config2c", "config3", "config4", "config5"],
                    help="run one secondary workload alone (profiling aid)")
    ap.add_argument("--small", action="store_true", help="with --only: shrink the leading dimension for a short profiler capture")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    return ours(args)


if __name__ == "__main__":
    sys.exit(main())
