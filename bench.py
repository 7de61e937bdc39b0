"""Benchmark of the matmul hot path: f32 8192 x 8192 x 8192 (the configuration the
headline metric is quoted on), one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

One "step" is one pass of the product over one set of synthetic operands
(N(0, 1/sqrt(8192)) entries, seed 3).  At N > 1 the product is split into output-column
blocks, one per rank, and C is all-gathered (strong scaling: the total work is fixed).
Prints ONE JSON line on rank 0.  Inputs (768 MiB with C) are far larger than L2, so no
explicit L2 flush is needed between timed iterations.

--impl reference times the reference's own CPU matmul kernel (oracle/_ref, compiled from
the reference's sources) on the host cores, on a bounded sample of the same product.
"""
from __future__ import annotations

import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

DIM = 8192
SEED = 3
METRIC = "f32 matmul TFLOP/s"
UNIT = "TFLOP/s"
WORKLOAD = "C4: single 2D f32 GEMM 8192x8192x8192, N(0,1/sqrt(8192)) entries, seed 3"
FLOPS_PER_STEP = 2.0 * DIM * DIM * DIM          # algorithmic: one multiply-add per (i, j, k)
BYTES_PER_STEP = 3.0 * DIM * DIM * 4            # A and B read once, C written once
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the pair kernel on this very
# workload, from one ncu capture (profiles/gemm_f32_3xtf32_pair_8192cubed.md): 2.457 GB + 0.264 GB.
DRAM_TRAFFIC_PER_FULL_LAUNCH = 2.457e9 + 0.264e9


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clock, power and clock-event (throttle) reasons through NVML in a thread
    while the timed region runs.  Only reads; changes no setting."""

    REASONS = {
        "hw_slowdown": 0x8,            # nvmlClocksEventReasonHwSlowdown
        "sw_thermal_slowdown": 0x20,   # nvmlClocksEventReasonSwThermalSlowdown
        "hw_thermal_slowdown": 0x40,   # nvmlClocksThrottleReasonHwThermalSlowdown
        "sw_power_cap": 0x4,           # nvmlClocksEventReasonSwPowerCap
    }

    def __init__(self, torch_device_index: int):
        self.samples = []
        self.stop_flag = threading.Event()
        self.thread = None
        self.handle = None
        self.nvml = None
        try:
            import pynvml
            import torch

            pynvml.nvmlInit()
            self.nvml = pynvml
            try:
                uuid = str(torch.cuda.get_device_properties(torch_device_index).uuid)
                if not uuid.startswith("GPU-"):
                    uuid = "GPU-" + uuid
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(torch_device_index)
        except Exception:
            self.nvml = None

    def _loop(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                power = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                try:
                    reasons = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:
                    reasons = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                self.samples.append((time.perf_counter(), sm, power, reasons))
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.nvml is None:
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self, t_begin=None, t_end=None):
        if self.nvml is None or self.thread is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["NVML unavailable"]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        n = self.nvml
        try:
            sm_max = float(n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM))
        except Exception:
            sm_max = None
        sel = [x for x in self.samples if (t_begin is None or x[0] >= t_begin) and (t_end is None or x[0] <= t_end)]
        if not sel:
            sel = self.samples
        if not sel:
            return {"sm_mhz": None, "sm_max_mhz": sm_max, "reasons": ["no samples"]}
        bits = 0
        for x in sel:
            bits |= int(x[3])
        reasons = sorted(name for name, mask in self.REASONS.items() if bits & mask)
        return {"sm_mhz": float(np.median([x[1] for x in sel])), "sm_max_mhz": sm_max,
                "power_w_max": float(max(x[2] for x in sel)), "samples": len(sel), "reasons": reasons}


# --------------------------------------------------------------------------- reference arm
def load_reference():
    """The reference's CPU matmul kernel compiled from its own sources (oracle/_ref), or the
    C port of it when that library is not in the tree."""
    ref = ROOT / "oracle" / "_ref" / "libttref.so"
    if ref.exists():
        return ctypes.CDLL(str(ref)), "reference"
    port = ROOT / "oracle" / "liboracle.so"
    if not port.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), str(port)], check=True, capture_output=True)
    return ctypes.CDLL(str(port)), "port"


def cpu_sample_seconds(lib, kind, a_rows: np.ndarray, b: np.ndarray) -> float:
    """Times lhs[rows, K] . rhs[K, M] on one host core with the reference kernel."""
    rows, K = a_rows.shape
    M = b.shape[1]
    out = np.empty((rows, M), dtype=np.float32)
    t0 = time.perf_counter()
    if kind == "reference":
        lib.ref_matmul_f32(ctypes.c_void_p(a_rows.ctypes.data), ctypes.c_void_p(b.ctypes.data),
                           ctypes.c_void_p(out.ctypes.data), ctypes.c_int64(1), ctypes.c_int(rows), ctypes.c_int(K),
                           ctypes.c_int(M))
    else:
        scratch = np.empty(M, dtype=np.float32)
        lib.oracle_matmul_fast_f32(ctypes.c_void_p(a_rows.ctypes.data), ctypes.c_void_p(b.ctypes.data),
                                   ctypes.c_void_p(out.ctypes.data), ctypes.c_int64(1), ctypes.c_int64(rows),
                                   ctypes.c_int64(K), ctypes.c_int64(M), ctypes.c_void_p(scratch.ctypes.data))
    return time.perf_counter() - t0


def host_operands(rows: int):
    rng = np.random.default_rng(SEED)
    std = DIM ** -0.5
    a = (rng.standard_normal((rows, DIM), dtype=np.float32) * np.float32(std))
    b = (rng.standard_normal((DIM, DIM), dtype=np.float32) * np.float32(std))
    return a, b


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # under torchrun only rank 0 measures the CPU arm
    lib, kind = load_reference()
    rows = 256  # per step: 256 of the 8192 rows of lhs = 1/32 of the product, about 1 s of CPU
    a, b = host_operands(rows)
    for _ in range(args.warmup):
        cpu_sample_seconds(lib, kind, a, b)
    t = 0.0
    for _ in range(args.steps):
        t += cpu_sample_seconds(lib, kind, a, b)
    flops = 2.0 * rows * DIM * DIM * args.steps
    value = flops / t / 1e12
    sample = f"{rows} of {DIM} lhs rows per step (1/{DIM // rows} of the product), single thread"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps * (DIM / rows),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "timed": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": kind, "sample": sample,
                         "host_cores_available": os.cpu_count()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- our arm
def run_ours(args):
    import torch
    import torch.distributed as dist

    import tinytensor_b200 as ttb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs CUDA devices; there is no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ttb.lib()  # fail loudly if the extension is missing

    # Operands: every rank holds the full A and B (placing them is set-up, not timed).
    g = torch.Generator(device=dev).manual_seed(SEED)
    std = DIM ** -0.5
    A = torch.randn((1, DIM, DIM), generator=g, device=dev) * std
    B = torch.randn((1, DIM, DIM), generator=g, device=dev) * std
    fused = args.exchange in ("fused", "fused-peer", "fused-multicast")
    sharded = ttb.ShardedMatmul(exchange={"fused": "peer", "fused-peer": "peer", "fused-multicast": "multicast"}.get(
        args.exchange, "auto")) if world > 1 else None
    if world > 1 and fused:
        # C in symmetric memory: the GEMM kernel itself stores each finished tile into every
        # rank's C over NVLink (fused all-gather); "nccl" keeps C private and all-gathers after.
        C = sharded.symmetric_output((1, DIM, DIM), torch.float32, dev)
    else:
        C = torch.empty((1, DIM, DIM), device=dev)
    part = ttb.partition(1, DIM, DIM, DIM, world, rank)
    exchange_desc = "NCCL all_gather + re-layout"
    if world > 1 and fused:
        multicast = sharded.exchange != "peer" and getattr(sharded._symm[1], "has_multicast_support", False)
        exchange_desc = ("fused into the GEMM kernel: each tile stored once through NVSwitch multicast (multimem.st)"
                         if multicast else
                         "fused into the GEMM kernel: bulk tensor stores from the epilogue to every peer over NVLink")

    def step():
        if sharded is None:
            ttb.batched_matmul(A, B, out=C)
        else:
            sharded(A, B, out=C)

    def kernel_only():
        # the rank's own share of the product, no exchange
        ttb.batched_matmul(A, B[:, :, part.begin:part.end], out=C[:, :, part.begin:part.end])

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = ttb.launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t_begin = time.perf_counter()
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    t_end = time.perf_counter()
    elapsed_ms = start.elapsed_time(stop)
    launches = ttb.launch_count() - launches0
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None

    # kernel-only timing for the roofline (same stream, events around the launches)
    for _ in range(2):
        kernel_only()
    barrier()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(args.steps):
        kernel_only()
    k1.record()
    barrier()
    kernel_ms = k0.elapsed_time(k1) / args.steps
    variant = ttb.last_variant().name
    ttb.check_device(local_rank)

    # end to end through the host-buffer C ABI call: pinned host operands in, result out
    e2e_steps = max(1, min(args.steps, 5))
    cols = part.end - part.begin
    hA = torch.empty((1, DIM, DIM), dtype=torch.float32, pin_memory=True)
    hB = torch.empty((1, DIM, max(cols, 1)), dtype=torch.float32, pin_memory=True)
    hC = torch.empty((1, DIM, max(cols, 1)), dtype=torch.float32, pin_memory=True)
    hA.copy_(A)
    hB.copy_(B[:, :, part.begin:part.end] if cols else B[:, :, :1])
    nA, nB, nC = hA.numpy(), hB.numpy(), hC.numpy()
    ttb.batched_matmul_host(nA, nB, out=nC, device=local_rank)  # warm-up: grows the staging buffers
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        ttb.batched_matmul_host(nA, nB, out=nC, device=local_rank)
    barrier()
    e2e_s = time.perf_counter() - t0
    h2d = nA.nbytes + nB.nbytes
    d2h = nC.nbytes

    if world > 1:
        t = torch.tensor([elapsed_ms, kernel_ms, e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms, kernel_ms, e2e_s = (float(x) for x in t.cpu())
        byt = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
        dist.all_reduce(byt, op=dist.ReduceOp.SUM)
        h2d, d2h = (int(x) for x in byt.cpu())

    if rank == 0:
        peaks, peak_kind = measured_peaks()
        ms_per_step = elapsed_ms / args.steps
        value = FLOPS_PER_STEP / (ms_per_step * 1e-3) / 1e12
        # Tensor-pipe roofline of the dominant kernel: this GPU's share of the algorithmic flops
        # over the kernel's own duration.  fp32 accuracy costs, per algorithmic multiply-add, one
        # TF32 multiply-add (the cost of two bf16 ones: dense TF32 runs at half the bf16 rate) and
        # two bf16 multiply-adds, i.e. four bf16 multiply-add times: the ceiling is bf16 / 4.
        # The classic 3xTF32 scheme would cost six (bf16 / 2 / 3); that figure is reported too.
        share = (part.end - part.begin) / DIM
        achieved = FLOPS_PER_STEP * share / (kernel_ms * 1e-3) / 1e12
        bf16 = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        peak = bf16 / 4.0
        # CPU baseline: the reference's CPU kernel on a bounded sample, one host core
        lib, kind = load_reference()
        rows = 2048
        a_rows, b_host = host_operands(rows)
        cpu_s = cpu_sample_seconds(lib, kind, a_rows, b_host)
        cpu_value = 2.0 * rows * DIM * DIM / cpu_s / 1e12
        # The kernel this library replaces, as a second reported baseline (N = 1 only): the
        # reference's own CUDA matmul kernel compiled from its sources (oracle/_ref), run on
        # this GPU on the same operands through the launch configuration of its runner.
        existing = None
        ref_cuda_path = ROOT / "oracle" / "_ref" / "libttref_cuda.so"
        if world == 1 and ref_cuda_path.exists():
            rc_lib = ctypes.CDLL(str(ref_cuda_path))
            rc_lib.ref_cuda_matmul_f32.restype = ctypes.c_int
            Cref = torch.empty((1, DIM, DIM), device=dev)

            def ref_kernel():
                rc = rc_lib.ref_cuda_matmul_f32(
                    ctypes.c_void_p(A.data_ptr()), ctypes.c_void_p(B.data_ptr()), ctypes.c_void_p(Cref.data_ptr()),
                    ctypes.c_int(1), ctypes.c_int(DIM), ctypes.c_int(DIM), ctypes.c_int(DIM),
                    ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
                if rc != 0:
                    raise RuntimeError(f"reference CUDA kernel launch failed: cudaError {rc}")

            ref_kernel()
            torch.cuda.synchronize()
            r0, r1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            r0.record()
            for _ in range(2):
                ref_kernel()
            r1.record()
            torch.cuda.synchronize()
            ref_ms = r0.elapsed_time(r1) / 2
            diff = float((Cref[0, :64] - C[0, :64]).abs().max() / C[0, :64].abs().max())
            existing = {"value": FLOPS_PER_STEP / (ref_ms * 1e-3) / 1e12, "unit": UNIT, "ms": ref_ms,
                        "kind": "reference",
                        "what": "tinytensor's matmul_kernel<float> (backend/cuda/kernel/matmul.cuh) compiled for sm_100a",
                        "max_diff_vs_ours_rel_to_max": diff}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "parallelism": (f"column blocks x{world} + all-gather of C "
                                       f"({exchange_desc})")
                       if world > 1 else "single GPU",
                       "l2": "operands (768 MiB with C) exceed the 126 MB L2; no explicit flush",
                       "kernel": variant, "arithmetic": ("split precision on tcgen05: TF32 product of the high parts + two bf16 "
                                      "correction products, fp32 accumulate in TMEM chunks, fp32 register sums")},
            "clocks": clocks,
            "e2e": {"value": FLOPS_PER_STEP / (e2e_s / e2e_steps) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "api": "ttb_batched_matmul_host (pinned host buffers, copies inside the timed region)"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                         "traffic": DRAM_TRAFFIC_PER_FULL_LAUNCH * share, "kernel_ms": kernel_ms,
                         "peak_source": f"{peak_kind}: bf16 sustained {bf16} TFLOP/s / 4 (one TF32 + two bf16 products per flop)",
                         "tf32_derived_peak_3x": bf16 / 2.0 / 3.0, "frac_of_tf32_derived_peak_3x": achieved / (bf16 / 6.0), "hbm_gbs_algorithmic": BYTES_PER_STEP * share / (kernel_ms * 1e-3) / 1e9},
            "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": 1, "kind": kind,
                             "sample": f"first {rows} of {DIM} lhs rows (1/{DIM // rows} of the product), {cpu_s:.1f} s",
                             "host_cores_available": os.cpu_count()},
            "existing_gpu_kernel": existing,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--exchange", default="fused", choices=["fused", "fused-peer", "fused-multicast", "nccl"],
                    help="N > 1: how C is all-gathered (fused into the GEMM kernel, or NCCL after it)")
    ap.add_argument("--workload", default="c4", choices=["c1", "c2", "c3", "c4", "c4b", "c5", "conv", "linear"],
                    help="c4 (default) is the headline configuration; c1..c5 are the remaining "
                         "BASELINE configurations, timed the same way (bench_configs.py); conv and linear "
                         "are the callers either side of the path (bench_callers.py)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload in ("conv", "linear"):
        import bench_callers

        bench_callers.run(args, measured_peaks, ClockSampler, load_reference)
    elif args.workload != "c4":
        import bench_configs

        bench_configs.run(args, measured_peaks, ClockSampler, load_reference)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
