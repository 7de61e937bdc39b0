"""Benchmark of the matmul hot path: f32 8192 x 8192 x 8192 (the configuration the
headline metric is quoted on), one process per GPU.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

One "step" is one pass of the product over one set of synthetic operands
(N(0, 1/sqrt(8192)) entries drawn with the reference's own generator, seed 3).  At N > 1 the
product is split into output-column blocks, one per rank, and C is all-gathered (strong
scaling: the total work is fixed).  Prints ONE JSON line on rank 0.  Inputs (768 MiB with C)
are far larger than L2, so no explicit L2 flush is needed between timed iterations.

After the timed region, untimed, EVERY rank checks the gathered C against a float64 product
on rows and columns sampled across tiles, CTA halves, raster groups and every rank's column
block, then runs three more products with rescaled operands and checks those too (a stale
tile or a peer store that landed in the wrong place shows up here); the run exits non-zero
when the 1e-5 gate is missed.  The line also carries the other BASELINE configurations
("other_configs", bench_configs.py), each with its own parity verdict.

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
GATE = 1e-5                                     # f32: max|c - c64| / max|c64|


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


def cpu_sample(lib, kind, a_rows: np.ndarray, b: np.ndarray):
    """lhs[rows, K] . rhs[K, M] on one host core with the reference kernel -> (seconds, result)."""
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
    return time.perf_counter() - t0, out


def reference_arm_operands(rows: int):
    """Operands of the reference arm, made without this library: the reference's own generator
    (oracle/_ref/libttref_full.so: Generator(3), normal(0, 8192^-1/2)) when it travelled, else
    numpy draws of the same distribution.  -> (first `rows` rows of A, B, how)."""
    full = ROOT / "oracle" / "_ref" / "libttref_full.so"
    sd = DIM ** -0.5
    if full.exists():
        sys.path.insert(0, str(ROOT / "tests"))
        import ref_full

        g = ref_full.Gen(SEED)
        a = g.normal(0.0, sd, (DIM, DIM))[:rows].copy()
        b = g.normal(0.0, sd, (DIM, DIM))
        return a, b, "tinytensor's Generator(3) and normal(), run by the reference library itself"
    rng = np.random.default_rng(SEED)
    a = rng.standard_normal((rows, DIM), dtype=np.float32) * np.float32(sd)
    b = rng.standard_normal((DIM, DIM), dtype=np.float32) * np.float32(sd)
    return a, b, "numpy draws of N(0, 1/sqrt(8192)) (the reference library did not travel)"


def error_vs_float64(got: np.ndarray, a_rows: np.ndarray, b: np.ndarray) -> float:
    want = a_rows.astype(np.float64) @ b.astype(np.float64)
    return float(np.abs(got - want).max() / np.abs(want).max())


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # under torchrun only rank 0 measures the CPU arm
    lib, kind = load_reference()
    rows = 256  # per step: 256 of the 8192 rows of lhs = 1/32 of the product, about 1 s of CPU
    a, b, how = reference_arm_operands(rows)
    for _ in range(args.warmup):
        cpu_sample(lib, kind, a, b)
    t = 0.0
    out = None
    for _ in range(args.steps):
        dt, out = cpu_sample(lib, kind, a, b)
        t += dt
    flops = 2.0 * rows * DIM * DIM * args.steps
    value = flops / t / 1e12
    sample = f"{rows} of {DIM} lhs rows per step (1/{DIM // rows} of the product), single thread"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * t / args.steps * (DIM / rows),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "timed": sample, "inputs": how},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": kind, "sample": sample,
                         "host_cores_available": os.cpu_count()},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "parity": {"max_rel_to_max": error_vs_float64(out, a, b), "gate": GATE,
                   "what": "the reference CPU kernel's own error on its sample, same measure"},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- our arm
def sample_points(world: int):
    """Rows and columns of C to verify: both CTAs of a pair tile (rows 0-127 / 128-255 of a
    256-row tile), tile edges, first / middle / last raster group (8 row tiles = 2048 rows), and
    for the columns every rank's block with its first and last column."""
    rows = sorted({0, 1, 127, 128, 255, 256, 383, 2047, 2048, 2049, 4095, 4096, 4224, 6143, 6272, 8063, 8064, 8191})
    cols = set()
    blk = DIM // world
    for r in range(world):
        cols.update({r * blk, r * blk + 1, r * blk + 129, r * blk + blk // 2 + 3, (r + 1) * blk - 1})
    cols.update({255, 256, 4095, 4096})
    return rows, sorted(c for c in cols if 0 <= c < DIM)


def check_against_float64(torch, A, B, C, rows, cols) -> float:
    """max|c - c64| / max|c64| over the sampled rows and columns of C = A . B (float64 on the GPU)."""
    r = torch.tensor(rows, device=A.device)
    c = torch.tensor(cols, device=A.device)
    want_r = torch.matmul(A[0, r].double(), B[0].double())
    want_c = torch.matmul(A[0].double(), B[0][:, c].double())
    scale = max(float(want_r.abs().max()), float(want_c.abs().max()))
    err = max(float((C[0, r].double() - want_r).abs().max()), float((C[0][:, c].double() - want_c).abs().max()))
    return err / scale


_T0 = time.perf_counter()


_PHASE = ["start"]


def watchdog(seconds: float) -> None:
    """Ends the process with a message naming the phase it was in if the run outlives `seconds`:
    a wait on another rank that never comes must not hold the GPUs until someone else's limit."""
    def run():
        time.sleep(seconds)
        print(f"[bench rank {os.environ.get('RANK', '0')}] gave up after {seconds:.0f} s in phase: {_PHASE[0]}",
              file=sys.stderr, flush=True)
        os._exit(3)
    threading.Thread(target=run, daemon=True).start()


def progress(msg: str) -> None:
    """One line per phase on stderr (stdout carries only the JSON line): a run that is cut short
    still shows how far every rank got."""
    _PHASE[0] = "after: " + msg
    print(f"[bench rank {os.environ.get('RANK', '0')} +{time.perf_counter() - _T0:7.1f}s] {msg}", file=sys.stderr,
          flush=True)


def sustained_step_count(ms_per_step: float, steps: int, torch, dist=None, device=None) -> int:
    """Steps of the >= 2 s loop, from the measured time of one step.  Every rank must come out with
    the SAME number: each step meets the other ranks at a barrier, and a rank with one step more
    would wait there for ever.  So the slowest rank's time decides (all-reduce MAX)."""
    ms_all = ms_per_step
    if dist is not None:
        t = torch.tensor([ms_per_step], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_all = float(t.item())
    return int(max(steps, min(4000, 2200.0 / max(ms_all, 1e-3))))


def run_ours(args):
    import torch
    import torch.distributed as dist

    import bench_configs
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
    for kv in args.ttb_option:
        key, _, val = kv.partition("=")
        ttb.set_option(key, int(val))
    progress("process group up, library loaded")
    peaks, peak_kind = measured_peaks()

    # Operands, drawn on the host as a tinytensor program draws them (Generator(3), normal) and
    # uploaded: every rank holds the full A and B (placing them is set-up, not timed).
    ops = ttb.config_operands("c4")
    hA = torch.from_numpy(ops["A"]).unsqueeze(0).pin_memory()
    hB = torch.from_numpy(ops["B"]).unsqueeze(0).pin_memory()
    A, B = hA.to(dev), hB.to(dev)
    progress("operands drawn and uploaded")
    fused = args.exchange in ("fused", "fused-peer", "fused-multicast")
    sharded = ttb.ShardedMatmul(exchange={"fused": "auto", "fused-peer": "peer", "fused-multicast": "multicast"}.get(
        args.exchange, "auto")) if world > 1 else None
    # Two C buffers used in turn.  At N > 1 with the fused exchange they live in symmetric memory:
    # the GEMM kernel itself stores each finished tile into every rank's C over NVLink, and a
    # rank only overwrites a buffer after every rank has passed the barrier of the product in
    # between (see ShardedMatmul.symmetric_output); "nccl" keeps C private and all-gathers after.
    if world > 1 and fused:
        Cs = [sharded.symmetric_output((1, DIM, DIM), torch.float32, dev) for _ in range(2)]
    else:
        Cs = [torch.empty((1, DIM, DIM), device=dev) for _ in range(2)]
    part = ttb.partition(1, DIM, DIM, DIM, world, rank)
    exchange_desc = "NCCL all_gather + re-layout"
    if world > 1 and fused:
        multicast = sharded.exchange != "peer" and sharded.multicast_available(Cs[0])
        exchange_desc = ("fused into the GEMM kernel: each tile stored once through NVSwitch multicast (multimem.st)"
                         if multicast else
                         "fused into the GEMM kernel: bulk tensor stores from the epilogue to every peer over NVLink")

    def step(i, kernel_done=None):
        if sharded is None:
            ttb.batched_matmul(A, B, out=Cs[i & 1])
            if kernel_done is not None:
                kernel_done.record()
        else:
            sharded(A, B, out=Cs[i & 1], kernel_done=kernel_done)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed_loop(n_steps, with_kernel_events):
        """n_steps back to back between two events; optionally an event pair around each step's
        kernel (recorded inside the same loop, so the kernel time can never exceed the step)."""
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
              for _ in range(n_steps)] if with_kernel_events else None
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sampler = ClockSampler(local_rank)
        barrier()
        sampler.start()
        t_begin = time.perf_counter()
        start.record()
        for i in range(n_steps):
            if ev is not None:
                ev[i][0].record()
                step(i, ev[i][1])
            else:
                step(i)
        stop.record()
        if n_steps > 100:
            progress(f"{n_steps} steps queued")
        barrier()
        if n_steps > 100:
            progress("ranks met after the loop")
        clocks = sampler.stop(t_begin, time.perf_counter())
        ms = start.elapsed_time(stop) / n_steps
        kernel = sum(a.elapsed_time(b) for a, b in ev) / n_steps if ev is not None else None
        return ms, kernel, clocks

    for i in range(max(args.warmup, 3)):
        step(i)
    progress("warm-up done")
    launches0 = ttb.launch_count()
    ms_per_step, kernel_ms, clocks = timed_loop(args.steps, True)
    launches = ttb.launch_count() - launches0
    variant = ttb.last_variant().name
    progress(f"timed loop done: {ms_per_step:.3f} ms per step")
    ttb.check_device(local_rank)

    # The same step for at least two seconds without a pause: the power-capped regime.
    sustained_steps = sustained_step_count(ms_per_step, args.steps, torch, dist if world > 1 else None, dev)
    sus_ms, _, sus_clocks = timed_loop(sustained_steps, False)
    progress(f"sustained loop done: {sus_ms:.3f} ms per step over {sustained_steps} steps")
    ttb.check_device(local_rank)

    # ---- verification, untimed, on every rank
    rows, cols = sample_points(world)
    errs = [check_against_float64(torch, A, B, Cs[(args.steps - 1) & 1], rows, cols),
            check_against_float64(torch, A, B, Cs[args.steps & 1], rows, cols)]
    for j in range(3):
        # new values in the same buffers: anything left over from an earlier product, and any
        # peer store that went astray, no longer matches
        A.mul_(-1.5 if j % 2 == 0 else 0.75)
        B.mul_(1.25)
        step(j)
        errs.append(check_against_float64(torch, A, B, Cs[j & 1], rows, cols))
    A.copy_(hA)
    B.copy_(hB)
    torch.cuda.synchronize()
    max_err = max(errs)
    progress(f"parity checked: {max_err:.2e}")

    # ---- breakdown of a step at N > 1 (each piece timed alone, same events method)
    breakdown = None
    if world > 1:
        def time_of(fn, n=10):
            for _ in range(2):
                fn()
            barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(n):
                fn()
            e.record()
            barrier()
            return s.elapsed_time(e) / n

        blk = Cs[0][:, :, part.begin:part.end]
        math_only = time_of(lambda: ttb.batched_matmul(A, B[:, :, part.begin:part.end], out=blk))
        breakdown = {"math_only_ms": math_only, "fused_kernel_ms": kernel_ms, "step_ms": ms_per_step}
        if fused:
            hdl = sharded._symm[Cs[0].untyped_storage().data_ptr()][1]
            breakdown["barrier_alone_ms"] = time_of(lambda: hdl.barrier(), 20)
            peers = [hdl.get_buffer((rank + i) % world, (1, DIM, DIM), torch.float32) for i in range(1, world)]

            def push():
                for pc in peers:
                    pc[:, :, part.begin:part.end].copy_(blk, non_blocking=True)

            copy_ms = time_of(push)
            sent = (world - 1) * blk.numel() * 4
            breakdown["peer_copy_alone_ms"] = copy_ms
            breakdown["peer_copy_alone_gbs_out_per_gpu"] = sent / (copy_ms * 1e-3) / 1e9
            breakdown["what"] = ("math_only: this rank's block, no exchange; fused_kernel: the same with every tile "
                                 "stored to all peers, measured inside the timed loop; barrier_alone: one "
                                 "symmetric-memory barrier; peer_copy_alone: this rank's block copied to every peer "
                                 "by plain strided device copies, all ranks at once, no math")
        ttb.check_device(local_rank)

    # ---- end to end: operands in pinned host memory, result back in host memory, every step
    progress("breakdown done")
    e2e_steps = max(1, min(args.steps, 5))
    if world == 1:
        hC = torch.empty((1, DIM, DIM), dtype=torch.float32, pin_memory=True)
        nA, nB, nC = hA.numpy(), hB.numpy(), hC.numpy()
        run_e2e = lambda: ttb.batched_matmul_host(nA, nB, out=nC, device=local_rank)
        h2d, d2h = nA.nbytes + nB.nbytes, nC.nbytes
        e2e_api = "ttb_batched_matmul_host (pinned host buffers, copies inside the timed region)"
    else:
        # one process per GPU: each holds its shard of the operands in its own pinned host memory
        (r0, r1), (c0, c1) = sharded.host_shards(DIM, DIM, DIM)
        hA_rows = hA[0, r0:r1].contiguous().pin_memory()
        hB_blk = hB[0][:, c0:c1].contiguous().pin_memory()
        hC_blk = torch.empty((DIM, c1 - c0), dtype=torch.float32, pin_memory=True)
        run_e2e = lambda: sharded.columns_from_host(hA_rows, hB_blk, hC_blk, DIM)
        h2d = hA_rows.numel() * 4 + hB_blk.numel() * 4
        d2h = hC_blk.numel() * 4
        e2e_api = ("ShardedMatmul.columns_from_host: each rank uploads its rows of A and its column block of B from "
                   "its own pinned host memory over its own PCIe link, A is all-gathered over NVLink, the rank's "
                   "block of C is downloaded")
    run_e2e()  # warm-up: grows the staging buffers
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        run_e2e()
    barrier()
    e2e_s = time.perf_counter() - t0
    progress(f"end-to-end loop done: {e2e_s / e2e_steps * 1e3:.1f} ms per step")
    e2e_err = None
    if world == 1:
        e2e_err = check_against_float64(torch, A, B, hC.to(dev), rows[:6], cols[:6])
    else:
        mine = [c for c in cols if part.begin <= c < part.end][:4]
        if mine:
            cc = torch.tensor(mine, device=dev)
            want = torch.matmul(A[0].double(), B[0][:, cc].double())
            got = hC_blk[:, [c - part.begin for c in mine]].to(dev).double()
            e2e_err = float((got - want).abs().max() / want.abs().max())
    max_err = max(max_err, e2e_err or 0.0)

    if world > 1:
        t = torch.tensor([ms_per_step, kernel_ms, e2e_s, sus_ms, max_err], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step, kernel_ms, e2e_s, sus_ms, max_err = (float(x) for x in t.cpu())
        byt = torch.tensor([h2d, d2h], device=dev, dtype=torch.float64)
        dist.all_reduce(byt, op=dist.ReduceOp.SUM)
        h2d, d2h = (int(x) for x in byt.cpu())
        if breakdown:
            keys = [k for k, v in breakdown.items() if isinstance(v, float)]
            bt = torch.tensor([breakdown[k] for k in keys], device=dev, dtype=torch.float64)
            dist.all_reduce(bt, op=dist.ReduceOp.MAX)
            for k, v in zip(keys, bt.cpu()):
                breakdown[k] = float(v)
            if "peer_copy_alone_ms" in breakdown:   # bandwidth from the slowest rank's time
                breakdown["peer_copy_alone_gbs_out_per_gpu"] = (world - 1) * (DIM // world) * DIM * 4 / (
                    breakdown["peer_copy_alone_ms"] * 1e-3) / 1e9
    parity = {"max_rel_to_max": max_err, "gate": GATE, "ok": bool(max_err <= GATE), "ranks_checked": world,
              "checked": f"{len(rows)} rows x all columns and {len(cols)} columns x all rows of both C buffers after "
                         "the timed loop, of three further products with rescaled operands, and of the end-to-end "
                         "result, each against a float64 product, on every rank"}

    # ---- measured ceilings from this library's own kernels (rank 0, untimed)
    own_peaks = {}
    other = {}
    if rank == 0:
        def best_ms(fn, n=5):
            fn()
            torch.cuda.synchronize()
            best = 1e9
            for _ in range(n):
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                fn()
                e.record()
                torch.cuda.synchronize()
                best = min(best, s.elapsed_time(e))
            return best

        # One TF32 pass of the same TMA -> tcgen05 pipeline with the converters idle: what this
        # kernel's data path delivers to kind::tf32 MMAs at this size (results are not fp32-accurate).
        ttb.set_option("tf32_terms", 1)
        ttb.set_option("tc_debug", 1)
        own_peaks["tf32_tflops_measured"] = FLOPS_PER_STEP / (best_ms(lambda: ttb.batched_matmul(A, B, out=Cs[0])) * 1e-3) / 1e12
        ttb.set_option("tf32_terms", 2)
        ttb.set_option("tc_debug", 0)
        own_peaks["tf32_what"] = ("this library's TMA -> tcgen05 pipeline, one kind::tf32 pass, converters idle, 8192^3, "
                                  "best of 5 launches (burst clocks); bound by the 4-byte operands' L2 -> SM traffic")
        own_peaks["fp64_tflops_measured"] = ttb.measure_fp64_tensor_peak(local_rank)
        own_peaks["fp64_what"] = "register-only loop of mma.sync.m16n8k4.f64, two 8-warp CTAs per SM, best of 3 launches"
        ttb.check_device(local_rank)
    fp64_peak = own_peaks.get("fp64_tflops_measured")

    # ---- the other BASELINE configurations at this N (c3 / c5 batch-sharded over all ranks)
    for name in ("c1", "c2", "c3", "c4b", "c5"):
        if world > 1 and name not in bench_configs.SHARDED and rank != 0:
            continue
        if args.skip_other_configs:
            break
        rec, _ = bench_configs.measure(name, torch, dist, ttb, dev, world, rank, 10, peaks, peak_kind, fp64_peak,
                                       with_graph=(name in ("c1", "c3")), with_e2e=False)
        other[name] = rec
        progress(f"configuration {name} measured")
    if world > 1:
        dist.barrier()

    if rank == 0:
        value = FLOPS_PER_STEP / (ms_per_step * 1e-3) / 1e12
        sus_value = FLOPS_PER_STEP / (sus_ms * 1e-3) / 1e12
        # Tensor-pipe roofline of the dominant kernel: this GPU's share of the algorithmic flops
        # over the kernel's own duration.  fp32 accuracy costs, per algorithmic multiply-add, one
        # TF32 multiply-add (the cost of two bf16 ones: dense TF32 runs at half the bf16 rate) and
        # two bf16 multiply-adds, i.e. four bf16 multiply-add times: the ceiling is bf16 / 4.  The
        # K-step timed loop is a burst (well under a second at full clocks): burst peak.  The
        # two-second loop runs power-capped: sustained peak.  Classic 3xTF32 would cost six
        # (bf16 / 2 / 3); that figure is reported beside it.
        share = (part.end - part.begin) / DIM
        achieved = FLOPS_PER_STEP * share / (kernel_ms * 1e-3) / 1e12
        burst = peaks["bf16_tflops"]
        sustained = peaks.get("bf16_tflops_sustained", burst)
        peak = burst / 4.0
        sus_achieved = FLOPS_PER_STEP * share / (sus_ms * 1e-3) / 1e12   # whole step: kernel + exchange
        # CPU baseline: the reference's CPU kernel on a bounded sample, one host core
        lib, kind = load_reference()
        cpu_rows = 2048
        a_rows = np.ascontiguousarray(ops["A"][:cpu_rows])
        cpu_s, cpu_out = cpu_sample(lib, kind, a_rows, ops["B"])
        cpu_value = 2.0 * cpu_rows * DIM * DIM / cpu_s / 1e12
        cpu_err = error_vs_float64(cpu_out[:256], a_rows[:256], ops["B"])
        # The kernel this library replaces, as a second reported baseline (N = 1 only): the
        # reference's own CUDA matmul kernel compiled from its sources (oracle/_ref), run on
        # this GPU on the same operands through the launch configuration of its runner.
        existing = None
        if world == 1:
            ref_ms = bench_configs.reference_cuda_kernel_ms(torch, [(A, B, Cs[1])], "f32", steps=2)
            if ref_ms:
                existing = {"value": FLOPS_PER_STEP / (ref_ms * 1e-3) / 1e12, "unit": UNIT, "ms": ref_ms,
                            "kind": "reference", "speedup_of_this_library": ref_ms / ms_per_step,
                            "what": "tinytensor's matmul_kernel<float> (backend/cuda/kernel/matmul.cuh) compiled for sm_100a"}
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": WORKLOAD,
                       "inputs": "tinytensor's Generator(3), normal(0, 8192^-1/2), restated (ttb_generator_*) and "
                                 "pinned to the reference library bit for bit",
                       "parallelism": (f"column blocks x{world} + all-gather of C ({exchange_desc}), two C buffers "
                                       "used in turn")
                       if world > 1 else "single GPU",
                       "l2": "operands (768 MiB with C) exceed the 126 MB L2; no explicit flush",
                       **({"library_options": list(args.ttb_option)} if args.ttb_option else {}),
                       "kernel": variant, "arithmetic": ("split precision on tcgen05: TF32 product of the high parts + two bf16 "
                                      "correction products, fp32 accumulate in TMEM chunks, fp32 register sums")},
            "clocks": clocks,
            "parity": parity,
            "e2e": {"value": FLOPS_PER_STEP / (e2e_s / e2e_steps) / 1e12, "unit": UNIT,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps, "api": e2e_api},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": UNIT, "frac": achieved / peak,
                         "traffic": None,
                         "traffic_source": "not measured in this run; one ncu capture of this kernel on this workload is "
                                           "summarised in profiles/gemm_f32_3xtf32_pair_8192cubed.md (2.58 GB per full launch)",
                         "kernel_ms": kernel_ms,
                         "peak_source": f"{peak_kind}: bf16 burst {burst} TFLOP/s / 4 (one TF32 + two bf16 products per "
                                        "flop); the timed loop lasts well under a second",
                         "time_x_mhz": kernel_ms * (clocks.get("sm_mhz") or 0.0),
                         "frac_of_3xtf32_derived_peak": achieved / (burst / 6.0),
                         "frac_of_own_tf32_pass_div_3": (achieved / (own_peaks["tf32_tflops_measured"] / 3.0)
                                                         if own_peaks.get("tf32_tflops_measured") else None),
                         "hbm_gbs_algorithmic": BYTES_PER_STEP * share / (kernel_ms * 1e-3) / 1e9},
            "sustained": {"value": sus_value, "unit": UNIT, "steps": sustained_steps, "ms_per_step": sus_ms,
                          "seconds": sus_ms * sustained_steps / 1e3, "clocks": sus_clocks,
                          "roofline_frac": sus_achieved / (sustained / 4.0), "peak": sustained / 4.0,
                          "peak_source": f"{peak_kind}: bf16 sustained {sustained} TFLOP/s / 4",
                          "time_x_mhz": sus_ms * (sus_clocks.get("sm_mhz") or 0.0),
                          "what": "the same step back to back for at least two seconds (power-capped clocks); at "
                                  "N > 1 the step includes the exchange"},
            "own_peaks": own_peaks,
            "breakdown": breakdown,
            "cpu_baseline": {"value": cpu_value, "unit": UNIT, "cores": 1, "kind": kind,
                             "sample": f"first {cpu_rows} of {DIM} lhs rows (1/{DIM // cpu_rows} of the product), {cpu_s:.1f} s",
                             "host_cores_available": os.cpu_count(),
                             "max_rel_to_max_vs_float64": cpu_err},
            "existing_gpu_kernel": existing,
            "other_configs": other,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    bad = [k for k, v in other.items() if not v["parity"]["ok"]]
    if not parity["ok"] or bad:
        raise SystemExit(f"parity check failed: headline {parity['max_rel_to_max']:.3e} (gate {GATE}), configs {bad}")


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
    ap.add_argument("--skip-other-configs", action="store_true",
                    help="c4 only: leave the other BASELINE configurations out of the line")
    ap.add_argument("--ttb-option", action="append", default=[], metavar="KEY=VALUE",
                    help="library option set before anything runs (ttb_set_option), for A/B runs; repeatable")
    ap.add_argument("--deadline", type=float, default=900.0,
                    help="seconds after which the process ends itself, naming the phase it was in")
    args = ap.parse_args()
    watchdog(args.deadline)
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
