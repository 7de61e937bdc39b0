"""The BASELINE configurations other than the headline one, measured the same way.

    python bench.py --workload c1|c2|c3|c4b|c5        one configuration, one JSON line
    bench.py's default line carries all five under "other_configs"

  c1   f32 512^3                                    (latency / HBM bound)
  c2   the six MLP products of 4096x784x1024 and 4096x1024x10, forward and backward,
       transposed operands as permuted views         (tensor bound + HBM-bound skinny ones)
  c3   attention-style batched f32: Q.K^T then S.V, B = 256, 128x64    (HBM bound)
  c4b  f64 4096^3                                    (FP64 tensor bound)
  c5   i32 batched 64 x (1024x512 . 512x1024)        (int8 tensor cores, byte planes)

Operands are drawn on the host with the reference's own generator and seeds
(tinytensor_b200.inputs.config_operands) and uploaded.  c3 and c5 shard over the batch dim at
N > 1 (no exchange step); the others run on rank 0 only.  One step = every product of the
configuration once.  Every measurement comes with a parity verdict of the same run (f32 / f64
against a wider product, i32 bit-exact) and with the time of the reference's own CUDA kernel
(oracle/_ref/libttref_cuda.so, when it travelled) on the same operands.
"""
from __future__ import annotations

import ctypes
import os
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
SHARDED = ("c3", "c5")


def _dev(torch, a, dev):
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def build_products(name, torch, dev, world, rank, ttb):
    """-> (products [(lhs, rhs, out)], description, dtype tag, host operands of this rank)."""
    e = lambda *s, dt=torch.float32: torch.empty(s, device=dev, dtype=dt)
    if name == "c1":
        ops = ttb.config_operands("c1")
        a, b = _dev(torch, ops["A"], dev).unsqueeze(0), _dev(torch, ops["B"], dev).unsqueeze(0)
        return [(a, b, e(1, 512, 512))], "C1: f32 512x512x512, U[-1,1), seed 0", "f32", ops
    if name == "c2":
        ops = ttb.config_operands("c2")
        X, W1, W2, dH, dC = (_dev(torch, ops[k], dev).unsqueeze(0) for k in ("X", "W1", "W2", "dH", "dC"))
        H = e(1, 4096, 1024)
        prods = [
            (X, W1.permute(0, 2, 1), H),                       # fwd1  X . W1^T
            (H, W2.permute(0, 2, 1), e(1, 4096, 10)),          # fwd2  H . W2^T
            (dH, W1, e(1, 4096, 784)),                         # bwd   dH . W1
            (X.permute(0, 2, 1), dH, e(1, 784, 1024)),         # bwd   X^T . dH
            (dC, W2, e(1, 4096, 1024)),                        # bwd   dC . W2
            (H.permute(0, 2, 1), dC, e(1, 1024, 10)),          # bwd   H^T . dC
        ]
        return prods, "C2: MLP forward+backward products, X[4096,784], W1[1024,784], W2[10,1024], seed 1", "f32", ops
    if name == "c3":
        part = ttb.partition(256, 128, 64, 128, world, rank)
        ops = ttb.config_operands("c3", batch_range=(part.begin, part.end))
        nb = part.end - part.begin
        Q, K, V = (_dev(torch, ops[k], dev) for k in ("Q", "K", "V"))
        S, O = e(nb, 128, 128), e(nb, 128, 64)
        return [(Q, K.permute(0, 2, 1), S), (S, V, O)], \
            f"C3: attention-style f32, Q.K^T then S.V, B=256 (this rank: {nb}), 128x64, N(0,1), seed 2", "f32", ops
    if name == "c4b":
        ops = ttb.config_operands("c4b")
        a, b = _dev(torch, ops["A"], dev).unsqueeze(0), _dev(torch, ops["B"], dev).unsqueeze(0)
        return [(a, b, e(1, 4096, 4096, dt=torch.float64))], "C4b: f64 4096x4096x4096, N(0,1/sqrt(8192)), seed 3", \
            "f64", ops
    if name == "c5":
        part = ttb.partition(64, 1024, 512, 1024, world, rank)
        ops = ttb.config_operands("c5", batch_range=(part.begin, part.end))
        nb = part.end - part.begin
        a, b = _dev(torch, ops["A"], dev), _dev(torch, ops["B"], dev)
        return [(a, b, e(nb, 1024, 1024, dt=torch.int32))], \
            f"C5: i32 batched 64 x (1024x512 . 512x1024) (this rank: {nb}), ints in [-8,8], seed 4", "i32", ops
    raise ValueError(name)


def parity(name, torch, prods):
    """Checks the outputs the timed kernels left behind.  -> dict(ok, what, max_err | None)."""
    worst = 0.0
    if name == "c5":
        a, b, o = prods[0]
        nb = min(a.shape[0], 4)
        want = torch.matmul(a[:nb].double(), b[:nb].double())   # |sums| <= 32768: exact in f64
        ok = bool(torch.equal(o[:nb].double(), want))
        return {"ok": ok, "gate": "bit-exact", "checked": f"{nb} batches of this rank against an exact f64 product"}
    if name == "c4b":
        a, b, o = prods[0]
        rows = [0, 1, 127, 128, 2047, 2048, 4094, 4095]
        al = a[0, rows].cpu().numpy().astype(np.longdouble)
        want = al @ b[0].cpu().numpy().astype(np.longdouble)
        got = o[0, rows].cpu().numpy().astype(np.longdouble)
        err = float(np.abs(got - want).max() / np.abs(want).max())
        return {"ok": err <= 1e-12, "gate": 1e-12, "max_rel_to_max": err, "checked": "8 rows against long double"}
    for l, r, o in prods:
        want = torch.matmul(l.double(), r.double())
        worst = max(worst, float((o.double() - want).abs().max() / want.abs().max()))
    return {"ok": worst <= 1e-5, "gate": 1e-5, "max_rel_to_max": worst, "checked": "every product against float64"}


def reference_cuda_kernel_ms(torch, prods, dtag, steps=3):
    """Time of tinytensor's own matmul_kernel<T> on the same products.  It takes contiguous
    operands only; permuted views are copied first, outside the timed region (the reference's
    runner makes those copies on every call, so this favours it)."""
    path = ROOT / "oracle" / "_ref" / "libttref_cuda.so"
    if not path.exists():
        return None
    lib = ctypes.CDLL(str(path))
    fn = getattr(lib, f"ref_cuda_matmul_{dtag}")
    fn.restype = ctypes.c_int
    cont = [(l.contiguous(), r.contiguous(), torch.empty_like(o)) for l, r, o in prods]
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run():
        for l, r, o in cont:
            rc = fn(ctypes.c_void_p(l.data_ptr()), ctypes.c_void_p(r.data_ptr()), ctypes.c_void_p(o.data_ptr()),
                    ctypes.c_int(l.shape[0]), ctypes.c_int(l.shape[1]), ctypes.c_int(l.shape[2]),
                    ctypes.c_int(r.shape[2]), stream)
            if rc != 0:
                raise RuntimeError(f"reference CUDA kernel launch failed: cudaError {rc}")

    run()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        run()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / steps


def roofline(name, peaks, peak_kind, share_flops, gbs, fp64_peak, burst):
    bf16 = peaks["bf16_tflops"] if burst else peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    regime = "burst" if burst else "sustained"
    if name in ("c1", "c3"):
        return {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                "frac": gbs / peaks["hbm_gbs"], "traffic": None, "peak_source": f"{peak_kind}: HBM copy bandwidth"}
    if name == "c2":
        return {"bound": "tensor", "achieved": share_flops, "peak": bf16 / 4.0, "unit": "TFLOP/s",
                "frac": share_flops / (bf16 / 4.0), "traffic": None, "hbm_gbs_algorithmic": gbs,
                "peak_source": f"{peak_kind}: bf16 {regime} / 4; three of the six products are skinny "
                               "(10 columns) and HBM-bound, they run on the CUDA-core kernel"}
    if name == "c4b":
        return {"bound": "tensor", "achieved": share_flops, "peak": fp64_peak, "unit": "TFLOP/s",
                "frac": share_flops / fp64_peak if fp64_peak else None, "traffic": None,
                "peak_source": "measured in this run: register-only loop of the kernel's own mma.sync.m16n8k4.f64 "
                               "(ttb_measure_fp64_tensor_peak)"}
    # c5: one int32 multiply-add = ten u8 x u8 tensor-core multiply-adds (byte planes, mod 2^32);
    # int8 runs at twice the bf16 rate, so the derived ceiling is bf16 x 2 / 10.
    derived = bf16 * 2.0 / 10.0
    return {"bound": "tensor", "achieved": share_flops, "peak": derived, "unit": "TOP/s",
            "frac": share_flops / derived, "traffic": None,
            "peak_source": f"{peak_kind}: bf16 {regime} x 2 (int8 rate) / 10 (u8 x u8 products per int32 multiply-add)",
            "hbm_gbs_algorithmic": gbs, "hbm_frac": gbs / peaks["hbm_gbs"]}


def measure(name, torch, dist, ttb, dev, world, rank, steps, peaks, peak_kind, fp64_peak, with_graph=True,
            with_e2e=True):
    """Times configuration `name` on this rank (all ranks for the batch-sharded ones) and returns the
    per-configuration record; collective calls inside are made by every rank of the group."""
    prods, desc, dtag, _ = build_products(name, torch, dev, world, rank, ttb)
    es = prods[0][0].element_size()
    flops = sum(2.0 * l.shape[0] * l.shape[1] * l.shape[2] * r.shape[2] for l, r, _ in prods)
    nbytes = sum(es * (l.numel() + r.numel() + o.numel()) for l, r, o in prods)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if nbytes < (256 << 20) else None
    sharded = world > 1 and name in SHARDED

    # The timed calls are prepared ones: the two ttb_view structures of a product are filled once
    # and a step is one foreign call per product, which is what a C++ host pays (the Python
    # convenience wrapper spends several times the call's own cost on filling them).
    prepared = [ttb.PreparedMatmul(l, r, o) for l, r, o in prods]

    def step():
        for pm in prepared:
            pm()

    def barrier():
        torch.cuda.synchronize()
        if sharded:
            dist.barrier()
            torch.cuda.synchronize()

    variants = []
    for _ in range(3):
        step()
    for l, r, o in prods:
        ttb.batched_matmul(l, r, out=o)
        variants.append(ttb.last_variant().name)
    barrier()
    launches0 = ttb.launch_count()
    total_ms = 0.0
    for _ in range(steps):
        if flush is not None:
            flush.zero_()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        step()
        e.record()
        barrier()
        total_ms += s.elapsed_time(e)
    launches = ttb.launch_count() - launches0
    ttb.check_device(dev.index)
    verdict = parity(name, torch, prods)

    graph_ms = None
    if with_graph:
        # The same step replayed from a CUDA graph: what the GPU needs once the host's launch work
        # (argument checks, tensor-map lookup, the foreign call) is out of the timed region.
        graph = None
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for pm in prepared:
                    pm(stream=side)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for pm in prepared:
                        pm(stream=side)
            torch.cuda.current_stream().wait_stream(side)
        except Exception as exc:  # capture is an extra: report why it was not taken
            graph = None
            graph_ms = f"not captured: {exc}"
        if sharded:
            # the timing loop below meets the other ranks at barriers: all of them, or none
            flag = torch.tensor([1.0 if graph is not None else 0.0], device=dev)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if float(flag) == 0.0 and graph is not None:
                graph, graph_ms = None, "not captured on another rank"
        if graph is not None:
            barrier()
            for _ in range(3):
                graph.replay()
            acc = 0.0
            for _ in range(steps):
                if flush is not None:
                    flush.zero_()
                barrier()
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                graph.replay()
                e.record()
                barrier()
                acc += s.elapsed_time(e)
            graph_ms = acc / steps
            ttb.check_device(dev.index)

    e2e = None
    if with_e2e:
        host = []
        for l, r, o in prods:
            hl = torch.empty(l.shape, dtype=l.dtype, pin_memory=True)
            hr = torch.empty(r.shape, dtype=r.dtype, pin_memory=True)
            hl.copy_(l)
            hr.copy_(r)
            host.append((hl.numpy(), hr.numpy(), torch.empty(o.shape, dtype=o.dtype, pin_memory=True).numpy()))
        for hl, hr, ho in host:
            ttb.batched_matmul_host(hl, hr, out=ho, device=dev.index)
        barrier()
        e2e_steps = max(1, min(steps, 5))
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            for hl, hr, ho in host:
                ttb.batched_matmul_host(hl, hr, out=ho, device=dev.index)
        barrier()
        e2e_s = (time.perf_counter() - t0) / e2e_steps
        e2e = {"seconds": e2e_s, "h2d": sum(hl.nbytes + hr.nbytes for hl, hr, _ in host),
               "d2h": sum(ho.nbytes for _, _, ho in host), "steps": e2e_steps}

    ref_ms = reference_cuda_kernel_ms(torch, prods, dtag) if rank == 0 else None
    ms_per_step = total_ms / steps
    flops_all, bytes_all = flops, nbytes
    if sharded:
        t = torch.tensor([ms_per_step, e2e["seconds"] if e2e else 0.0, 0.0 if verdict["ok"] else 1.0], device=dev,
                         dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step = float(t[0])
        if e2e:
            e2e["seconds"] = float(t[1])
        verdict["ok"] = bool(float(t[2]) == 0.0)
        verdict["ranks_checked"] = world
        tot = torch.tensor([flops, nbytes, e2e["h2d"] if e2e else 0, e2e["d2h"] if e2e else 0], device=dev,
                           dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        flops_all, bytes_all = float(tot[0]), float(tot[1])
        if e2e:
            e2e["h2d"], e2e["d2h"] = int(tot[2]), int(tot[3])
    unit = "TFLOP/s" if dtag != "i32" else "TOP/s"
    value = flops_all / (ms_per_step * 1e-3) / 1e12
    gbs = nbytes / (ms_per_step * 1e-3) / 1e9
    share = flops / (ms_per_step * 1e-3) / 1e12
    rec = {
        "workload": desc, "value": value, "unit": unit, "dtype": dtag, "n_gpus": world if sharded else 1,
        "us_per_step": ms_per_step * 1e3, "steps": steps, "kernels": variants, "gpu_launches": int(launches),
        "calls": "prepared C-ABI calls, one per product (argument structures built once, as a C++ host builds them)",
        "parallelism": f"batch shards x{world}, no exchange" if sharded else "single GPU",
        "l2": "256 MiB buffer written between timed steps" if flush is not None
        else "operands exceed the 126 MB L2; no explicit flush",
        # a timed step is far shorter than a second: the GPU runs at its burst clocks
        "roofline": roofline(name, peaks, peak_kind, share, gbs, fp64_peak, burst=True),
        "parity": verdict,
        "cuda_graph": ({"us_per_step": graph_ms * 1e3, "value": flops / (graph_ms * 1e-3) / 1e12}
                       if isinstance(graph_ms, float) else ({"note": graph_ms} if graph_ms else None)),
        "existing_gpu_kernel": ({"us_per_step": ref_ms * 1e3, "value": flops / (ref_ms * 1e-3) / 1e12, "unit": unit,
                                 "speedup_of_this_library": ref_ms / ms_per_step if not sharded else None,
                                 "what": "tinytensor's matmul_kernel<T> (backend/cuda/kernel/matmul.cuh) for sm_100a, "
                                         "rank 0's products, permuted operands copied contiguous beforehand"}
                                if ref_ms else None),
    }
    if e2e:
        rec["e2e"] = {"value": flops_all / e2e["seconds"] / 1e12, "unit": unit, "h2d_bytes_per_step": int(e2e["h2d"]),
                      "d2h_bytes_per_step": int(e2e["d2h"]), "steps": e2e["steps"],
                      "api": "ttb_batched_matmul_host (pinned host buffers, copies inside the timed region)"}
    return rec, prods


def cpu_baseline(prods, dtag, load_reference):
    """The reference CPU kernel on the first product, bounded to about 10^10 multiply-adds."""
    lib, kind = load_reference()
    l, r, _ = prods[0]
    hl = np.ascontiguousarray(l[:1].cpu().numpy())
    hr = np.ascontiguousarray(r[:1].cpu().numpy())
    rows = int(max(1, min(hl.shape[1], 1.0e10 / (2.0 * hl.shape[2] * hr.shape[2]))))
    hl = np.ascontiguousarray(hl[:, :rows])
    out = np.empty((1, rows, hr.shape[2]), dtype=hl.dtype)
    fn = getattr(lib, ("ref_matmul_" if kind == "reference" else "oracle_matmul_") + dtag)
    t0 = time.perf_counter()
    if kind == "reference":
        fn(ctypes.c_void_p(hl.ctypes.data), ctypes.c_void_p(hr.ctypes.data), ctypes.c_void_p(out.ctypes.data),
           ctypes.c_int64(1), ctypes.c_int(rows), ctypes.c_int(hl.shape[2]), ctypes.c_int(hr.shape[2]))
    else:
        fn(ctypes.c_void_p(hl.ctypes.data), ctypes.c_void_p(hr.ctypes.data), ctypes.c_void_p(out.ctypes.data),
           ctypes.c_int64(1), ctypes.c_int64(rows), ctypes.c_int64(hl.shape[2]), ctypes.c_int64(hr.shape[2]))
    cpu_s = time.perf_counter() - t0
    return {"value": 2.0 * rows * hl.shape[2] * hr.shape[2] / cpu_s / 1e12,
            "unit": "TFLOP/s" if dtag != "i32" else "TOP/s", "cores": 1, "kind": kind,
            "sample": f"first product, first {rows} lhs rows of batch 0, {cpu_s:.2f} s",
            "host_cores_available": os.cpu_count()}


def run(args, measured_peaks, ClockSampler, load_reference):
    """`bench.py --workload cX`: one configuration as its own JSON line."""
    import json

    import torch
    import torch.distributed as dist

    import tinytensor_b200 as ttb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs CUDA devices; there is no CPU fallback")
    if world > 1 and args.workload not in SHARDED:
        raise SystemExit(f"--workload {args.workload} runs on one GPU only (it does not shard over the batch)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ttb.lib()
    peaks, peak_kind = measured_peaks()
    fp64_peak = ttb.measure_fp64_tensor_peak(local_rank) if args.workload == "c4b" else None
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    t_begin = time.perf_counter()
    rec, prods = measure(args.workload, torch, dist, ttb, dev, world, rank, args.steps, peaks, peak_kind, fp64_peak)
    clocks = sampler.stop(t_begin, time.perf_counter()) if rank == 0 else None
    if rank == 0:
        line = {
            "metric": f"{rec['dtype']} matmul {rec['unit']}", "value": rec["value"], "unit": rec["unit"],
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": rec["us_per_step"] / 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": rec["dtype"],
            "data": "synthetic",
            "config": {"workload": rec["workload"], "kernels": rec["kernels"], "parallelism": rec["parallelism"],
                       "l2": rec["l2"], "inputs": "the reference's Generator(seed) restated (ttb_generator_*)"},
            "clocks": clocks, "e2e": rec.get("e2e"), "gpu_launches": rec["gpu_launches"], "roofline": rec["roofline"],
            "parity": rec["parity"], "us_per_step": rec["us_per_step"], "cuda_graph": rec["cuda_graph"],
            "existing_gpu_kernel": rec["existing_gpu_kernel"],
            "cpu_baseline": cpu_baseline(prods, rec["dtype"], load_reference),
        }
        if fp64_peak:
            line["fp64_tflops_measured"] = fp64_peak
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if not rec["parity"]["ok"]:
        raise SystemExit(f"parity check failed for {args.workload}: {rec['parity']}")
