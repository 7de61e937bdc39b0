"""The other BASELINE configurations, as `bench.py --workload c1|c2|c3|c4b|c5`.

bench.py's default line is the headline configuration (c4, f32 8192^3).  These are the
parity-test configurations timed the same way (CUDA events on the launching stream,
warm-up, max over ranks), so that each has a measured throughput and roofline fraction:

  c1   f32 512^3                                    (latency / HBM bound)
  c2   the six MLP products of 4096x784x1024 and 4096x1024x10, forward and backward,
       transposed operands as permuted views         (tensor bound + HBM-bound skinny ones)
  c3   attention-style batched f32: Q.K^T then S.V, B = 256, 128x64    (HBM bound)
  c4b  f64 4096^3                                    (FP64 tensor bound)
  c5   i32 batched 64 x (1024x512 . 512x1024)        (int32 multiply-add issue bound)

c3 and c5 shard over the batch dim at N > 1 (no exchange step: "weak" per batch, total work
fixed); the others run at N = 1 only.  One step = every product of the configuration once.
"""
from __future__ import annotations

import json
import os
import time

import numpy as np


def _products(name, torch, dev, world, rank, ttb):
    """Returns (list of (lhs, rhs, out) rank-3 views, description, dtype tag, seed)."""
    g = torch.Generator(device=dev)
    if name == "c1":
        g.manual_seed(0)
        a = torch.rand((1, 512, 512), generator=g, device=dev) * 2 - 1
        b = torch.rand((1, 512, 512), generator=g, device=dev) * 2 - 1
        return [(a, b, torch.empty((1, 512, 512), device=dev))], "C1: f32 512x512x512, U[-1,1), seed 0", "f32"
    if name == "c2":
        g.manual_seed(1)
        X = torch.rand((1, 4096, 784), generator=g, device=dev)
        W1 = (torch.rand((1, 1024, 784), generator=g, device=dev) * 2 - 1) / 784 ** 0.5
        W2 = (torch.rand((1, 10, 1024), generator=g, device=dev) * 2 - 1) / 1024 ** 0.5
        dH = torch.rand((1, 4096, 1024), generator=g, device=dev) * 2 - 1
        dC = torch.rand((1, 4096, 10), generator=g, device=dev) * 2 - 1
        H = torch.empty((1, 4096, 1024), device=dev)
        e = lambda *s: torch.empty(s, device=dev)
        prods = [
            (X, W1.permute(0, 2, 1), H),                       # fwd1  X . W1^T
            (H, W2.permute(0, 2, 1), e(1, 4096, 10)),          # fwd2  H . W2^T
            (dH, W1, e(1, 4096, 784)),                         # bwd   dH . W1
            (X.permute(0, 2, 1), dH, e(1, 784, 1024)),         # bwd   X^T . dH
            (dC, W2, e(1, 4096, 1024)),                        # bwd   dC . W2
            (H.permute(0, 2, 1), dC, e(1, 1024, 10)),          # bwd   H^T . dC
        ]
        return prods, "C2: MLP forward+backward products, X[4096,784], W1[1024,784], W2[10,1024], seed 1", "f32"
    if name == "c3":
        g.manual_seed(2)
        B = 256
        part = ttb.partition(B, 128, 64, 128, world, rank)
        nb = part.end - part.begin
        Q, K, V = (torch.randn((nb, 128, 64), generator=g, device=dev) for _ in range(3))
        S = torch.empty((nb, 128, 128), device=dev)
        O = torch.empty((nb, 128, 64), device=dev)
        return [(Q, K.permute(0, 2, 1), S), (S, V, O)], \
            f"C3: attention-style f32, Q.K^T then S.V, B=256 (this rank: {nb}), 128x64, N(0,1), seed 2", "f32"
    if name == "c4b":
        g.manual_seed(3)
        n = 4096
        a = torch.randn((1, n, n), generator=g, device=dev, dtype=torch.float64) * 8192 ** -0.5
        b = torch.randn((1, n, n), generator=g, device=dev, dtype=torch.float64) * 8192 ** -0.5
        return [(a, b, torch.empty((1, n, n), device=dev, dtype=torch.float64))], \
            "C4b: f64 4096x4096x4096, N(0,1/sqrt(8192)), seed 3", "f64"
    if name == "c5":
        g.manual_seed(4)
        part = ttb.partition(64, 1024, 512, 1024, world, rank)
        nb = part.end - part.begin
        a = torch.randint(-8, 9, (nb, 1024, 512), generator=g, device=dev, dtype=torch.int32)
        b = torch.randint(-8, 9, (nb, 512, 1024), generator=g, device=dev, dtype=torch.int32)
        return [(a, b, torch.empty((nb, 1024, 1024), device=dev, dtype=torch.int32))], \
            f"C5: i32 batched 64 x (1024x512 . 512x1024) (this rank: {nb}), ints in [-8,8], seed 4", "i32"
    raise ValueError(name)


def run(args, measured_peaks, ClockSampler, load_reference):
    import torch
    import torch.distributed as dist

    import tinytensor_b200 as ttb

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs CUDA devices; there is no CPU fallback")
    if world > 1 and args.workload not in ("c3", "c5"):
        raise SystemExit(f"--workload {args.workload} runs on one GPU only (it does not shard over the batch)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ttb.lib()
    prods, desc, dtag = _products(args.workload, torch, dev, world, rank, ttb)
    es = prods[0][0].element_size()
    flops = sum(2.0 * l.shape[0] * l.shape[1] * l.shape[2] * r.shape[2] for l, r, _ in prods)
    nbytes = sum(es * (l.numel() + r.numel() + o.numel()) for l, r, o in prods)
    # L2 flush between timed steps for the configurations that would otherwise sit in L2
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if nbytes < (256 << 20) else None

    def step():
        for l, r, o in prods:
            ttb.batched_matmul(l, r, out=o)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    variants = []
    for l, r, o in prods:
        ttb.batched_matmul(l, r, out=o)
        variants.append(ttb.last_variant().name)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches0 = ttb.launch_count()
    total_ms = 0.0
    t_begin = time.perf_counter()
    for _ in range(args.steps):
        if flush is not None:
            flush.zero_()
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        step()
        e.record()
        barrier()
        total_ms += s.elapsed_time(e)
    t_end = time.perf_counter()
    launches = ttb.launch_count() - launches0
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    ttb.check_device(local_rank)

    # The same step replayed from a CUDA graph: what the GPU needs once the host's launch work
    # (argument checks, tensor-map encoding, ctypes) is out of the timed region.  Small
    # configurations are bound by that host work when launched call by call.
    graph_ms = None
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            step()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                step()
        torch.cuda.current_stream().wait_stream(side)
        barrier()
        for _ in range(3):
            graph.replay()
        acc = 0.0
        for _ in range(args.steps):
            if flush is not None:
                flush.zero_()
            barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            graph.replay()
            e.record()
            barrier()
            acc += s.elapsed_time(e)
        graph_ms = acc / args.steps
        ttb.check_device(local_rank)
    except Exception as exc:  # capture is an extra: report why it was not taken
        graph_ms = f"not captured: {exc}"

    # end to end through the host-buffer entry point (pinned operands in, result out)
    host = []
    for l, r, o in prods:
        hl = torch.empty(l.shape, dtype=l.dtype, pin_memory=True)
        hr = torch.empty(r.shape, dtype=r.dtype, pin_memory=True)
        hl.copy_(l)
        hr.copy_(r)
        host.append((hl.numpy(), hr.numpy(), torch.empty(o.shape, dtype=o.dtype, pin_memory=True).numpy()))
    for hl, hr, ho in host:
        ttb.batched_matmul_host(hl, hr, out=ho, device=local_rank)
    barrier()
    e2e_steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for hl, hr, ho in host:
            ttb.batched_matmul_host(hl, hr, out=ho, device=local_rank)
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    h2d = sum(hl.nbytes + hr.nbytes for hl, hr, _ in host)
    d2h = sum(ho.nbytes for _, _, ho in host)

    ms_per_step = total_ms / args.steps
    if world > 1:
        t = torch.tensor([ms_per_step, e2e_s], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_per_step, e2e_s = (float(x) for x in t.cpu())
        tot = torch.tensor([flops, nbytes, h2d, d2h], device=dev, dtype=torch.float64)
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        flops_all, bytes_all, h2d, d2h = (float(x) for x in tot.cpu())
    else:
        flops_all, bytes_all = flops, nbytes
    if rank == 0:
        peaks, peak_kind = measured_peaks()
        value = flops_all / (ms_per_step * 1e-3) / 1e12
        gbs = nbytes / (ms_per_step * 1e-3) / 1e9          # this rank's algorithmic bytes
        share_flops = flops / (ms_per_step * 1e-3) / 1e12   # this rank's algorithmic flops
        bf16 = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
        if args.workload in ("c1", "c3"):
            roof = {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                    "peak_source": f"{peak_kind}: HBM copy bandwidth"}
        elif args.workload == "c2":
            roof = {"bound": "tensor", "achieved": share_flops, "peak": bf16 / 4.0, "unit": "TFLOP/s",
                    "frac": share_flops / (bf16 / 4.0), "traffic": None, "hbm_gbs_algorithmic": gbs,
                    "peak_source": f"{peak_kind}: bf16 sustained / 4; three of the six products are skinny "
                                   "(10 columns) and HBM-bound, they run on the CUDA-core kernel"}
        elif args.workload == "c4b":
            roof = {"bound": "tensor", "achieved": share_flops, "peak": 40.0, "unit": "TFLOP/s",
                    "frac": share_flops / 40.0, "traffic": None,
                    "peak_source": "nominal FP64 tensor rate of B200 (40 TFLOP/s); no measured figure available"}
        else:  # c5
            # One int32 multiply-add = ten u8 x u8 tensor-core multiply-adds (byte planes, mod 2^32);
            # int8 runs at twice the bf16 rate, so the derived ceiling is bf16 x 2 / 10.
            derived = bf16 * 2.0 / 10.0
            imad = 148 * 64 * 2 * 1.965e9 / 1e12  # 64 int32 multiply-add lanes per SM per clock
            roof = {"bound": "tensor", "achieved": share_flops, "peak": derived, "unit": "TOP/s",
                    "frac": share_flops / derived, "traffic": None,
                    "peak_source": f"{peak_kind}: bf16 sustained x 2 (int8 rate) / 10 (u8 x u8 products per int32 "
                                   "multiply-add)",
                    "hbm_gbs_algorithmic": gbs, "hbm_frac": gbs / peaks["hbm_gbs"],
                    "cuda_core_imad_nominal_tops": imad}
        # CPU baseline: the reference CPU kernel on the first product, bounded to about 10^10 flops
        import ctypes
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
        cpu_value = 2.0 * rows * hl.shape[2] * hr.shape[2] / cpu_s / 1e12
        line = {
            "metric": f"{dtag} matmul T{'FL' if dtag != 'i32' else ''}OP/s", "value": value,
            "unit": "TFLOP/s" if dtag != "i32" else "TOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": dtag, "data": "synthetic",
            "config": {"workload": desc, "kernels": variants,
                       "parallelism": f"batch shards x{world}, no exchange" if world > 1 else "single GPU",
                       "l2": "256 MiB buffer written between timed steps" if flush is not None
                       else "operands exceed the 126 MB L2; no explicit flush"},
            "clocks": clocks,
            "e2e": {"value": flops_all / e2e_s / 1e12, "unit": "TFLOP/s" if dtag != "i32" else "TOP/s",
                    "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "steps": e2e_steps,
                    "api": "ttb_batched_matmul_host (pinned host buffers, copies inside the timed region)"},
            "gpu_launches": int(launches),
            "roofline": roof,
            "us_per_step": ms_per_step * 1e3,
            "cuda_graph": ({"us_per_step": graph_ms * 1e3, "value": flops / (graph_ms * 1e-3) / 1e12,
                            "what": "the step captured once into a CUDA graph and replayed (this rank)"}
                           if isinstance(graph_ms, float) else {"us_per_step": None, "note": graph_ms}),
            "cpu_baseline": {"value": cpu_value, "unit": "TFLOP/s" if dtag != "i32" else "TOP/s", "cores": 1,
                             "kind": kind, "sample": f"first product, first {rows} lhs rows of batch 0, {cpu_s:.2f} s",
                             "host_cores_available": os.cpu_count()},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
