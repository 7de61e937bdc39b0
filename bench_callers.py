"""The callers either side of the matmul path, as `bench.py --workload conv|linear` (one GPU).

  conv    conv2d forward + backward of one ResNet-style layer, f32: input [32, 64, 56, 56],
          weight [128, 64, 3, 3], bias, stride 1, padding 1.  One step = forward, then backward
          (grad_input, grad_weight, grad_bias).  Algorithmic flops = the three GEMMs,
          3 x 2 * B * C_out * C_in*K*K * H_out*W_out.
  linear  tinytensor's Linear forward + relu, f32: x [8192, 4096] . W [4096, 4096] + bias, as ONE
          fused kernel, with the unfused sequence (product, then an in-place bias-add-relu pass over
          the output, the extra read + write the reference's separate kernels cost) timed beside it.

Timed like every other line of bench.py: CUDA events on the launching stream, >= 3 warm-up
steps, a 256 MiB buffer written between timed steps when the tensors would sit in L2.
"""
from __future__ import annotations

import ctypes
import json
import os
import time

import numpy as np


def _events(torch):
    return torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)


def _time(torch, fn, steps, flush):
    total = 0.0
    for _ in range(steps):
        if flush is not None:
            flush.zero_()
        torch.cuda.synchronize()
        s, e = _events(torch)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / steps


def run(args, measured_peaks, ClockSampler, load_reference):
    import torch

    import tinytensor_b200 as ttb

    if int(os.environ.get("WORLD_SIZE", "1")) > 1:
        raise SystemExit(f"--workload {args.workload} runs on one GPU only")
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs CUDA devices; there is no CPU fallback")
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    ttb.lib()
    warm = max(args.warmup, 3)
    peaks, peak_kind = measured_peaks()
    bf16 = peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"])
    g = torch.Generator(device=dev).manual_seed(7)
    sampler = ClockSampler(0)

    if args.workload == "conv":
        B, C_in, C_out, H, K, S, P = 32, 64, 128, 56, 3, 1, 1
        x = torch.randn((B, C_in, H, H), generator=g, device=dev)
        w = torch.randn((C_out, C_in, K, K), generator=g, device=dev) * (C_in * K * K) ** -0.5
        bias = torch.randn((C_out,), generator=g, device=dev)
        y = ttb.conv2d(x, w, bias, S, P)
        go = torch.randn(y.shape, generator=g, device=dev)
        hw = y.shape[2] * y.shape[3]
        gemm_flops = 2.0 * B * C_out * C_in * K * K * hw

        def fwd():
            ttb.conv2d(x, w, bias, S, P)

        def bwd():
            ttb.conv2d_backward(go, x, w, S, P)

        def step():
            fwd()
            bwd()

        for _ in range(warm):
            step()
        torch.cuda.synchronize()
        sampler.start()
        l0 = ttb.launch_count()
        t_begin = time.perf_counter()
        ms = _time(torch, step, args.steps, None)   # 231 MB of columns + 103 MB of tensors exceed L2
        t_end = time.perf_counter()
        launches = ttb.launch_count() - l0
        clocks = sampler.stop(t_begin, t_end)
        ms_fwd = _time(torch, fwd, max(3, args.steps // 2), None)
        ms_bwd = _time(torch, bwd, max(3, args.steps // 2), None)
        ttb.check_device(0)

        # end to end: pinned host tensors in, forward, result out
        hx, hw_, hb = (t.cpu().pin_memory() for t in (x, w, bias))
        hy = torch.empty(y.shape, dtype=y.dtype).pin_memory()

        def e2e_step():
            dx, dw, db = (t.to(dev, non_blocking=True) for t in (hx, hw_, hb))
            hy.copy_(ttb.conv2d(dx, dw, db, S, P), non_blocking=True)
            torch.cuda.synchronize()

        e2e_step()
        t0 = time.perf_counter()
        n_e2e = max(1, min(args.steps, 5))
        for _ in range(n_e2e):
            e2e_step()
        e2e_s = (time.perf_counter() - t0) / n_e2e

        # the reference's CUDA kernels, forward without bias (unroll + matmul per batch item)
        existing = None
        ref_cuda = os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle", "_ref", "libttref_cuda.so")
        if os.path.exists(ref_cuda):
            rc_lib = ctypes.CDLL(ref_cuda)
            yr = torch.empty_like(y)
            unrolled = torch.empty(C_in * K * K * hw, device=dev)
            st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

            def ref_fwd():
                rc = rc_lib.ref_cuda_conv2d_forward_f32(
                    ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()), ctypes.c_void_p(yr.data_ptr()),
                    ctypes.c_void_p(unrolled.data_ptr()), B, C_in, H, H, C_out, K, S, P, st)
                assert rc == 0

            ref_fwd()
            ms_ref = _time(torch, ref_fwd, 3, None)
            ours = ttb.conv2d(x, w, None, S, P)
            diff = float((ours - yr).abs().max() / yr.abs().max())
            existing = {"value": gemm_flops / (ms_ref * 1e-3) / 1e12, "unit": "TFLOP/s", "ms": ms_ref,
                        "kind": "reference", "max_diff_vs_ours_rel_to_max": diff,
                        "what": "tinytensor's unroll_kernel + matmul_kernel<float> per batch item "
                                "(backend/cuda/conv.cu:126-160), forward without bias, compiled for sm_100a"}

        # CPU baseline: the reference's CPU conv kernels, forward, 2 batch items
        lib, kind = load_reference()
        nb = 2
        xs = np.ascontiguousarray(x[:nb].cpu().numpy())
        ws, bs = w.cpu().numpy(), bias.cpu().numpy()
        ys = np.empty((nb, C_out, y.shape[2], y.shape[3]), dtype=np.float32)
        fn = getattr(lib, ("ref" if kind == "reference" else "oracle") + "_conv2d_forward_f32")
        t0 = time.perf_counter()
        fn(ctypes.c_void_p(xs.ctypes.data), ctypes.c_void_p(ws.ctypes.data), ctypes.c_void_p(bs.ctypes.data),
           ctypes.c_void_p(ys.ctypes.data), nb, C_in, H, H, C_out, K, S, P)
        cpu_s = time.perf_counter() - t0
        value = 3.0 * gemm_flops / (ms * 1e-3) / 1e12
        line = {
            "metric": "f32 conv2d forward+backward TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": 1,
            "steps": args.steps, "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"conv2d f32 fwd+bwd: input [{B},{C_in},{H},{H}], weight [{C_out},{C_in},{K},{K}], "
                                   f"bias, stride {S}, padding {P}, N(0,1) data, seed 7",
                       "parallelism": "single GPU", "kernels": ttb.last_variant().name,
                       "l2": "columns buffer (231 MB) and tensors exceed the 126 MB L2; no explicit flush"},
            "clocks": clocks,
            "forward": {"ms": ms_fwd, "tflops": gemm_flops / (ms_fwd * 1e-3) / 1e12},
            "backward": {"ms": ms_bwd, "tflops": 2.0 * gemm_flops / (ms_bwd * 1e-3) / 1e12},
            "e2e": {"value": gemm_flops / e2e_s / 1e12, "unit": "TFLOP/s",
                    "h2d_bytes_per_step": int(hx.nbytes + hw_.nbytes + hb.nbytes), "d2h_bytes_per_step": int(hy.nbytes),
                    "steps": n_e2e, "api": "tinytensor_b200.conv2d forward on tensors copied from pinned host "
                                           "memory, result copied back, inside the timed region"},
            "gpu_launches": int(launches),
            "roofline": {"bound": "tensor", "achieved": value, "peak": bf16 / 4.0, "unit": "TFLOP/s",
                         "frac": value / (bf16 / 4.0), "traffic": None,
                         "peak_source": f"{peak_kind}: bf16 sustained / 4 (hybrid split); the step also holds the "
                                        "HBM-bound im2col / col2im / reduction kernels"},
            "cpu_baseline": {"value": nb / B * gemm_flops / cpu_s / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": kind,
                             "sample": f"forward of the first {nb} batch items, {cpu_s:.2f} s",
                             "host_cores_available": os.cpu_count()},
            "existing_gpu_kernel": existing,
        }
        print(json.dumps(line), flush=True)
        return

    # ---- linear
    N, K, M = 8192, 4096, 4096
    x = torch.randn((1, N, K), generator=g, device=dev)
    w = torch.randn((1, K, M), generator=g, device=dev) * K ** -0.5
    bias = torch.randn((M,), generator=g, device=dev)
    out = torch.empty((1, N, M), device=dev)
    flops = 2.0 * N * K * M

    def fused():
        ttb.batched_matmul_fused(x, w, bias, ttb.Activation.RELU, out=out)

    def unfused():
        ttb.batched_matmul(x, w, out=out)
        out.add_(bias).relu_()   # stands for the reference's expand + add kernel and relu kernel

    for _ in range(warm):
        fused()
        unfused()
    torch.cuda.synchronize()
    sampler.start()
    l0 = ttb.launch_count()
    t_begin = time.perf_counter()
    ms = _time(torch, fused, args.steps, None)
    t_end = time.perf_counter()
    launches = ttb.launch_count() - l0
    clocks = sampler.stop(t_begin, t_end)
    ms_unfused = _time(torch, unfused, args.steps, None)
    ttb.check_device(0)
    value = flops / (ms * 1e-3) / 1e12
    lib, kind = load_reference()
    rows = 128
    xs = np.ascontiguousarray(x[0, :rows].cpu().numpy())
    ws = np.ascontiguousarray(w[0].cpu().numpy())
    ys = np.empty((rows, M), dtype=np.float32)
    fn = getattr(lib, "ref_matmul_f32" if kind == "reference" else "oracle_matmul_f32")
    t0 = time.perf_counter()
    if kind == "reference":
        fn(ctypes.c_void_p(xs.ctypes.data), ctypes.c_void_p(ws.ctypes.data), ctypes.c_void_p(ys.ctypes.data),
           ctypes.c_int64(1), ctypes.c_int(rows), ctypes.c_int(K), ctypes.c_int(M))
    else:
        fn(ctypes.c_void_p(xs.ctypes.data), ctypes.c_void_p(ws.ctypes.data), ctypes.c_void_p(ys.ctypes.data),
           ctypes.c_int64(1), ctypes.c_int64(rows), ctypes.c_int64(K), ctypes.c_int64(M))
    cpu_s = time.perf_counter() - t0
    line = {
        "metric": "f32 linear+relu TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"Linear forward + relu, f32: x [{N},{K}] . W [{K},{M}] + bias, seed 7",
                   "parallelism": "single GPU", "kernels": ttb.last_variant().name,
                   "l2": "operands (336 MiB with the output) exceed the 126 MB L2; no explicit flush"},
        "clocks": clocks,
        "unfused": {"ms": ms_unfused, "tflops": flops / (ms_unfused * 1e-3) / 1e12,
                    "what": "the same product, then bias add and relu as passes over the output"},
        "e2e": None,
        "gpu_launches": int(launches),
        "roofline": {"bound": "tensor", "achieved": value, "peak": bf16 / 4.0, "unit": "TFLOP/s",
                     "frac": value / (bf16 / 4.0), "traffic": None,
                     "peak_source": f"{peak_kind}: bf16 sustained / 4 (hybrid split)"},
        "cpu_baseline": {"value": 2.0 * rows * K * M / cpu_s / 1e12, "unit": "TFLOP/s", "cores": 1, "kind": kind,
                         "sample": f"the product for the first {rows} rows of x (no bias, no relu), {cpu_s:.2f} s",
                         "host_cores_available": os.cpu_count()},
    }
    print(json.dumps(line), flush=True)
