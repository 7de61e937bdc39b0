"""The no-allocation entry point (ttb_batched_matmul_static_scratch).

It exists for host programs that cannot let the library allocate: they own all device
memory through their own allocator or a fixed budget, or they cannot take the device-wide
synchronisation of cudaMalloc in their loop.  The K-split partial sums live in a fixed
16 MiB device array instead of a cudaMalloc'ed workspace.

Checked here, through the C ABI: its result equals the ordinary entry point's on two calls
in a row (the second with another dtype and shape, so stale partial sums from the first call
would show), and results beyond the fixed array are refused with a clear message.  This file
sorts last on purpose: a run that stops at the first failure has then already run everything
else.  It also passes when run alone in a fresh process.
"""
import ctypes

import numpy as np
import pytest
import torch

from gpu_util import dev, host, rel_to_max

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5


def _call_static(ttb, a, b, out):
    """Straight through the C ABI, no Python convenience layer in between."""
    from tinytensor_b200.backend import _DTYPE_CODE, view_of

    lv, rv = view_of(a), view_of(b)
    rc = ttb.lib().ttb_batched_matmul_static_scratch(
        ctypes.byref(lv), ctypes.byref(rv), ctypes.c_void_p(out.data_ptr()), _DTYPE_CODE[a.dtype],
        a.device.index or 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc


def test_static_scratch_matches_ordinary_entry_point_twice_in_a_row(ttb):
    rng = np.random.default_rng(41)
    # call 1: i32, skinny output with a long K (many K splits), transposed-view lhs
    a1 = rng.integers(-1000, 1000, (2, 300, 2048)).astype(np.int32)
    b1 = rng.integers(-1000, 1000, (2, 2048, 12)).astype(np.int32)
    A1 = dev(a1.transpose(0, 2, 1)).permute(0, 2, 1)  # same values, K no longer contiguous
    B1 = dev(b1)
    out1 = torch.empty((2, 300, 12), dtype=torch.int32, device="cuda")
    assert _call_static(ttb, A1, B1, out1) == 0, ttb.lib().ttb_last_error()
    ref1 = ttb.batched_matmul(A1, B1)
    assert torch.equal(out1, ref1)  # integers: bit-exact, wrap-around included

    # call 2, straight after: f32, different shape -- shares the same scratch array
    a2 = rng.standard_normal((1, 200, 1500)).astype(np.float32)
    b2 = rng.standard_normal((1, 1500, 96)).astype(np.float32)
    A2, B2 = dev(a2), dev(b2)
    out2 = torch.empty((1, 200, 96), dtype=torch.float32, device="cuda")
    assert _call_static(ttb, A2, B2, out2) == 0, ttb.lib().ttb_last_error()
    ref2 = ttb.batched_matmul(A2, B2)
    want = np.matmul(a2.astype(np.float64), b2.astype(np.float64))
    assert rel_to_max(host(out2), want) <= F32_TOL
    assert rel_to_max(host(out2), host(ref2).astype(np.float64)) <= F32_TOL

    # and the first problem again: the second call's leftovers must not leak into it
    out3 = torch.empty_like(out1)
    assert _call_static(ttb, A1, B1, out3) == 0
    assert torch.equal(out3, ref1)
    ttb.check_device(0)


def test_static_scratch_through_the_python_wrapper_all_dtypes(ttb, oracle):
    rng = np.random.default_rng(42)
    for dt in (np.uint8, np.int16, np.int64, np.float64):
        if np.dtype(dt).kind in "iu":
            a = rng.integers(0, 120, (1, 70, 600)).astype(dt)
            b = rng.integers(0, 120, (1, 600, 45)).astype(dt)
        else:
            a = rng.standard_normal((1, 70, 600)).astype(dt)
            b = rng.standard_normal((1, 600, 45)).astype(dt)
        out = torch.empty((1, 70, 45), dtype=dev(a).dtype, device="cuda")
        ttb.batched_matmul_static_scratch(dev(a), dev(b), out)
        if np.dtype(dt).kind in "iu":
            assert np.array_equal(host(out), oracle.matmul(a, b)), dt
        else:
            want = np.matmul(a.astype(np.longdouble), b.astype(np.longdouble))
            assert rel_to_max(host(out), want) <= 1e-12


def test_static_scratch_refuses_results_beyond_the_fixed_array(ttb):
    # 2 splits x 2048 x 2048 x 4 bytes = 32 MiB > 16 MiB
    a = torch.zeros((1, 2048, 64), device="cuda")
    b = torch.zeros((1, 64, 2048), device="cuda")
    out = torch.empty((1, 2048, 2048), device="cuda")
    rc = _call_static(ttb, a, b, out)
    assert rc == -9  # TTB_ELIMIT
    msg = ttb.lib().ttb_last_error().decode()
    assert "scratch" in msg and "16777216" in msg
    with pytest.raises(ttb.TTBError):
        ttb.batched_matmul_static_scratch(a, b, out)


def test_static_scratch_calls_leave_device_memory_and_current_device_alone(ttb):
    """After one warm-up call (which loads the library's device image, scratch array included),
    further calls of other shapes and dtypes neither take nor return device memory -- seen from
    the driver (free bytes) and from the library's own pool counters -- and the calling thread's
    current device stays what it was."""
    rng = np.random.default_rng(43)
    cases = []
    for dt, shape in ((np.float32, (1, 90, 700, 33)), (np.int16, (3, 40, 512, 17)), (np.float64, (1, 16, 2048, 130)),
                      (np.int64, (2, 33, 300, 65))):
        B, N, K, M = shape
        if np.dtype(dt).kind in "iu":
            a, b = rng.integers(-9, 9, (B, N, K)).astype(dt), rng.integers(-9, 9, (B, K, M)).astype(dt)
        else:
            a, b = rng.standard_normal((B, N, K)).astype(dt), rng.standard_normal((B, K, M)).astype(dt)
        A, Bm = dev(a), dev(b)
        cases.append((A, Bm, torch.empty((B, N, M), dtype=A.dtype, device="cuda")))
    assert _call_static(ttb, *cases[0]) == 0, ttb.lib().ttb_last_error()   # warm-up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info(0)
    stats0 = ttb.device_memory_stats(0)
    device0 = torch.cuda.current_device()
    for _ in range(2):
        for A, Bm, out in cases:
            assert _call_static(ttb, A, Bm, out) == 0, ttb.lib().ttb_last_error()
            assert torch.cuda.current_device() == device0
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info(0)
    assert free1 == free0
    assert ttb.device_memory_stats(0) == stats0
    for A, Bm, out in cases:
        assert torch.equal(out, ttb.batched_matmul(A, Bm)) or rel_to_max(
            host(out), host(ttb.batched_matmul(A, Bm)).astype(np.float64)) <= F32_TOL
    ttb.check_device(0)
