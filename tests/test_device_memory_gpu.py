"""Stream-ordered cached allocations and device-to-device copies (the library side of what
tinytensor's DeviceMemory<T> and Tensor::to(Device) do with cudaMalloc / cudaFree and a host
bounce: tinytensor/tensor/backend/cuda/data_types.cu:38-50,102-116,
tinytensor/autograd/unary_ops.cpp:67-83)."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _as_tensor(ptr, n, dtype=torch.float32):
    """A torch view of `n` elements at a raw device address (no ownership)."""
    class _Holder:
        pass

    h = _Holder()
    typestr = {torch.float32: "<f4", torch.int32: "<i4", torch.uint8: "|u1"}[dtype]
    h.__cuda_array_interface__ = {"shape": (n,), "typestr": typestr, "data": (ptr, False), "version": 2}
    return torch.as_tensor(h, device="cuda")


def test_alloc_free_counters_and_reuse(ttb):
    before = ttb.device_memory_stats(0)
    n = 1 << 20
    p = ttb.device_alloc(4 * n)
    assert p != 0 and p % 256 == 0
    s1 = ttb.device_memory_stats(0)
    assert s1["current"] == before["current"] + 4 * n
    assert s1["total"] == before["total"] + 4 * n
    assert s1["reserved"] >= s1["current"]
    t = _as_tensor(p, n)
    t.fill_(3.0)
    assert float(t.sum().item()) == 3.0 * n
    del t
    ttb.device_free(p)
    s2 = ttb.device_memory_stats(0)
    assert s2["current"] == before["current"]
    assert s2["total"] == s1["total"]
    assert s2["reserved"] >= 4 * n          # the block stays cached in the pool
    q = ttb.device_alloc(4 * n)             # same size, same stream: served from the cache
    assert q != 0
    assert ttb.device_memory_stats(0)["reserved"] == s2["reserved"]
    ttb.device_free(q)
    torch.cuda.synchronize()


def test_result_buffer_from_the_pool_feeds_the_product(ttb, oracle):
    """What the tinytensor-side adapter does: allocate the result from the pool, run the product into it,
    free it in stream order."""
    rng = np.random.default_rng(5)
    a = rng.integers(-9, 10, (2, 70, 33), dtype=np.int32)
    b = rng.integers(-9, 10, (2, 33, 52), dtype=np.int32)
    A, B = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    p = ttb.device_alloc(2 * 70 * 52 * 4)
    out = _as_tensor(p, 2 * 70 * 52, torch.int32).view(2, 70, 52)
    ttb.batched_matmul(A, B, out=out)
    got = out.cpu().numpy()
    del out
    ttb.device_free(p)
    assert np.array_equal(got, oracle.matmul(a, b))


def test_many_sizes_stay_disjoint(ttb):
    sizes = [1, 7, 256, 4096, 100_000, 1 << 22]
    ptrs = [ttb.device_alloc(s) for s in sizes]
    spans = sorted(zip(ptrs, sizes))
    for (p0, s0), (p1, _) in zip(spans, spans[1:]):
        assert p0 + s0 <= p1
    for i, (p, s) in enumerate(zip(ptrs, sizes)):
        _as_tensor(p, s, torch.uint8).fill_(i + 1)
    for i, (p, s) in enumerate(zip(ptrs, sizes)):
        t = _as_tensor(p, s, torch.uint8)
        assert int(t.min().item()) == i + 1 and int(t.max().item()) == i + 1
    for p in ptrs:
        ttb.device_free(p)
    torch.cuda.synchronize()


def test_zero_bytes_null_and_foreign_pointers(ttb):
    assert ttb.device_alloc(0) == 0
    ttb.device_free(0)                       # NULL: no-op
    foreign = torch.empty(16, device="cuda")
    with pytest.raises(ttb.TTBError, match="not allocated by ttb_device_alloc"):
        ttb.device_free(foreign.data_ptr())
    p = ttb.device_alloc(64)
    ttb.device_free(p)
    with pytest.raises(ttb.TTBError, match="freed already"):
        ttb.device_free(p)
    out = ctypes.c_void_p()
    assert ttb.lib().ttb_device_alloc(ctypes.byref(out), 64, torch.cuda.device_count(), None) == -4  # TTB_EDEVICE
    assert ttb.lib().ttb_device_alloc(None, 64, 0, None) == -1


def test_trim_returns_cached_blocks(ttb):
    p = ttb.device_alloc(8 << 20)
    ttb.device_free(p)
    assert ttb.device_memory_stats(0)["reserved"] >= 8 << 20
    ttb.device_trim(0)
    s = ttb.device_memory_stats(0)
    assert s["reserved"] == s["current"] or s["reserved"] < 8 << 20


def test_alloc_and_free_inside_a_cuda_graph(ttb):
    """Allocation and release are stream-ordered, so a product with a pool-allocated temporary can be
    recorded into a CUDA graph."""
    a = torch.randn(1, 64, 64, device="cuda")
    out = torch.zeros(1, 64, 64, device="cuda")
    want = ttb.batched_matmul(a, a).clone()
    L = ttb.lib()
    ttb.device_free(ttb.device_alloc(64 * 64 * 4))  # the pool exists before the capture starts
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            p = ttb.device_alloc(64 * 64 * 4, stream=side)
            # While the capture runs the block is only a reserved address, so it is handed to the
            # C entry points as a raw pointer (torch cannot wrap it yet).
            va = ttb.view_of(a)
            stream = ctypes.c_void_p(side.cuda_stream)
            assert L.ttb_batched_matmul(ctypes.byref(va), ctypes.byref(va), ctypes.c_void_p(p), 5, 0, stream) == 0
            assert L.ttb_copy_device_to_device(ctypes.c_void_p(out.data_ptr()), 0, ctypes.c_void_p(p), 0,
                                               64 * 64 * 4, stream) == 0
            ttb.device_free(p, stream=side)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(2):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, want)


def test_copy_same_device(ttb):
    src = torch.arange(100_000, dtype=torch.int32, device="cuda").view(100, 1000)
    out = ttb.to_device(src.t(), 0)          # a permuted view: made contiguous first, like to_vec
    assert out.shape == (1000, 100) and torch.equal(out, src.t())
    assert ttb.lib().ttb_copy_device_to_device(None, 0, ctypes.c_void_p(src.data_ptr()), 0, 16, None) == -1


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_copy_between_devices(ttb):
    src = torch.randn(1 << 20, device="cuda:0")
    out = ttb.to_device(src, 1)
    torch.cuda.synchronize(1)
    assert out.device.index == 1 and torch.equal(out.cpu(), src.cpu())
    p = ttb.device_alloc(4 << 20, device=0)  # pool memory of device 0, read by device 1
    t = _as_tensor(p, 1 << 20)
    t.copy_(src)
    torch.cuda.synchronize(0)
    out2 = torch.empty(1 << 20, device="cuda:1")
    rc = ttb.lib().ttb_copy_device_to_device(ctypes.c_void_p(out2.data_ptr()), 1, ctypes.c_void_p(p), 0, 4 << 20,
                                             ctypes.c_void_p(torch.cuda.current_stream(1).cuda_stream))
    assert rc == 0
    torch.cuda.synchronize(1)
    assert torch.equal(out2.cpu(), src.cpu())
    del t
    ttb.device_free(p, device=0)
