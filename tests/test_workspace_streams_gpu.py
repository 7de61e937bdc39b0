"""Scratch workspaces are keyed by (device, stream): products that split K (partial sums in a
cached buffer) on two streams of one device run side by side without sharing it; a buffer that
would have to grow while its stream is being captured into a CUDA graph is refused with a clear
message, and a buffer a captured launch used stays valid after a larger call outgrew it."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host

pytestmark = pytest.mark.gpu


def test_two_streams_splitting_k_do_not_share_partial_sums(ttb, oracle, reset_options):
    rng = np.random.default_rng(90)
    ttb.set_option("force_variant", int(ttb.Variant.SIMT_SPLITK))
    shapes = [(1, 96, 8192, 80), (2, 64, 6144, 128)]   # few tiles, long K: many K splits each
    data = []
    for B, N, K, M in shapes:
        a = rng.integers(-2 ** 20, 2 ** 20, (B, N, K)).astype(np.int32)
        b = rng.integers(-2 ** 20, 2 ** 20, (B, K, M)).astype(np.int32)
        data.append((dev(a), dev(b), oracle.matmul(a, b)))
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    outs = [[torch.empty((d[0].shape[0], d[0].shape[1], d[1].shape[2]), dtype=torch.int32, device="cuda")
             for _ in range(8)] for d in data]
    torch.cuda.synchronize()
    for it in range(8):       # interleave launches so that the two streams overlap on the GPU
        for s, (A, Bm, _), o in zip(streams, data, outs):
            ttb.batched_matmul(A, Bm, out=o[it], stream=s)
            assert ttb.last_variant() == ttb.Variant.SIMT_SPLITK
    torch.cuda.synchronize()
    for (_, _, want), o in zip(data, outs):
        for got in o:
            assert np.array_equal(host(got), want)   # wrap-around sums, bit-exact
    ttb.check_device(0)


def test_growth_during_capture_is_refused_and_captured_buffers_survive(ttb, oracle, reset_options):
    rng = np.random.default_rng(91)
    ttb.set_option("force_variant", int(ttb.Variant.SIMT_SPLITK))
    a = rng.integers(-9, 10, (1, 64, 4096, )).astype(np.int32).reshape(1, 64, 4096)
    b = rng.integers(-9, 10, (1, 4096, 64)).astype(np.int32)
    A, Bm = dev(a), dev(b)
    out = torch.zeros((1, 64, 64), dtype=torch.int32, device="cuda")
    side = torch.cuda.Stream()                      # a fresh stream: nothing cached for it yet
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with pytest.raises(ttb.TTBError, match="before the capture"):
            with torch.cuda.graph(graph, stream=side):
                ttb.batched_matmul(A, Bm, out=out, stream=side)
    torch.cuda.synchronize()
    # the same call once outside a capture, then the capture goes through
    with torch.cuda.stream(side):
        ttb.batched_matmul(A, Bm, out=out, stream=side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            ttb.batched_matmul(A, Bm, out=out, stream=side)
        # a much larger split-K product on the same stream outgrows the cached buffer ...
        big_a = dev(rng.integers(-9, 10, (4, 128, 8192)).astype(np.int32))
        big_b = dev(rng.integers(-9, 10, (4, 8192, 128)).astype(np.int32))
        ttb.batched_matmul(big_a, big_b, stream=side)
    torch.cuda.synchronize()
    # ... and the graph, which still writes its partial sums through the old one, replays right
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert np.array_equal(host(out), oracle.matmul(a, b))
    ttb.check_device(0)
