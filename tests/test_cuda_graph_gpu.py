"""The products can be recorded into a CUDA graph and replayed (launch-bound loops of small
products are what graphs are for).  Replays must give the same result as direct calls, also for
a shape that uses stream-K: its ready flags are raised by the writer and lowered again by the one
reader, so every launch (and every replay) starts from flags at zero."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host, random_operands, rel_to_max

pytestmark = pytest.mark.gpu


def _capture(fn):
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        fn()  # warm-up on the capturing stream: one-time allocations happen here
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            fn()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    return graph


@pytest.mark.parametrize("dt,shape", [(np.float32, (1, 512, 512, 512)), (np.float32, (8, 128, 64, 128)),
                                      (np.int32, (2, 256, 256, 256)), (np.float64, (1, 200, 96, 120)),
                                      (np.int16, (2, 45, 70, 38))])
def test_replay_matches_direct_call(ttb, oracle, dt, shape):
    rng = np.random.default_rng(80)
    B, N, K, M = shape
    a, b = random_operands(rng, dt, B, N, K, M, -9, 10)
    A, Bm = dev(a), dev(b)
    out = torch.zeros((B, N, M), dtype=A.dtype, device="cuda")
    direct = ttb.batched_matmul(A, Bm).clone()
    graph = _capture(lambda: ttb.batched_matmul(A, Bm, out=out))
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, direct)
    # new operand values in the same buffers: the graph reads them on replay
    a2, b2 = random_operands(rng, dt, B, N, K, M, -9, 10)
    A.copy_(dev(a2))
    Bm.copy_(dev(b2))
    graph.replay()
    torch.cuda.synchronize()
    if np.dtype(dt).kind in "iu":
        assert np.array_equal(host(out), oracle.matmul(a2, b2))
    else:
        want = np.matmul(a2.astype(np.float64), b2.astype(np.float64))
        assert rel_to_max(host(out), want) <= (1e-5 if dt == np.float32 else 1e-12)
    ttb.check_device(0)


def test_streamk_shape_replays_correctly(ttb, reset_options):
    """512 x 512 x 8192: sixteen tiles with 256 K blocks each -- stream-K when launched directly."""
    rng = np.random.default_rng(81)
    a, b = random_operands(rng, np.float32, 1, 512, 8192, 512)
    A, Bm = dev(a), dev(b)
    out = torch.zeros((1, 512, 512), device="cuda")
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    graph = _capture(lambda: ttb.batched_matmul(A, Bm, out=out))
    for _ in range(4):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert rel_to_max(host(out), want) <= 1e-5
    ttb.check_device(0)
