"""Multi-GPU parity of the partitioner on real devices (skipped with fewer than two GPUs):
one process per GPU over NCCL.  The column-block product with the all-gather fused into the
GEMM kernel (three ways to reach the peers, bit-identical to each other) and the NCCL all-gather
form must agree with each other and with the single-GPU product to a few ulp of max|C|;
batch-sharded products must equal the unsharded ones."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    results = {}
    try:
        import tinytensor_b200 as ttb

        g = torch.Generator(device=dev).manual_seed(7)
        # column blocks: f32 (fused and NCCL exchange), ragged sizes included
        # "many_tiles": every CTA pair works through several tiles, so the tile-by-tile forwarding and
        # the jointly forwarded last tile are both exercised
        for name, (n, k, m) in {"square": (1024, 512, 1024), "ragged": (1000, 520, 1300),
                                "many_tiles": (4096, 256, 8192)}.items():
            A = torch.randn((1, n, k), generator=g, device=dev)
            B = torch.randn((1, k, m), generator=g, device=dev)
            full = ttb.batched_matmul(A, B)
            fused = ttb.ShardedMatmul(exchange="peer")
            C = fused.symmetric_output((1, n, m), torch.float32, dev)
            C.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            # a shard's K blocks may be dealt out differently from the full product's (stream-K),
            # so sums associate differently: equal to within a few ulp of max|C|, not bit-equal
            close = lambda x: bool(float((x - full).abs().max() / full.abs().max()) <= 2e-6)
            results[f"{name}_fused"] = close(fused(A, B, out=C))
            plain = ttb.ShardedMatmul()
            results[f"{name}_nccl"] = close(plain(A, B))
            # The fused kernel cuts K differently from the plain one (its tiles are made to finish
            # evenly over time, see the kernel), so the two forms agree to rounding, not bit for
            # bit; the three ways the fused kernel can reach the peers deliver the very same sums.
            ref = fused(A, B, out=C).clone()
            results[f"{name}_fused_vs_nccl"] = bool(float((ref - plain(A, B)).abs().max() / full.abs().max()) <= 2e-6)
            # forwarding warps instead of the epilogue's bulk tensor stores
            ttb.set_option("peer_tma", 0)
            C.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            results[f"{name}_fused_forwarding_warps_eq_tensor_stores"] = bool(torch.equal(fused(A, B, out=C), ref))
            ttb.set_option("peer_tma", 1)
            # through NVSwitch multicast (one multimem store per tile), where the symmetric
            # buffer has a multicast mapping
            if getattr(fused._symm[1], "has_multicast_support", False) and m % (4 * world) == 0:
                fused.exchange = "multicast"
                C.fill_(float("nan"))
                torch.cuda.synchronize()
                dist.barrier()
                results[f"{name}_fused_multicast_eq_tensor_stores"] = bool(torch.equal(fused(A, B, out=C), ref))
                fused.exchange = "peer"
                results["multicast_available"] = True
        # column blocks, integer dtype: goes through the NCCL exchange, bit-exact
        Ai = torch.randint(-8, 9, (1, 300, 128), generator=g, device=dev, dtype=torch.int32)
        Bi = torch.randint(-8, 9, (1, 128, 512), generator=g, device=dev, dtype=torch.int32)
        results["i32_columns"] = bool(torch.equal(ttb.ShardedMatmul()(Ai, Bi), ttb.batched_matmul(Ai, Bi)))
        # batch sharding: no exchange unless asked for
        Q = torch.randn((16, 128, 64), generator=g, device=dev)
        K = torch.randn((16, 128, 64), generator=g, device=dev)
        sm = ttb.ShardedMatmul()
        want = ttb.batched_matmul(Q, K.permute(0, 2, 1))
        part = sm.plan(Q, K.permute(0, 2, 1))
        own = sm(Q, K.permute(0, 2, 1), gather=False)
        results["batch_own"] = bool(torch.equal(own, want[part.begin:part.end]))
        results["batch_gather"] = bool(torch.equal(sm(Q, K.permute(0, 2, 1)), want))
        ttb.check_device(rank)
        torch.cuda.synchronize()
    except Exception as e:  # report instead of hanging the parent
        results["exception"] = repr(e)
    finally:
        q.put((rank, results))
        dist.destroy_process_group()


def test_partitioner_on_two_or_more_gpus():
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = [q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, res in got:
        assert "exception" not in res, (rank, res["exception"])
        bad = [k for k, v in res.items() if v is not True]
        assert not bad, (rank, bad)
