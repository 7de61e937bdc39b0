"""Multi-GPU parity of the partitioner on real devices (skipped with fewer than two GPUs):
one process per GPU over NCCL.  The column-block product with the all-gather fused into the
GEMM kernel (three ways to reach the peers, bit-identical to each other) and the NCCL all-gather
form are checked on EVERY rank against a float64 product (the f32 gate, 1e-5 of max|C|) and
against each other; back-to-back fused products with changing operands and a read of C between
them, with no host-side synchronisation, must each be right (the cross-rank ordering rule of
ShardedMatmul); batch-sharded products (configurations 3 and 5 included) must equal the
unsharded ones and the oracle; a tensor moved between two GPUs arrives intact."""
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
        # "paired": at two ranks a block of 100 pair tiles with 128 K blocks each -- every tile is cut
        # and every unit's range is longer than a tile, so the fused kernel pairs its units (odd ones
        # walk their range backwards, the two that share a tile settle by ticket which one stores)
        for name, (n, k, m) in {"square": (1024, 512, 1024), "ragged": (1000, 520, 1300),
                                "many_tiles": (4096, 256, 8192), "paired": (2560, 4096, 5120)}.items():
            A = torch.randn((1, n, k), generator=g, device=dev)
            B = torch.randn((1, k, m), generator=g, device=dev)
            full = ttb.batched_matmul(A, B)
            want64 = torch.matmul(A.double(), B.double())
            gate = lambda x: bool(float((x.double() - want64).abs().max() / want64.abs().max()) <= 1e-5)
            fused = ttb.ShardedMatmul(exchange="peer")
            C = fused.symmetric_output((1, n, m), torch.float32, dev)
            C.fill_(float("nan"))
            torch.cuda.synchronize()
            dist.barrier()
            # a shard's K blocks may be dealt out differently from the full product's (stream-K),
            # so sums associate differently: equal to within a few ulp of max|C|, not bit-equal
            close = lambda x: bool(float((x - full).abs().max() / full.abs().max()) <= 2e-6)
            got = fused(A, B, out=C)
            results[f"{name}_fused"] = close(got)
            results[f"{name}_fused_vs_float64"] = gate(got)
            plain = ttb.ShardedMatmul()
            got = plain(A, B)
            results[f"{name}_nccl"] = close(got)
            results[f"{name}_nccl_vs_float64"] = gate(got)
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
            if fused.multicast_available(C) and m % (4 * world) == 0:
                fused.exchange = "multicast"
                C.fill_(float("nan"))
                torch.cuda.synchronize()
                dist.barrier()
                results[f"{name}_fused_multicast_eq_tensor_stores"] = bool(torch.equal(fused(A, B, out=C), ref))
                fused.exchange = "peer"
                results["multicast_available"] = True
        # Back-to-back fused products, different operands every time, C read between the calls by
        # work on the same stream, no host-side synchronisation and no process-group barrier: one
        # buffer (a barrier goes in front of each rewrite) and two buffers used in turn.
        n, k, m = 1024, 384, 2048
        steps = 6
        As = [torch.randn((1, n, k), generator=g, device=dev) for _ in range(steps)]
        Bs = [torch.randn((1, k, m), generator=g, device=dev) for _ in range(steps)]
        wants = [torch.matmul(a.double(), b.double()) for a, b in zip(As, Bs)]
        for label, nbuf in (("one_buffer", 1), ("two_buffers", 2)):
            sm = ttb.ShardedMatmul(exchange="peer")
            bufs = [sm.symmetric_output((1, n, m), torch.float32, dev) for _ in range(nbuf)]
            errs = torch.zeros(steps, dtype=torch.float64, device=dev)
            torch.cuda.synchronize()
            dist.barrier()
            for i in range(steps):
                c = sm(As[i], Bs[i], out=bufs[i % nbuf])
                # the consumer: a full read of this rank's C, enqueued on the same stream
                errs[i] = (c.double() - wants[i]).abs().max() / wants[i].abs().max()
                if rank == i % world:
                    torch.cuda._sleep(2_000_000)   # one rank lags behind: the others must not overwrite what it reads
            torch.cuda.synchronize()
            results[f"back_to_back_{label}"] = bool(float(errs.max()) <= 1e-5)
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
        # configurations 3 and 5 sharded over the batch dim: seeded operands as the reference draws
        # them, this rank's share against the oracle (f32 within the gate, i32 bit-exact)
        sys.path.insert(0, str(ROOT / "tests"))
        import numpy as np
        import oracle_lib

        o = oracle_lib.load()
        p3 = ttb.partition(256, 128, 64, 128, world, rank)
        ops = ttb.config_operands("c3", batch_range=(p3.begin, p3.end))
        Qd, Kd, Vd = (torch.from_numpy(ops[k]).to(dev) for k in ("Q", "K", "V"))
        S = ttb.batched_matmul(Qd, Kd.permute(0, 2, 1))
        O = ttb.batched_matmul(S, Vd)
        s64 = np.matmul(ops["Q"].astype(np.float64), ops["K"].astype(np.float64).transpose(0, 2, 1))
        o64 = np.matmul(S.cpu().numpy().astype(np.float64), ops["V"].astype(np.float64))
        results["c3_shard_qk"] = bool(np.abs(S.cpu().numpy() - s64).max() / np.abs(s64).max() <= 1e-5)
        results["c3_shard_sv"] = bool(np.abs(O.cpu().numpy() - o64).max() / np.abs(o64).max() <= 1e-5)
        p5 = ttb.partition(64, 1024, 512, 1024, world, rank)
        nb = min(p5.end - p5.begin, 2)   # two batches of the share: the oracle is a CPU loop
        ops = ttb.config_operands("c5", batch_range=(p5.begin, p5.begin + nb))
        got = ttb.batched_matmul(torch.from_numpy(ops["A"]).to(dev), torch.from_numpy(ops["B"]).to(dev))
        results["c5_shard_bit_exact"] = bool(np.array_equal(got.cpu().numpy(), o.matmul(ops["A"], ops["B"])))
        # the host-buffer form of the column split: every rank uploads its rows of lhs and its block of rhs
        fullA = torch.randn((1000, 520), generator=torch.Generator().manual_seed(5))
        fullB = torch.randn((520, 1300), generator=torch.Generator().manual_seed(6))
        sm = ttb.ShardedMatmul()
        (r0, r1), (c0, c1) = sm.host_shards(1000, 520, 1300)
        hA = fullA[r0:r1].contiguous().pin_memory()
        hB = fullB[:, c0:c1].contiguous().pin_memory()
        hC = torch.zeros((1000, c1 - c0)).pin_memory()
        sm.columns_from_host(hA, hB, hC, 1000)
        want = torch.matmul(fullA.double(), fullB.double())[:, c0:c1]
        results["columns_from_host"] = bool(c1 == c0 or float((hC.double() - want).abs().max() / want.abs().max()) <= 1e-5)
        # Tensor::to(Device) between two GPUs as one peer copy
        src = torch.randn((3, 1000, 77), generator=g, device=dev)[:, ::2]
        peer = (rank + 1) % world
        moved = ttb.to_device(src, peer)
        results["to_device"] = bool(moved.device.index == peer and torch.equal(moved.cpu(), src.cpu()))
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
