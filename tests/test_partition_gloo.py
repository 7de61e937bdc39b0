"""The N>1 host path on CPU: two gloo ranks run the partitioner with the oracle standing
in for the per-rank CUDA product, and must reassemble exactly the single-process result."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, q):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle_lib
        import tinytensor_b200 as ttb

        o = oracle_lib.load()

        def local(a, b, out):
            out.copy_(torch.from_numpy(o.matmul(a.numpy(), b.numpy())))

        B, N, K, M, dtype = case
        g = torch.Generator().manual_seed(1234)
        if dtype == "i32":
            lhs = torch.randint(-8, 9, (B, N, K), generator=g, dtype=torch.int32)
            rhs = torch.randint(-8, 9, (B, K, M), generator=g, dtype=torch.int32)
        else:
            lhs = torch.randn((B, N, K), generator=g, dtype=torch.float32)
            rhs = torch.randn((B, K, M), generator=g, dtype=torch.float32)
        sm = ttb.ShardedMatmul(local_matmul=local)
        part = sm.plan(lhs, rhs)
        got = sm(lhs, rhs)
        want = torch.from_numpy(o.matmul(lhs.numpy(), rhs.numpy()))
        # also the non-gathered form: a rank holds only its own share
        mine = sm(lhs, rhs, gather=False)
        if part.kind == "batch":
            own_ok = torch.equal(mine, want[part.begin:part.end])
        else:
            own_ok = torch.equal(mine[:, :, part.begin:part.end], want[:, :, part.begin:part.end])
        q.put((rank, part.kind, part.begin, part.end, torch.equal(got, want), own_ok))
    finally:
        dist.destroy_process_group()


CASES = [
    (6, 33, 70, 41, "i32"),      # batch sharding, even split
    (5, 33, 70, 41, "f32"),      # batch sharding, uneven split (3 + 2)
    (1, 50, 64, 512, "i32"),     # column blocks, even (256 + 256)
    (1, 50, 64, 300, "f32"),     # column blocks, uneven (256 + 44)
    (1, 50, 64, 100, "i32"),     # fewer 128-column units than ranks: rank 1 gets nothing
]


@pytest.mark.parametrize("case", CASES)
def test_two_rank_partitioner_matches_single_process(case):
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, case, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    results.sort()
    kinds = {r[1] for r in results}
    assert kinds == {"batch" if case[0] > 1 else "columns"}
    # ranges tile the sharded dim
    assert results[0][2] == 0 and results[0][3] == results[1][2]
    assert results[1][3] == (case[0] if case[0] > 1 else case[3])
    assert all(r[4] for r in results), "gathered result differs from the single-process product"
    assert all(r[5] for r in results), "a rank's own share differs"
