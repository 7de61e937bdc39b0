"""bench.py's multi-rank bookkeeping on CPU (two gloo ranks): numbers that decide how many steps a
rank runs must agree between the ranks, whatever each rank measured by itself."""
import os
import socket
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, str(ROOT))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import bench

        # the two ranks measured step times that round to different counts (1265 and 1264)
        mine = 1.7380 if rank == 0 else 1.7395
        alone = bench.sustained_step_count(mine, 20, torch)
        agreed = bench.sustained_step_count(mine, 20, torch, dist, torch.device("cpu"))
        q.put((rank, alone, agreed))
    finally:
        dist.destroy_process_group()


def test_sustained_step_count_is_the_same_on_every_rank():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    (_, alone0, agreed0), (_, alone1, agreed1) = got
    assert alone0 != alone1          # by themselves the ranks would disagree ...
    assert agreed0 == agreed1        # ... together they do not
    assert agreed0 == min(alone0, alone1)   # the slowest rank's time decides
