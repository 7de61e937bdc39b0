"""ShardedMatmul.host_shards on CPU: how the host-resident operands of one column-sharded product
are cut over the ranks (rows of lhs for the upload + all-gather, columns of rhs / out for the
product).  For every world size the row ranges tile [0, N) and the column ranges tile [0, M)
exactly, in rank order, ragged sizes included; column blocks start on the partitioner's alignment."""
import pytest

import tinytensor_b200 as ttb


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("N,K,M", [(8192, 8192, 8192), (1000, 520, 1300), (5, 7, 3), (129, 64, 257), (4096, 784, 10)])
def test_host_shards_tile_rows_and_columns(world, N, K, M):
    sm = ttb.ShardedMatmul(local_matmul=lambda a, b, o: None)
    sm.world = world
    rows, cols = [], []
    for rank in range(world):
        sm.rank = rank
        (r0, r1), (c0, c1) = sm.host_shards(N, K, M)
        assert 0 <= r0 <= r1 <= N and 0 <= c0 <= c1 <= M
        part = ttb.partition(1, N, K, M, world, rank)
        assert (c0, c1) == (part.begin, part.end)      # the product's own split
        rows.append((r0, r1))
        cols.append((c0, c1))
    for ranges, extent in ((rows, N), (cols, M)):
        assert ranges[0][0] == 0 and ranges[-1][1] == extent
        for (a0, a1), (b0, b1) in zip(ranges, ranges[1:]):
            assert a1 == b0                              # contiguous, in rank order, no overlap
    # every rank's row count is the same except for the tail (the all-gather buffer is world x rows)
    per = -(-N // world)
    assert all(r1 - r0 in (per, max(0, N - per * i)) or r1 - r0 <= per for i, (r0, r1) in enumerate(rows))
