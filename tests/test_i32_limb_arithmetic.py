"""The arithmetic behind the i32 tensor-core kernel (tinytensor_b200/csrc/gemm_i32_tcgen05.cu),
restated in numpy: an int32 product mod 2^32 equals the shifted sum of the four byte-weight
accumulators P_s = sum_k sum_{i+j=s} a_i[k] b_j[k] of u8 x u8 products, each P_s itself only
known mod 2^32 (the tensor core's s32 accumulator wraps).  Compared with the oracle (the reference
CPU kernel's restatement), full-range values and long K included."""
import numpy as np
import pytest


def byte_planes(x: np.ndarray):
    u = x.astype(np.int32).view(np.uint32)
    return [((u >> (8 * i)) & 0xFF).astype(np.uint32) for i in range(4)]


def limb_product(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """a [N,K] . b [K,M] as the kernel forms it: ten plane products into four wrapping
    accumulators, combined with shifts.  uint32 arithmetic wraps like the s32 accumulator's bits."""
    ap, bp = byte_planes(a), byte_planes(b)
    acc = [np.zeros((a.shape[0], b.shape[1]), dtype=np.uint32) for _ in range(4)]
    pairs = 0
    with np.errstate(over="ignore"):
        for i in range(4):
            for j in range(4 - i):
                acc[i + j] += ap[i] @ bp[j]      # uint32 matmul: sums wrap mod 2^32
                pairs += 1
        assert pairs == 10
        c = acc[0] + (acc[1] << np.uint32(8)) + (acc[2] << np.uint32(16)) + (acc[3] << np.uint32(24))
    return c.view(np.int32)


def wrap_product(a, b):
    with np.errstate(over="ignore"):
        return (a.astype(np.int64).view(np.uint64) @ b.astype(np.int64).view(np.uint64)).astype(np.uint32).view(np.int32)


@pytest.mark.parametrize("shape", [(5, 7, 3), (33, 64, 20), (16, 1000, 9)])
def test_full_range_operands(oracle, shape):
    rng = np.random.default_rng(11)
    n, k, m = shape
    info = np.iinfo(np.int32)
    a = rng.integers(info.min, info.max, (n, k), dtype=np.int32, endpoint=True)
    b = rng.integers(info.min, info.max, (k, m), dtype=np.int32, endpoint=True)
    got = limb_product(a, b)
    assert np.array_equal(got, wrap_product(a, b))
    assert np.array_equal(got, oracle.matmul(a[None], b[None])[0])


def test_accumulators_that_wrap_many_times():
    """All bytes 0xFF over K = 70000: P_3 alone passes 2^32 more than once, the result is still exact."""
    k = 70000
    a = np.full((2, k), -1, dtype=np.int32)
    b = np.full((k, 3), -1, dtype=np.int32)
    assert 4 * 255 * 255 * k > 2 ** 32
    assert np.array_equal(limb_product(a, b), np.full((2, 3), k, dtype=np.int64).astype(np.int32))


def test_extremes():
    a = np.array([[np.iinfo(np.int32).min, np.iinfo(np.int32).max, -1, 0, 1]], dtype=np.int32)
    b = a.T.copy()
    assert np.array_equal(limb_product(a, b), wrap_product(a, b))
