"""GPU parity tests of the streaming kernels for products with one tiny dim (classifier heads
and their gradients: BASELINE config 2's H.W2^T, dC.W2, H^T.dC), every dtype, against the oracle.
Automatic dispatch must pick them (variant SIMT_SKINNY) and results must meet the same gates as
every other kernel: integers bit for bit, f32 1e-5, f64 1e-12."""
import numpy as np
import pytest
import torch

import refcases
from gpu_util import dev, host, random_operands, rel_to_max

pytestmark = pytest.mark.gpu


def _check(got, a, b, oracle, addend=None):
    dt = a.dtype
    if dt.kind in "iu":
        want = oracle.matmul(a, b)
        if addend is not None:
            want = (want.astype(np.int64) + addend).astype(dt) if dt != np.int64 else want + addend
        assert got.dtype == dt and np.array_equal(got, want)
    else:
        wide = np.float64 if dt == np.float32 else np.longdouble
        want = np.matmul(a.astype(wide), b.astype(wide))
        if addend is not None:
            want = want + addend
        assert rel_to_max(got, want) <= (1e-5 if dt == np.float32 else 1e-12)


SHAPES = {
    "row_dot (M tiny, lhs rows along K)": (2, 300, 700, 10),
    "row_dot ragged": (1, 33, 65, 1),
    "outer (K tiny)": (2, 200, 10, 300),
    "outer ragged": (1, 77, 3, 35),
    "tiny N (transposed roles)": (2, 10, 700, 300),
    "vec.mat": (1, 1, 513, 260),
}


@pytest.mark.parametrize("dt", refcases.DTYPES)
@pytest.mark.parametrize("name", list(SHAPES))
def test_contiguous_operands(ttb, oracle, dt, name):
    rng = np.random.default_rng(90)
    B, N, K, M = SHAPES[name]
    a, b = random_operands(rng, dt, B, N, K, M, -9, 10)
    got = host(ttb.batched_matmul(dev(a), dev(b)))
    assert ttb.last_variant() == ttb.Variant.SIMT_SKINNY, name
    _check(got, a, b, oracle)


@pytest.mark.parametrize("dt", [np.float32, np.int32, np.float64, np.uint8])
def test_config2_skinny_products_as_views(ttb, oracle, dt):
    """The three skinny products of config 2 with the views autograd produces:
    H.W2^T (rhs a permuted view), dC.W2, H^T.dC (lhs a permuted view -> col_stream + split K)."""
    rng = np.random.default_rng(91)
    H = random_operands(rng, dt, 1, 1024, 512, 1, -9, 10)[0]          # [1, 1024, 512]
    W2 = random_operands(rng, dt, 1, 10, 512, 1, -9, 10)[0]           # [1, 10, 512]
    dC = random_operands(rng, dt, 1, 1024, 10, 1, -9, 10)[0]          # [1, 1024, 10]
    dH, dW2, ddC = dev(H), dev(W2), dev(dC)
    got = host(ttb.batched_matmul(dH, dW2.permute(0, 2, 1)))
    assert ttb.last_variant() == ttb.Variant.SIMT_SKINNY
    _check(got, H, W2.transpose(0, 2, 1), oracle)
    got = host(ttb.batched_matmul(ddC, dW2))
    assert ttb.last_variant() == ttb.Variant.SIMT_SKINNY
    _check(got, dC, W2, oracle)
    got = host(ttb.batched_matmul(dH.permute(0, 2, 1), ddC))
    assert ttb.last_variant() == ttb.Variant.SIMT_SKINNY
    _check(got, H.transpose(0, 2, 1), dC, oracle)


def test_fused_addend_strided_output_and_broadcast(ttb, oracle):
    rng = np.random.default_rng(92)
    a, b = random_operands(rng, np.int32, 3, 150, 260, 7, -99, 100)
    bias = rng.integers(-1000, 1000, 7).astype(np.int32)
    got = host(ttb.batched_matmul_fused(dev(a), dev(b), dev(bias)))
    assert ttb.last_variant() == ttb.Variant.SIMT_SKINNY
    _check(got, a, b, oracle, bias)
    # accumulate in place into a strided destination, lhs batch-broadcast
    wide = torch.zeros((3, 150, 14), dtype=torch.int32, device="cuda")
    view = wide[:, :, ::2]
    start = rng.integers(-1000, 1000, (3, 150, 7)).astype(np.int32)
    view.copy_(dev(start))
    A1 = dev(a[:1]).expand(3, 150, 260)
    ttb.batched_matmul_fused(A1, dev(b), view, out=view)
    assert ttb.last_variant() == ttb.Variant.SIMT_SKINNY
    _check(host(view.contiguous()), np.broadcast_to(a[:1], a.shape), b, oracle, start)
    assert (wide[:, :, 1::2] == 0).all()
    # f32 with relu, K tiny
    x, w = random_operands(rng, np.float32, 1, 500, 10, 128)
    got = host(ttb.batched_matmul_fused(dev(x), dev(w), None, ttb.Activation.RELU))
    assert ttb.last_variant() == ttb.Variant.SIMT_SKINNY
    want = np.maximum(np.matmul(x.astype(np.float64), w.astype(np.float64)), 0)
    assert rel_to_max(got, want) <= 1e-5


def test_wraparound(ttb, oracle):
    rng = np.random.default_rng(93)
    for dt in (np.uint8, np.int16, np.int32, np.int64):
        info = np.iinfo(dt)
        a = rng.integers(info.min, info.max, (1, 64, 300), dtype=dt, endpoint=True)
        b = rng.integers(info.min, info.max, (1, 300, 5), dtype=dt, endpoint=True)
        got = host(ttb.batched_matmul(dev(a), dev(b)))
        assert ttb.last_variant() == ttb.Variant.SIMT_SKINNY
        assert np.array_equal(got, oracle.matmul(a, b))
