"""GPU parity tests of the fused epilogue (ttb_batched_matmul_fused): act(lhs.rhs + addend).

What the reference does with separate kernels -- Linear's matmul + expand + add
(nn/linear.cpp:45-48), conv2d's per-channel bias add (backend/cuda/conv.cu:163-183), add_grad's
accumulation (tensor/tensor.cpp:1137-1160), relu (backend/common/kernel/unary.hpp:403-407) --
must come out the same from one kernel: integers bit for bit (wrap-around included), f32 within
1e-5 and f64 within 1e-12 of a wide-precision product plus addend."""
import numpy as np
import pytest
import torch

import refcases
from gpu_util import dev, host, random_operands, rel_to_max

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
F64_TOL = 1e-12


def _want(a, b, addend, relu):
    dt = a.dtype
    if dt.kind in "iu":
        full = refcases.expected(a, b)
        if addend is not None:
            full = (full + np.broadcast_to(addend, full.shape)).astype(dt)  # numpy integer add wraps
        return full
    wide = np.float64 if dt == np.float32 else np.longdouble
    full = np.matmul(a.astype(wide), b.astype(wide))
    if addend is not None:
        full = full + np.broadcast_to(addend, full.shape).astype(wide)
    if relu:
        full = np.maximum(full, 0)
    return full


def _check(got, want, dt):
    if np.dtype(dt).kind in "iu":
        assert got.dtype == np.dtype(dt)
        assert np.array_equal(got, want)
    else:
        assert rel_to_max(got, want) <= (F32_TOL if np.dtype(dt) == np.float32 else F64_TOL)


def _addends(rng, dt, B, N, M):
    """name -> numpy addend broadcastable to [B,N,M]."""
    def draw(shape):
        if np.dtype(dt).kind in "iu":
            info = np.iinfo(dt)
            return rng.integers(info.min // 2, info.max // 2, shape).astype(dt)
        return (rng.standard_normal(shape) * 3).astype(dt)
    return {"column bias": draw((M,)), "row bias": draw((N, 1)), "full": draw((B, N, M)),
            "per batch scalar": draw((B, 1, 1))}


@pytest.mark.parametrize("dt", refcases.DTYPES)
def test_addend_forms_small(ttb, dt):
    """Ragged shapes around the tile edges, every dtype, every broadcast form."""
    rng = np.random.default_rng(41)
    for (B, N, K, M) in ((2, 45, 70, 38), (1, 130, 129, 260), (3, 1, 33, 17)):
        a, b = random_operands(rng, dt, B, N, K, M, -9, 10)
        A, Bm = dev(a), dev(b)
        for name, add in _addends(rng, dt, B, N, M).items():
            got = host(ttb.batched_matmul_fused(A, Bm, dev(add)))
            _check(got, _want(a, b, add, False), dt)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_relu_and_bias(ttb, dt):
    rng = np.random.default_rng(42)
    a, b = random_operands(rng, dt, 2, 150, 96, 200)
    bias = rng.standard_normal(200).astype(dt)
    got = host(ttb.batched_matmul_fused(dev(a), dev(b), dev(bias), ttb.Activation.RELU))
    want = _want(a, b, bias, True)
    _check(got, want, dt)
    assert (got >= 0).all() and (got == 0).any() and (got > 0).any()
    # relu alone
    got = host(ttb.batched_matmul_fused(dev(a), dev(b), None, ttb.Activation.RELU))
    _check(got, _want(a, b, None, True), dt)


def test_relu_passes_nan_like_the_reference(ttb):
    """std::max(x, 0) returns x when x is NaN (the comparison is false)."""
    a = torch.ones(1, 32, 32, device="cuda")
    b = torch.ones(1, 32, 32, device="cuda")
    a[0, 3, 5] = float("nan")
    got = ttb.batched_matmul_fused(a, b, None, ttb.Activation.RELU)
    assert torch.isnan(got[0, 3]).all() and (got[0, 4] == 32).all()


def test_relu_on_integers_raises(ttb):
    a = torch.ones(1, 8, 8, dtype=torch.int32, device="cuda")
    with pytest.raises(ttb.TTBError):
        ttb.batched_matmul_fused(a, a, None, ttb.Activation.RELU)
    with pytest.raises(ttb.TTBError):
        ttb.batched_matmul_fused(a, a, torch.ones(1, 8, 9, dtype=torch.int32, device="cuda"))


@pytest.mark.parametrize("dt", [np.int32, np.uint8, np.int64, np.float32, np.float64])
def test_accumulate_in_place(ttb, dt):
    """addend == out: out += lhs.rhs, also into a strided destination."""
    rng = np.random.default_rng(43)
    B, N, K, M = 2, 140, 64, 150
    a, b = random_operands(rng, dt, B, N, K, M, -9, 10)
    start = _addends(rng, dt, B, N, M)["full"]
    C = dev(start.copy())
    ttb.batched_matmul_fused(dev(a), dev(b), C, out=C)
    _check(host(C), _want(a, b, start, False), dt)
    ttb.batched_matmul_fused(dev(a), dev(b), C, out=C)  # twice: 2 * product + start
    if np.dtype(dt).kind in "iu":
        want = (refcases.expected(a, b) * np.array(2, dtype=dt) + start).astype(dt)
        assert np.array_equal(host(C), want)
    wide = torch.zeros((B, N, 2 * M), dtype=C.dtype, device="cuda")
    view = wide[:, :, ::2]
    view.copy_(dev(start))
    ttb.batched_matmul_fused(dev(a), dev(b), view, out=view)
    _check(host(view.contiguous()), _want(a, b, start, False), dt)
    assert (wide[:, :, 1::2] == 0).all()


@pytest.mark.parametrize("variant", ["SIMT", "SIMT_SPLITK", "TCGEN05_3XTF32", "TCGEN05_2CTA"])
def test_f32_every_variant(ttb, variant, reset_options):
    """The addend and relu go through whichever kernel writes the final value: the plain SIMT
    store, the split-K reduction, the tensor-core epilogue (one CTA and CTA pairs)."""
    rng = np.random.default_rng(44)
    B, N, K, M = 1, 300, 1024, 520
    a, b = random_operands(rng, np.float32, B, N, K, M)
    ttb.set_option("force_variant", int(ttb.Variant[variant]))
    for name, add in _addends(rng, np.float32, B, N, M).items():
        got = host(ttb.batched_matmul_fused(dev(a), dev(b), dev(add), ttb.Activation.RELU))
        used = ttb.last_variant().name
        assert used == variant or (variant == "SIMT_SPLITK" and used == "SIMT")  # the split is a heuristic
        _check(got, _want(a, b, add, True), np.float32)


def test_f32_streamk_owner_adds(ttb, reset_options):
    """Stream-K: only the unit that owns a tile adds the addend, after the partial sums."""
    rng = np.random.default_rng(45)
    a, b = random_operands(rng, np.float32, 1, 512, 4096, 512)
    add = rng.standard_normal((512, 1)).astype(np.float32)
    ttb.set_option("streamk", 1)
    C = dev(rng.standard_normal((1, 512, 512)).astype(np.float32))
    start = host(C).copy()
    got = host(ttb.batched_matmul_fused(dev(a), dev(b), dev(add)))
    _check(got, _want(a, b, add, False), np.float32)
    ttb.batched_matmul_fused(dev(a), dev(b), C, out=C)
    _check(host(C), _want(a, b, start, False), np.float32)


@pytest.mark.parametrize("dt", [np.int32, np.float64])
def test_splitk_reduce_adds(ttb, dt, reset_options):
    rng = np.random.default_rng(46)
    a, b = random_operands(rng, dt, 1, 130, 4096, 10, -8, 9)
    add = _addends(rng, dt, 1, 130, 10)["column bias"]
    ttb.set_option("force_variant", int(ttb.Variant.SIMT_SPLITK))
    got = host(ttb.batched_matmul_fused(dev(a), dev(b), dev(add)))
    assert ttb.last_variant() == ttb.Variant.SIMT_SPLITK
    _check(got, _want(a, b, add, False), dt)


def test_linear_matches_reference_form(ttb):
    """Linear.forward: x[..., in] . W[in, out] + bias (nn/linear.cpp:41-50), any leading dims."""
    rng = np.random.default_rng(47)
    x = rng.standard_normal((4, 33, 96)).astype(np.float32)
    w = rng.standard_normal((96, 50)).astype(np.float32)
    bias = rng.standard_normal(50).astype(np.float32)
    got = host(ttb.linear(dev(x), dev(w), dev(bias)))
    want = x.astype(np.float64) @ w.astype(np.float64) + bias
    assert got.shape == (4, 33, 50)
    assert rel_to_max(got, want) <= F32_TOL
