"""GPU parity tests of conv2d forward / backward (ttb_conv2d_forward / ttb_conv2d_backward), the
other caller of the reference's matmul kernel (backend/cuda/conv.cu:149-160, :324-362).

The oracle (oracle/conv_oracle.c) restates the reference's CPU runner and is pinned against the
reference's own kernels and test data by tests/test_oracle_conv.py.  Integers must match it bit
for bit; f32 within 1e-5 and f64 within 1e-12 of a float64 / long-double result, relative to the
largest magnitude, as for matmul.  Cases: the reference's tests/test_conv.cpp:99-183 and
tests/test_conv_autograd.cpp:43-107, plus ragged / strided / padded geometries and the chunked
path."""
import numpy as np
import pytest
import torch

import oracle_lib
import refcases
from gpu_util import dev, host, rel_to_max

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5
F64_TOL = 1e-12


def _iota(shape, dt):
    return (np.arange(int(np.prod(shape))) % 10).astype(dt).reshape(shape)


def _draw(rng, dt, shape, ints=(-5, 6)):
    if np.dtype(dt).kind in "iu":
        return rng.integers(ints[0], ints[1], shape).astype(dt)
    return rng.standard_normal(shape).astype(dt)


def _close(got, want, dt):
    if np.dtype(dt).kind in "iu":
        assert got.dtype == np.dtype(dt) and np.array_equal(got, want)
    else:
        wide = np.float64 if np.dtype(dt) == np.float32 else np.longdouble
        assert rel_to_max(got, want.astype(wide)) <= (F32_TOL if np.dtype(dt) == np.float32 else F64_TOL)


@pytest.mark.parametrize("dt", refcases.DTYPES)
@pytest.mark.parametrize("stride,padding", [(1, 0), (2, 1)])
def test_reference_forward_cases(ttb, oracle, dt, stride, padding):
    """tests/test_conv.cpp:99-145: i % 10 data, every dtype; exact for floats too (small integers)."""
    x, w = _iota((4, 3, 64, 64), dt), _iota((128, 3, 3, 3), dt)
    got = host(ttb.conv2d(dev(x), dev(w), None, stride, padding))
    want = oracle.conv2d_forward(x, w, None, stride, padding)
    assert got.shape == want.shape and np.array_equal(got, want)
    assert np.array_equal(got, oracle_lib.conv2d_direct(x, w, stride, padding).astype(dt))


def test_reference_forward_with_bias_f32(ttb, oracle):
    """tests/test_conv.cpp:147-183: integers in [-5, 5] as f32, bias, 68x28, stride 2, padding 1."""
    rng = np.random.default_rng(60)
    x, w, b = (_draw(rng, np.int32, s).astype(np.float32) for s in ((4, 3, 68, 28), (128, 3, 3, 3), (128,)))
    got = host(ttb.conv2d(dev(x), dev(w), dev(b), 2, 1))
    want = oracle.conv2d_forward(x, w, b, 2, 1)
    assert np.abs(got - want).max() <= 1e-6  # the reference test's atol; exact here


@pytest.mark.parametrize("dt", refcases.DTYPES)
@pytest.mark.parametrize("geom", [
    dict(B=3, C_in=5, C_out=20, H=19, W=14, K=3, S=1, P=0),
    dict(B=2, C_in=4, C_out=33, H=17, W=23, K=5, S=2, P=2),
    dict(B=2, C_in=8, C_out=16, H=12, W=12, K=1, S=1, P=0),
    dict(B=1, C_in=2, C_out=7, H=9, W=31, K=3, S=3, P=1),
    dict(B=2, C_in=3, C_out=6, H=6, W=6, K=6, S=1, P=0),   # kernel == image: one output pixel
])
def test_forward_and_backward_random(ttb, oracle, dt, geom):
    rng = np.random.default_rng(61)
    g = geom
    x = _draw(rng, dt, (g["B"], g["C_in"], g["H"], g["W"]))
    w = _draw(rng, dt, (g["C_out"], g["C_in"], g["K"], g["K"]))
    b = _draw(rng, dt, (g["C_out"],))
    y = host(ttb.conv2d(dev(x), dev(w), dev(b), g["S"], g["P"]))
    _close(y, oracle.conv2d_forward(x, w, b, g["S"], g["P"]), dt)
    go = _draw(rng, dt, y.shape)
    gx, gw, gb = ttb.conv2d_backward(dev(go), dev(x), dev(w), g["S"], g["P"])
    ox, ow, ob = oracle.conv2d_backward(go, x, w, g["S"], g["P"])
    _close(host(gx), ox, dt)
    _close(host(gw), ow, dt)
    _close(host(gb), ob, dt)


def test_reference_autograd_case_f64(ttb, oracle):
    """tests/test_conv_autograd.cpp:43-107: f64, B=4, C_in=3, C_out=64, 38x28, K=3, S=2, P=1;
    the reference accepts atol 1e-4 against torch, here the f64 gate applies."""
    rng = np.random.default_rng(62)
    x, w, b = (_draw(rng, np.int32, s).astype(np.float64) for s in ((4, 3, 38, 28), (64, 3, 3, 3), (64,)))
    y = ttb.conv2d(dev(x), dev(w), dev(b), 2, 1)
    go = _draw(rng, np.int32, tuple(y.shape)).astype(np.float64)
    gx, gw, gb = ttb.conv2d_backward(dev(go), dev(x), dev(w), 2, 1)
    ox, ow, ob = oracle.conv2d_backward(go, x, w, 2, 1)
    for got, want in ((gx, ox), (gw, ow), (gb, ob)):
        assert np.abs(host(got) - want).max() <= 1e-4
        _close(host(got), want, np.float64)


@pytest.mark.parametrize("dt", [np.float32, np.float64, np.int32])
def test_layer_sized_case(ttb, oracle, dt):
    """A ResNet-style layer: 32 -> 64 channels, 28x28, 3x3, padding 1 -- big enough for the
    tensor-core kernels (f32: K = 288 for forward, 784 for grad_w, 64 for grad_x)."""
    rng = np.random.default_rng(63)
    x, w, b = _draw(rng, dt, (4, 32, 28, 28)), _draw(rng, dt, (64, 32, 3, 3)), _draw(rng, dt, (64,))
    y = host(ttb.conv2d(dev(x), dev(w), dev(b), 1, 1))
    if dt == np.float32:
        assert ttb.last_variant().name.startswith("TCGEN05")
    _close(y, oracle.conv2d_forward(x, w, b, 1, 1), dt)
    go = _draw(rng, dt, y.shape)
    gx, gw, gb = ttb.conv2d_backward(dev(go), dev(x), dev(w), 1, 1)
    ox, ow, ob = oracle.conv2d_backward(go, x, w, 1, 1)
    _close(host(gx), ox, dt)
    _close(host(gw), ow, dt)
    _close(host(gb), ob, dt)


def test_chunked_batches_match_one_pass(ttb, oracle, reset_options):
    """A 1 MiB columns budget forces groups of batch items (and accumulation of grad_w across
    groups); results equal the one-pass run bit for bit for integers."""
    rng = np.random.default_rng(64)
    x, w, b = _draw(rng, np.int32, (7, 6, 40, 40)), _draw(rng, np.int32, (10, 6, 3, 3)), _draw(rng, np.int32, (10,))
    go_shape = (7, 10, 38, 38)
    go = _draw(rng, np.int32, go_shape)
    ttb.set_option("conv_columns_mb", 1)  # 54 x 1472 x 4 B = 318 KB per item: 3 items per group
    y = host(ttb.conv2d(dev(x), dev(w), dev(b), 1, 0))
    gx, gw, gb = (host(t) for t in ttb.conv2d_backward(dev(go), dev(x), dev(w), 1, 0))
    assert np.array_equal(y, oracle.conv2d_forward(x, w, b, 1, 0))
    ox, ow, ob = oracle.conv2d_backward(go, x, w, 1, 0)
    assert np.array_equal(gx, ox) and np.array_equal(gw, ow) and np.array_equal(gb, ob)


def test_bad_arguments_raise(ttb):
    x = torch.ones(1, 3, 8, 8, device="cuda")
    with pytest.raises(ttb.TTBError):
        ttb.conv2d(x, torch.ones(4, 2, 3, 3, device="cuda"))          # channels differ
    with pytest.raises(ttb.TTBError):
        ttb.conv2d(x, torch.ones(4, 3, 3, 2, device="cuda"))          # kernel not square
    with pytest.raises(ttb.TTBError):
        ttb.conv2d(x, torch.ones(4, 3, 9, 9, device="cuda"))          # kernel larger than the image
    with pytest.raises(ttb.TTBError):
        ttb.conv2d(x, torch.ones(4, 3, 3, 3, device="cuda"), None, 0, 0)  # stride 0
    with pytest.raises(ttb.TTBError):
        ttb.conv2d(x, torch.ones(4, 3, 3, 3, device="cuda", dtype=torch.float64))
