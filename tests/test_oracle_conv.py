"""Pins the conv2d oracle (oracle/conv_oracle.c) -- CPU only.

1. Against the reference's own test data: tests/test_conv.cpp:99-145 builds X and W as
   `i % 10`, B=4, C_in=3, C_out=128, 64x64, K=3, (stride, padding) = (1, 0) and (2, 1), for every
   dtype but bool, and expects the direct 7-loop definition with accumulation in T
   (test_conv.cpp:28-73).  Integers must match bit for bit (u8 / i16 wrap), floats exactly too on
   this data (small integers).
2. Against the reference's own CPU kernels compiled into oracle/_ref/libttref_strict.so, on
   random data, forward and backward, bit for bit (same summation order; floating-point
   contraction off in both).
3. Backward against the definition of the gradients (float64 einsum)."""
import numpy as np
import pytest

import oracle_lib
import refcases


def _iota(shape, dt):
    n = int(np.prod(shape))
    return (np.arange(n) % 10).astype(dt).reshape(shape)


@pytest.mark.parametrize("dt", refcases.DTYPES)
@pytest.mark.parametrize("stride,padding", [(1, 0), (2, 1)])
def test_reference_forward_cases(oracle, dt, stride, padding):
    x = _iota((4, 3, 64, 64), dt)
    w = _iota((128, 3, 3, 3), dt)
    want = oracle_lib.conv2d_direct(x, w, stride, padding)
    got = oracle.conv2d_forward(x, w, None, stride, padding)
    assert got.shape == want.shape
    assert np.array_equal(got, want.astype(dt))
    if oracle.ref is not None:
        assert np.array_equal(oracle.conv2d_forward(x, w, None, stride, padding, which="ref"), got)


def _random_case(rng, dt, B=3, C_in=3, C_out=20, H=19, W=14, K=3):
    if np.dtype(dt).kind in "iu":
        draw = lambda s: rng.integers(-5, 6, s).astype(dt)  # the reference's rand_vec range (test_conv.cpp:86-95)
    else:
        draw = lambda s: rng.standard_normal(s).astype(dt)
    return draw((B, C_in, H, W)), draw((C_out, C_in, K, K)), draw((C_out,))


@pytest.mark.parametrize("dt", refcases.DTYPES)
@pytest.mark.parametrize("stride,padding", [(1, 0), (2, 1), (1, 2), (3, 1)])
def test_port_equals_reference_kernels(oracle, dt, stride, padding):
    if oracle.ref_strict is None:
        pytest.skip("oracle/_ref/libttref_strict.so not built (no reference tree at build time)")
    rng = np.random.default_rng(50)
    x, w, bias = _random_case(rng, dt)
    y = oracle.conv2d_forward(x, w, bias, stride, padding)
    assert np.array_equal(y, oracle.conv2d_forward(x, w, bias, stride, padding, which="ref_strict"))
    g = _random_case(rng, dt, B=y.shape[0], C_in=y.shape[1], H=y.shape[2], W=y.shape[3])[0]
    gx, gw, _ = oracle.conv2d_backward(g, x, w, stride, padding)
    rx, rw, _ = oracle.conv2d_backward(g, x, w, stride, padding, which="ref_strict")
    assert np.array_equal(gx, rx) and np.array_equal(gw, rw)


@pytest.mark.parametrize("stride,padding", [(1, 0), (2, 1), (1, 1)])
def test_backward_matches_gradient_definition(oracle, stride, padding):
    """tests/test_conv_autograd.cpp:43-107 checks the f64 gradients against torch; here the
    same quantities come from their definition."""
    rng = np.random.default_rng(51)
    x, w, _ = _random_case(rng, np.float64, B=4, C_in=3, C_out=16, H=38, W=28)
    K = w.shape[2]
    H_out = (x.shape[2] + 2 * padding - K) // stride + 1
    W_out = (x.shape[3] + 2 * padding - K) // stride + 1
    g = rng.standard_normal((4, 16, H_out, W_out))
    gx, gw, gb = oracle.conv2d_backward(g, x, w, stride, padding)
    xp = np.zeros((4, 3, x.shape[2] + 2 * padding, x.shape[3] + 2 * padding))
    xp[:, :, padding:padding + x.shape[2], padding:padding + x.shape[3]] = x
    want_gw = np.zeros_like(w)
    want_gxp = np.zeros_like(xp)
    for p in range(K):
        for q in range(K):
            sl = (slice(None), slice(None), slice(p, p + stride * (H_out - 1) + 1, stride),
                  slice(q, q + stride * (W_out - 1) + 1, stride))
            want_gw[:, :, p, q] = np.einsum("bmhw,bchw->mc", g, xp[sl])
            want_gxp[sl] += np.einsum("bmhw,mc->bchw", g, w[:, :, p, q])
    want_gx = want_gxp[:, :, padding:padding + x.shape[2], padding:padding + x.shape[3]]
    assert np.allclose(gw, want_gw, rtol=1e-12, atol=1e-11)
    assert np.allclose(gx, want_gx, rtol=1e-12, atol=1e-11)
    assert np.allclose(gb, g.sum(axis=(0, 2, 3)), rtol=1e-12, atol=1e-11)


def test_integer_bias_and_backward_wrap(oracle):
    rng = np.random.default_rng(52)
    x = rng.integers(0, 256, (2, 2, 9, 8)).astype(np.uint8)
    w = rng.integers(0, 256, (5, 2, 3, 3)).astype(np.uint8)
    bias = rng.integers(0, 256, 5).astype(np.uint8)
    y = oracle.conv2d_forward(x, w, bias, 1, 1)
    want = (oracle_lib.conv2d_direct(x, w, 1, 1).astype(np.uint64) + bias[None, :, None, None]).astype(np.uint8)
    assert np.array_equal(y, want)
    g = rng.integers(0, 256, y.shape).astype(np.uint8)
    _, _, gb = oracle.conv2d_backward(g, x, w, 1, 1)
    assert np.array_equal(gb, g.astype(np.uint64).sum(axis=(0, 2, 3)).astype(np.uint8))


GOLDEN = __import__("pathlib").Path(__file__).resolve().parent / "golden" / "conv_golden.npz"


def test_port_matches_golden_vectors(oracle):
    """tests/golden/conv_golden.npz holds outputs of the reference's own CPU conv2d kernels
    (made by tests/golden/make_golden_conv.py where the reference tree exists).  The C
    restatement must reproduce them bit for bit, forward and backward, for every dtype, also
    where oracle/_ref is absent."""
    data = np.load(GOLDEN)
    keys = sorted(k[:-5] for k in data.files if k.endswith("_geom"))
    assert len(keys) == 24
    for key in keys:
        s, p = (int(v) for v in data[key + "_geom"])
        x, w, bias = data[key + "_x"], data[key + "_w"], data[key + "_bias"]
        assert np.array_equal(oracle.conv2d_forward(x, w, bias, s, p), data[key + "_y"]), key
        gx, gw, _ = oracle.conv2d_backward(data[key + "_g"], x, w, s, p)
        assert np.array_equal(gx, data[key + "_gx"]) and np.array_equal(gw, data[key + "_gw"]), key
