"""The gradients of matmul, as tinytensor's autograd obtains them from the same backend
operator: grad_lhs = grad . rhs^T and grad_rhs = lhs^T . grad on permuted views
(autograd/binary_ops.cpp:172-179).  Mirrors tests/test_matmul_autograd.cpp:43-261: the five rank
forms, f64, integers in [-5, 5] as data (its rand_vec), sizes 2048, 379 x 635 and the batched
case; the reference compares with torch at atol 1e-4 .. 1e-6, here the gradients are compared
with their definition under the f64 gate (1e-12 of the largest magnitude), and for f32 / i32
under the gates of those dtypes."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host, rel_to_max

pytestmark = pytest.mark.gpu

N, M, K, B = 256 + 123, 512 + 123, 128 + 19, 5

FORMS = {
    "dot": ((2048,), (2048,), ()),
    "vector-matrix": ((N,), (N, M), (M,)),
    "matrix-vector": ((N, M), (M,), (N,)),
    "matrix-matrix": ((N, K), (K, M), (N, M)),
    "batched": ((B, N, K), (B, K, M), (B, N, M)),
}


def _definition(l, r, g):
    """Gradients from the definition, in wide precision, shaped like the operands."""
    wide = np.longdouble if l.dtype == np.float64 else np.float64
    l3 = l.astype(wide).reshape((1, 1, -1) if l.ndim == 1 else ((1,) + l.shape if l.ndim == 2 else l.shape))
    r3 = r.astype(wide).reshape((1, -1, 1) if r.ndim == 1 else ((1,) + r.shape if r.ndim == 2 else r.shape))
    g3 = g.astype(wide).reshape((l3.shape[0], l3.shape[1], r3.shape[2]))
    gl = np.matmul(g3, r3.transpose(0, 2, 1)).reshape(l.shape)
    gr = np.matmul(l3.transpose(0, 2, 1), g3).reshape(r.shape)
    return gl, gr


@pytest.mark.parametrize("dt", [np.float64, np.float32, np.int32])
@pytest.mark.parametrize("form", list(FORMS))
def test_gradients_match_their_definition(ttb, dt, form):
    rng = np.random.default_rng(100)
    ls, rs, gs = FORMS[form]
    draw = lambda s: rng.integers(-5, 6, s).astype(dt)
    l, r = draw(ls), draw(rs)
    g = draw(gs if gs else (1,))
    out = ttb.matmul(dev(l), dev(r))
    assert tuple(out.shape) == (gs if gs else (1,))  # the reference's dot product is flattened to [1]
    gl, gr = ttb.matmul_backward(dev(l), dev(r), dev(g))
    want_l, want_r = _definition(l, r, g)
    assert tuple(gl.shape) == l.shape and tuple(gr.shape) == r.shape
    if np.dtype(dt).kind == "i":
        assert np.array_equal(host(gl), want_l.astype(np.int64).astype(dt))
        assert np.array_equal(host(gr), want_r.astype(np.int64).astype(dt))
    else:
        tol = 1e-12 if dt == np.float64 else 1e-5
        assert rel_to_max(host(gl), want_l) <= tol
        assert rel_to_max(host(gr), want_r) <= tol
        assert np.abs(host(gl) - want_l).max() <= 1e-4 and np.abs(host(gr) - want_r).max() <= 1e-4


def test_gradients_of_strided_operands(ttb):
    """Operands that are themselves views (a sliced weight, a transposed activation): backward
    permutes them again; nothing is cloned on the way."""
    rng = np.random.default_rng(101)
    big = rng.standard_normal((2, 300, 260))
    l_t = dev(big)[:, 10:210, 4:260:2]                      # [2, 200, 128], strides (78000, 260, 2)
    r_t = dev(rng.standard_normal((2, 96, 128))).permute(0, 2, 1)  # [2, 128, 96] stored transposed
    g = rng.standard_normal((2, 200, 96))
    gl, gr = ttb.matmul_backward(l_t, r_t, dev(g))
    want_l, want_r = _definition(host(l_t), host(r_t), g)
    assert rel_to_max(host(gl), want_l) <= 1e-12 and rel_to_max(host(gr), want_r) <= 1e-12


def test_bad_grad_shape_raises(ttb):
    a = torch.ones(4, 5, device="cuda")
    with pytest.raises(ttb.TTBError):
        ttb.matmul_backward(a, torch.ones(5, 6, device="cuda"), torch.ones(4, 7, device="cuda"))
