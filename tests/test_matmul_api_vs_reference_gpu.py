"""tinytensor_b200.matmul / matmul_backward on the GPU against the reference's own compiled
tinytensor::matmul and Tensor::backward() (CPU backend): the golden fixture the reference library
produced (tests/golden/reference_api_golden.npz), and the library itself when it travelled
(oracle/_ref/libttref_full.so).  Covers what the kernels' own parity tests do not: result rank
and shape per rank form, the promoted dtype, and the gradients' layout for permuted views
(tests/test_matmul_autograd.cpp:43-261 exercises the same through torch)."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from gpu_util import dev, host, rel_to_max

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import ref_full  # noqa: E402
from make_reference_api_golden import FORMS, PROMOTIONS  # noqa: E402

pytestmark = pytest.mark.gpu
GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_api_golden.npz")
FORM_IDS = [f[0] for f in FORMS]


def _view(t, perm):
    return t.permute(*perm) if perm is not None else t


def _close(got, want):
    if want.dtype.kind in "iu":
        return np.array_equal(got, want)
    # both sides sum in the operands' precision, in different orders
    tol = 1e-5 if want.dtype == np.float32 else 1e-12
    return got.shape == want.shape and rel_to_max(got, want.astype(np.float64)) <= tol


@pytest.mark.parametrize("pair", PROMOTIONS, ids=[f"{np.dtype(a).name}-{np.dtype(b).name}" for a, b in PROMOTIONS])
@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
def test_values_shape_and_promoted_dtype(ttb, form, pair):
    name, _, _, lp, rp = form
    key = f"mm_{name}_{np.dtype(pair[0]).name}_{np.dtype(pair[1]).name}"
    a, b, want = GOLDEN[key + "_lhs"], GOLDEN[key + "_rhs"], GOLDEN[key + "_out"]
    got = host(ttb.matmul(_view(dev(a), lp), _view(dev(b), rp)))
    assert got.dtype == want.dtype and got.shape == want.shape
    assert _close(got, want)


@pytest.mark.parametrize("dt", [np.float64, np.float32])
@pytest.mark.parametrize("form", FORMS, ids=FORM_IDS)
def test_gradients(ttb, form, dt):
    name, _, _, lp, rp = form
    key = f"bw_{name}_{np.dtype(dt).name}"
    a, b, g = GOLDEN[key + "_lhs"], GOLDEN[key + "_rhs"], GOLDEN[key + "_grad"]
    ta, tb = dev(a), dev(b)
    gl, gr = ttb.matmul_backward(_view(ta, lp), _view(tb, rp), dev(g))
    # the reference returns the gradient of the LEAF, in the leaf's layout: undo the view
    inv = lambda p: tuple(np.argsort(p)) if p is not None else None
    gl, gr = host(_view(gl, inv(lp))), host(_view(gr, inv(rp)))
    assert _close(np.ascontiguousarray(gl), GOLDEN[key + "_glhs"])
    assert _close(np.ascontiguousarray(gr), GOLDEN[key + "_grhs"])


@pytest.mark.skipif(not ref_full.available(), reason="oracle/_ref/libttref_full.so did not travel")
def test_against_the_reference_library_on_seeded_inputs(ttb):
    """Operands drawn with the reference's generator, products by both: C1 as BASELINE gives it
    and ragged / permuted / promoted forms."""
    ops = ttb.config_operands("c1")
    want = ref_full.matmul(ops["A"], ops["B"])
    got = host(ttb.matmul(dev(ops["A"]), dev(ops["B"])))
    assert got.shape == want.shape == (512, 512)
    assert rel_to_max(got, np.matmul(ops["A"].astype(np.float64), ops["B"].astype(np.float64))) <= 1e-5
    assert rel_to_max(got, want.astype(np.float64)) <= 2e-5
    g = ttb.Generator(11)
    a = g.uniform_int(-50, 50, (3, 67, 129))
    b = g.normal(0, 1, (3, 45, 129), np.float64)
    want = ref_full.matmul(a, b, None, (0, 2, 1))
    got = host(ttb.matmul(dev(a), dev(b).permute(0, 2, 1)))
    assert got.dtype == np.float64 and _close(got, want)
    grad = g.normal(0, 1, (3, 67, 45), np.float64)
    af = a.astype(np.float64)
    ga, gb = ref_full.matmul_backward(af, b, grad, None, (0, 2, 1))
    gl, gr = ttb.matmul_backward(dev(af), dev(b).permute(0, 2, 1), dev(grad))
    assert _close(host(gl), ga) and _close(np.ascontiguousarray(host(gr.permute(0, 2, 1))), gb)
