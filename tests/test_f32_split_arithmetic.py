"""The split arithmetic of the f32 tensor-core kernel (tinytensor_b200/csrc/gemm_f32_tcgen05.cu,
hybrid form), restated in numpy: with big = x truncated to TF32 and d = x - big (exact),
    A.B  ~=  big_A.big_B + bf16(d_A).bf16(B) + bf16(A).bf16(d_B)
misses only d_A.d_B and the bf16 rounding of the two corrections, about 2^-19 per term.  Here
the three products are summed in float64, so what is measured is the split itself, not the
accumulation order.  Non-finite elements are zero in the bf16 tiles and travel through the
TF32 product alone."""
import numpy as np
import pytest


def trunc_tf32(x: np.ndarray) -> np.ndarray:
    return (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def to_bf16(x: np.ndarray) -> np.ndarray:
    """Round to nearest even to 8 mantissa bits, returned as float32 (finite inputs)."""
    u = x.astype(np.float32).view(np.uint32).astype(np.uint64)
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return u.astype(np.uint32).view(np.float32)


def split(x: np.ndarray):
    """(big, bf16 low part, bf16 whole) as the converter warps produce them."""
    big = trunc_tf32(x)
    with np.errstate(invalid="ignore"):
        d = x - big                                   # NaN exactly where x is Inf or NaN
    keep = d == d
    low = np.where(keep, to_bf16(np.where(keep, d, 0)), 0).astype(np.float32)
    whole = np.where(keep, to_bf16(np.where(keep, x, 0)), 0).astype(np.float32)
    return big, low, whole


def hybrid_product(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    ab, al, aw = split(a)
    bb, bl, bw = split(b)
    f = np.float64
    with np.errstate(invalid="ignore", over="ignore"):
        return ab.astype(f) @ bb.astype(f) + al.astype(f) @ bw.astype(f) + aw.astype(f) @ bl.astype(f)


def test_low_part_is_exact_and_small():
    rng = np.random.default_rng(0)
    x = (rng.standard_normal(100000) * np.exp(rng.uniform(-20, 20, 100000))).astype(np.float32)
    big = trunc_tf32(x)
    d = x - big
    assert np.array_equal(big.astype(np.float64) + d.astype(np.float64), x.astype(np.float64))
    assert np.all(np.abs(d) <= np.abs(x) * 2.0 ** -10)
    assert np.all(np.sign(d) * np.sign(x) >= 0)       # truncation toward zero: same sign, or zero


@pytest.mark.parametrize("k", [64, 1024, 8192])
def test_split_meets_the_fp32_class_gate(k):
    rng = np.random.default_rng(k)
    a = rng.standard_normal((48, k)).astype(np.float32)
    b = rng.standard_normal((k, 40)).astype(np.float32)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    err = np.abs(hybrid_product(a, b) - ref).max() / np.abs(ref).max()
    assert err <= 2e-6                                # the kernel's gate is 1e-5
    one_pass = np.abs(trunc_tf32(a).astype(np.float64) @ trunc_tf32(b).astype(np.float64) - ref).max() / np.abs(ref).max()
    assert one_pass > 20 * err                        # a single TF32 product is far from it


def test_non_finite_elements_behave_as_in_fp32():
    a = np.array([[1.0, np.inf, 2.0, 0.5], [1.0, 2.0, 3.0, 4.0], [np.nan, 1.0, 1.0, 1.0]], dtype=np.float32)
    b = np.array([[1.0, 0.0], [1.0, 0.0], [-1.0, 3.0], [2.0, 1.0]], dtype=np.float32)
    with np.errstate(invalid="ignore"):
        want = a.astype(np.float64) @ b.astype(np.float64)
    got = hybrid_product(a, b)
    assert got[0, 0] == np.inf and np.isnan(got[0, 1]) == np.isnan(want[0, 1])   # Inf x 0 is NaN in fp32 too
    assert np.allclose(got[1], want[1], rtol=1e-6)
    assert np.isnan(got[2]).all() and np.isnan(want[2]).all()
