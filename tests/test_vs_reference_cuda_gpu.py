"""Parity against the reference's own CUDA kernel (tinytensor/tensor/backend/cuda/kernel/
matmul.cuh compiled from its sources into oracle/_ref/libttref_cuda.so): the kernel this
library replaces, run on the same GPU on the same inputs.  Integers must agree bit for bit
(wrap-around included); floats within the f32 / f64 gates.  Skipped when that library has not
been built."""
import numpy as np
import pytest
import torch

import oracle_lib
import refcases
from gpu_util import dev, host, random_operands, rel_to_max

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_cuda():
    r = oracle_lib.load_ref_cuda()
    if r is None:
        pytest.skip("oracle/_ref/libttref_cuda.so not built")
    return r


@pytest.mark.parametrize("dt", refcases.DTYPES)
def test_reference_test_case_matches_reference_cuda_kernel(ttb, ref_cuda, dt):
    lhs, rhs = refcases.batched(dt, B=2)
    L, R = dev(lhs), dev(rhs)
    ours = ttb.batched_matmul(L, R)
    theirs = ref_cuda.matmul(L, R)
    assert torch.equal(ours, theirs)  # exact for floats too on this integer-valued data


@pytest.mark.parametrize("dt", [np.uint8, np.int16, np.int32, np.int64])
def test_full_range_integers_match_reference_cuda_kernel(ttb, ref_cuda, dt):
    info = np.iinfo(dt)
    rng = np.random.default_rng(51)
    a = rng.integers(info.min, info.max, (3, 130, 257), dtype=dt, endpoint=True)
    b = rng.integers(info.min, info.max, (3, 257, 70), dtype=dt, endpoint=True)
    assert torch.equal(ttb.batched_matmul(dev(a), dev(b)), ref_cuda.matmul(dev(a), dev(b)))


def test_strided_views_match_reference_cuda_kernel_on_cloned_operands(ttb, ref_cuda):
    """The reference clones a strided view before multiplying; this library reads the view in
    place.  Same values either way."""
    rng = np.random.default_rng(52)
    a, b = random_operands(rng, np.int32, 2, 100, 96, 64, -50, 50)
    L = dev(a.transpose(0, 2, 1)).permute(0, 2, 1)   # backward's lhs^T view
    R = dev(b.transpose(0, 2, 1)).permute(0, 2, 1)
    assert not L.is_contiguous() and not R.is_contiguous()
    assert torch.equal(ttb.batched_matmul(L, R), ref_cuda.matmul(L, R))


@pytest.mark.parametrize("dt,tol", [(np.float32, 1e-5), (np.float64, 1e-12)])
def test_floats_agree_with_reference_cuda_kernel_within_gate(ttb, ref_cuda, dt, tol):
    rng = np.random.default_rng(53)
    a, b = random_operands(rng, dt, 2, 256, 1024, 384)
    ours = host(ttb.batched_matmul(dev(a), dev(b)))
    theirs = host(ref_cuda.matmul(dev(a), dev(b)))
    want = np.matmul(a.astype(np.longdouble), b.astype(np.longdouble))
    assert rel_to_max(ours, want) <= tol
    assert rel_to_max(theirs, want) <= tol          # the reference meets the same gate
    assert rel_to_max(ours, theirs.astype(np.longdouble)) <= 2 * tol
