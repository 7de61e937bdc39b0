"""GPU parity tests of the i32 tensor-core kernel (byte planes on tcgen05 kind::i8).

The kernel must equal the reference's wrap-around int32 product bit for bit for EVERY input:
the ten u8 x u8 partial products and their shifted sum are exact mod 2^32, including sums far
beyond 2^31 inside the tensor core's s32 accumulators.  Checked against the oracle (C
restatement of the reference's CPU kernel) and, for the forced-variant cases, against this
library's own CUDA-core kernel."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host

pytestmark = pytest.mark.gpu


@pytest.fixture(params=["cta", "pair"])
def forced(ttb, reset_options, request):
    """Both forms of the kernel: one CTA per 128 x 128 tile, and CTA pairs on 256 x 128 tiles."""
    ttb.set_option("force_variant", int(ttb.Variant.TCGEN05_I8LIMB))
    ttb.set_option("two_cta", 0 if request.param == "cta" else 1)
    return ttb


def _full_range(rng, shape):
    return rng.integers(-2**31, 2**31, shape, dtype=np.int64).astype(np.int32)


@pytest.mark.parametrize("shape", [(1, 128, 32, 128), (1, 128, 64, 128), (2, 130, 100, 260), (3, 45, 72, 40),
                                   (1, 1, 36, 4), (1, 257, 516, 132), (4, 64, 1148, 96)])
def test_full_range_operands_wrap_exactly(forced, oracle, shape):
    rng = np.random.default_rng(70)
    B, N, K, M = shape
    a, b = _full_range(rng, (B, N, K)), _full_range(rng, (B, K, M))
    got = host(forced.batched_matmul(dev(a), dev(b)))
    assert forced.last_variant() == forced.Variant.TCGEN05_I8LIMB
    assert np.array_equal(got, oracle.matmul(a, b))


def test_accumulators_wrap_beyond_2_to_32(forced, oracle):
    """All bytes 0xFF, K = 65536: every byte-plane sum is (s + 1) * 65536 * 255^2 > 2^32."""
    K = 65536
    a = np.full((1, 128, K), -1, dtype=np.int32)
    b = np.full((1, K, 128), -1, dtype=np.int32)
    got = host(forced.batched_matmul(dev(a), dev(b)))
    assert (got == K).all()          # (-1) * (-1) * K
    rng = np.random.default_rng(71)
    a, b = _full_range(rng, (1, 128, 20000)), _full_range(rng, (1, 20000, 132))
    a[0, :64] |= 0x7F7F7F7F          # rows with large bytes everywhere
    got = host(forced.batched_matmul(dev(a), dev(b)))
    assert np.array_equal(got, oracle.matmul(a, b))


def test_views_without_copies(forced, oracle):
    """Transposed (MN-major lhs / K-major rhs), offset and batch-broadcast views."""
    rng = np.random.default_rng(72)
    B, N, K, M = 2, 152, 96, 140
    a, b = _full_range(rng, (B, N, K)), _full_range(rng, (B, K, M))
    want = oracle.matmul(a, b)
    A, Bm = dev(a), dev(b)
    At = A.permute(0, 2, 1).contiguous().permute(0, 2, 1)     # lhs stored [K, N]
    Bt = Bm.permute(0, 2, 1).contiguous().permute(0, 2, 1)    # rhs stored [M, K]
    for l, r in ((A, Bm), (At, Bm), (A, Bt), (At, Bt)):
        got = host(forced.batched_matmul(l, r))
        assert forced.last_variant() == forced.Variant.TCGEN05_I8LIMB
        assert np.array_equal(got, want)
    big = torch.zeros((B + 1, N + 3, K + 4), dtype=torch.int32, device="cuda")
    big[1:, 2:2 + N, 4:4 + K] = A
    assert np.array_equal(host(forced.batched_matmul(big[1:, 2:2 + N, 4:4 + K], Bm)), want)
    got = host(forced.batched_matmul(A, Bm[:1].expand(B, K, M)))
    assert np.array_equal(got, oracle.matmul(a, np.broadcast_to(b[:1], b.shape)))


def test_matches_cuda_core_kernel_and_is_default(ttb, oracle, reset_options):
    """The shape of BASELINE config 5 (reduced batch): automatic dispatch takes the tensor-core
    kernel and agrees with the CUDA-core kernel bit for bit."""
    rng = np.random.default_rng(73)
    a = rng.integers(-8, 9, (4, 1024, 512)).astype(np.int32)
    b = rng.integers(-8, 9, (4, 512, 1024)).astype(np.int32)
    A, Bm = dev(a), dev(b)
    auto = ttb.batched_matmul(A, Bm)
    assert ttb.last_variant() == ttb.Variant.TCGEN05_I8LIMB
    ttb.set_option("int_tensor", 0)
    simt = ttb.batched_matmul(A, Bm)
    assert ttb.last_variant() in (ttb.Variant.SIMT, ttb.Variant.SIMT_SPLITK)
    assert torch.equal(auto, simt)
    assert np.array_equal(host(auto)[:1], oracle.matmul(a[:1], b[:1]))


def test_fused_addend_and_strided_output(forced, oracle):
    rng = np.random.default_rng(74)
    a, b = _full_range(rng, (2, 200, 64)), _full_range(rng, (2, 64, 136))
    bias = _full_range(rng, (136,))
    got = host(forced.batched_matmul_fused(dev(a), dev(b), dev(bias)))
    want = (oracle.matmul(a, b).astype(np.int64) + bias).astype(np.int32)
    assert np.array_equal(got, want)
    C = dev(want.copy())
    forced.batched_matmul_fused(dev(a), dev(b), C, out=C)      # accumulate in place
    assert np.array_equal(host(C), (want.astype(np.int64) + oracle.matmul(a, b)).astype(np.int32))
    wide = torch.full((2, 200, 2 * 136), -7, dtype=torch.int32, device="cuda")
    forced.batched_matmul(dev(a), dev(b), out=wide[:, :, ::2])
    assert np.array_equal(host(wide[:, :, ::2].contiguous()), oracle.matmul(a, b))
    assert (wide[:, :, 1::2] == -7).all()


def test_ineligible_views_fall_back_to_cuda_cores(ttb, oracle, reset_options):
    """A view the tensor maps cannot describe (inner stride 2) still multiplies correctly."""
    rng = np.random.default_rng(75)
    a, b = _full_range(rng, (1, 256, 512)), _full_range(rng, (1, 256, 256))
    A = dev(a)[:, :, ::2]
    got = host(ttb.batched_matmul(A, dev(b)))
    assert ttb.last_variant() in (ttb.Variant.SIMT, ttb.Variant.SIMT_SPLITK)
    assert np.array_equal(got, oracle.matmul(a[:, :, ::2], b))


def test_wait_that_runs_out_is_reported_and_the_context_survives(forced, oracle):
    """Failure detection without a GPU fault, as for the f32 kernel: a test switch makes the TMA
    producer arm its first stage but never load it.  Every wait is bounded (2 s): the roles (in
    both CTAs of a pair) give up, tensor memory is freed, the kernel returns, the host reads the
    error word, and the next call on the same context is correct."""
    rng = np.random.default_rng(76)
    a, b = _full_range(rng, (1, 256, 64)), _full_range(rng, (1, 64, 256))
    forced.check_device(0)
    forced.set_option("tc_debug", 16)
    forced.batched_matmul(dev(a), dev(b))
    with pytest.raises(forced.TTBError) as info:
        forced.check_device(0)
    assert info.value.status == -6  # TTB_ETIMEOUT
    forced.set_option("tc_debug", 0)
    forced.check_device(0)
    assert np.array_equal(host(forced.batched_matmul(dev(a), dev(b))), oracle.matmul(a, b))
    forced.check_device(0)
