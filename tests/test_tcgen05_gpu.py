"""Parity tests specific to the tcgen05 / TMEM / TMA f32 kernel.  It has three arithmetic
modes ("tf32_terms"): 2 = hybrid split, the default (TF32 product of the big parts plus two bf16
correction products), 3 = classic 3xTF32, 1 = one TF32 pass (test only); and two tile forms
(one CTA, CTA pair).

The kernel is forced, so a view it cannot take is an error rather than a silent detour
through the SIMT kernel.  Operand layouts cover the four major combinations that forward
and backward produce: row-major lhs (K-major), transposed-view lhs (MN-major), row-major
rhs (MN-major) and transposed-view rhs (K-major)."""
import numpy as np
import pytest
import torch

from gpu_util import dev, host, rel_to_max

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5


@pytest.fixture(params=["cta", "pair"])
def forced(request, ttb, reset_options):
    """Forces the tensor-core kernel, once as single-CTA tiles and once as CTA pairs."""
    ttb.set_option("force_variant", int(ttb.Variant.TCGEN05_3XTF32 if request.param == "cta" else ttb.Variant.TCGEN05_2CTA))
    return ttb


def padded(t: torch.Tensor, pad_to: int = 4) -> torch.Tensor:
    """Same values, but the innermost extent of the STORAGE is rounded up to `pad_to`
    elements so that row strides are multiples of 16 bytes (a TMA requirement); the view
    keeps the ragged logical shape, which exercises out-of-bounds zero fill."""
    *lead, n = t.shape
    npad = (n + pad_to - 1) // pad_to * pad_to
    store = torch.zeros((*lead, npad), dtype=t.dtype, device=t.device)
    store[..., :n] = t
    return store[..., :n]


def layouts(a: torch.Tensor, b: torch.Tensor):
    """The four operand-major combinations of the same logical product."""
    a_k = padded(a)                                             # [B,N,K] K contiguous
    a_mn = padded(a.permute(0, 2, 1).contiguous()).permute(0, 2, 1)  # N contiguous
    b_mn = padded(b)                                            # [B,K,M] M contiguous
    b_k = padded(b.permute(0, 2, 1).contiguous()).permute(0, 2, 1)   # K contiguous
    return {"kmaj.mnmaj": (a_k, b_mn), "kmaj.kmaj": (a_k, b_k), "mnmaj.mnmaj": (a_mn, b_mn),
            "mnmaj.kmaj": (a_mn, b_k)}


@pytest.mark.parametrize("shape", [(1, 128, 32, 128), (1, 128, 64, 128), (2, 256, 96, 384), (1, 379, 1147, 635),
                                   (3, 130, 70, 33), (1, 17, 40, 257)])
def test_single_tf32_pass_is_exact_on_small_integers(forced, shape):
    """Integers up to 2048 are exact in TF32 and the sums stay below 2^24, so even one
    TF32 pass must reproduce the wrapping-free integer product exactly.  This isolates the
    TMA maps, shared-memory descriptors and the TMEM read-back from the split arithmetic."""
    B, N, K, M = shape
    rng = np.random.default_rng(31)
    a = rng.integers(-9, 10, (B, N, K)).astype(np.float32)
    b = rng.integers(-9, 10, (B, K, M)).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64)).astype(np.float32)
    forced.set_option("tf32_terms", 1)
    for name, (l, r) in layouts(dev(a), dev(b)).items():
        got = host(forced.batched_matmul(l, r))
        assert forced.last_variant() in (forced.Variant.TCGEN05_3XTF32, forced.Variant.TCGEN05_2CTA)
        assert np.array_equal(got, want), name
    forced.check_device(0)


@pytest.mark.parametrize("terms", [2, 3])
@pytest.mark.parametrize("shape", [(1, 128, 128, 128), (1, 379, 1147, 635), (4, 200, 300, 150), (1, 512, 4096, 256)])
def test_split_meets_f32_tolerance_all_layouts(forced, shape, terms):
    B, N, K, M = shape
    forced.set_option("tf32_terms", terms)
    rng = np.random.default_rng(32)
    a = rng.standard_normal((B, N, K)).astype(np.float32)
    b = rng.standard_normal((B, K, M)).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    for name, (l, r) in layouts(dev(a), dev(b)).items():
        got = host(forced.batched_matmul(l, r))
        assert rel_to_max(got, want) <= F32_TOL, name
    forced.check_device(0)


def test_single_pass_is_not_enough_and_split_is(forced):
    """The reason for the split: one TF32 pass misses 1e-5, three passes meet it."""
    rng = np.random.default_rng(33)
    a = rng.standard_normal((1, 256, 2048)).astype(np.float32)
    b = rng.standard_normal((1, 2048, 256)).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    forced.set_option("tf32_terms", 1)
    one = rel_to_max(host(forced.batched_matmul(dev(a), dev(b))), want)
    forced.set_option("tf32_terms", 3)
    three = rel_to_max(host(forced.batched_matmul(dev(a), dev(b))), want)
    forced.set_option("tf32_terms", 2)
    hybrid = rel_to_max(host(forced.batched_matmul(dev(a), dev(b))), want)
    assert one > F32_TOL
    assert three <= F32_TOL
    assert hybrid <= F32_TOL


def test_hybrid_bf16_tile_layouts_are_exact_on_small_integers(forced):
    """The hybrid split's bf16 tiles (written by the converters, read by kind::f16 MMAs) in all
    four operand layouts: with the layout-check switch the kernel adds bf16(A).bf16(B) to the
    TF32 product, which on small integers must be exactly twice the product."""
    rng = np.random.default_rng(38)
    a = rng.integers(-9, 10, (2, 300, 100)).astype(np.float32)
    b = rng.integers(-9, 10, (2, 100, 260)).astype(np.float32)
    want = (2 * np.matmul(a.astype(np.float64), b.astype(np.float64))).astype(np.float32)
    forced.set_option("tf32_terms", 2)
    forced.set_option("tc_debug", 8)
    for name, (l, r) in layouts(dev(a), dev(b)).items():
        assert np.array_equal(host(forced.batched_matmul(l, r)), want), name
    forced.check_device(0)


def test_all_positive_operands_stay_inside_the_gate(forced):
    """Sums that only grow are the worst case for the tensor core's truncating accumulator;
    the chunked accumulation keeps them inside 1e-5."""
    rng = np.random.default_rng(39)
    a = np.abs(rng.standard_normal((1, 256, 8192))).astype(np.float32)
    b = np.abs(rng.standard_normal((1, 8192, 256))).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    for terms in (2, 3):
        forced.set_option("tf32_terms", terms)
        assert rel_to_max(host(forced.batched_matmul(dev(a), dev(b))), want) <= F32_TOL, terms


def test_tensor_core_reads_fp32_words_as_truncated_tf32(forced):
    """The split assumes kind::tf32 ignores the low 13 mantissa bits of an fp32 word.
    Rewriting the raw tile with its explicitly masked big part must therefore not change
    a single bit of the result."""
    rng = np.random.default_rng(34)
    a = rng.standard_normal((1, 256, 512)).astype(np.float32)
    b = rng.standard_normal((1, 512, 256)).astype(np.float32)
    forced.set_option("tf32_terms", 3)
    plain = host(forced.batched_matmul(dev(a), dev(b)))
    forced.set_option("mask_big", 1)
    masked = host(forced.batched_matmul(dev(a), dev(b)))
    assert np.array_equal(plain, masked)


def test_long_k_accumulation_error(forced):
    """K = 8192 (the headline shape's depth) on N(0, 1/sqrt(K)) entries."""
    K = 8192
    rng = np.random.default_rng(35)
    a = (rng.standard_normal((1, 256, K)) * K ** -0.5).astype(np.float32)
    b = (rng.standard_normal((1, K, 384)) * K ** -0.5).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    got = host(forced.batched_matmul(dev(a), dev(b)))
    assert rel_to_max(got, want) <= F32_TOL


def test_broadcast_batch_and_offset_views(forced):
    rng = np.random.default_rng(36)
    a = rng.standard_normal((5, 128, 64)).astype(np.float32)
    b = rng.standard_normal((1, 64, 256)).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    got = host(forced.batched_matmul(dev(a), dev(b).expand(5, 64, 256)))
    assert rel_to_max(got, want) <= F32_TOL
    # offset view: rows 8.. of a larger matrix, columns 64..192 of a wider rhs
    big = dev(rng.standard_normal((1, 300, 64)).astype(np.float32))
    wide = dev(rng.standard_normal((1, 64, 512)).astype(np.float32))
    l, r = big[:, 8:264, :], wide[:, :, 64:192]
    want = np.matmul(host(l).astype(np.float64), host(r).astype(np.float64))
    assert rel_to_max(host(forced.batched_matmul(l, r)), want) <= F32_TOL


def test_strided_output(forced):
    rng = np.random.default_rng(37)
    a = dev(rng.standard_normal((1, 256, 128)).astype(np.float32))
    b = dev(rng.standard_normal((1, 128, 512)).astype(np.float32))
    C = torch.zeros((1, 256, 512), device="cuda")
    for c0 in (0, 256):
        forced.batched_matmul(a, b[:, :, c0:c0 + 256], out=C[:, :, c0:c0 + 256])
    full = forced.batched_matmul(a, b)
    assert torch.equal(C, full)


def test_ineligible_view_is_refused_when_forced_and_rerouted_when_not(forced):
    a = torch.randn((1, 64, 70), device="cuda")[:, :, ::2]  # inner step 2
    b = torch.randn((1, 35, 64), device="cuda")
    with pytest.raises(forced.TTBError):
        forced.batched_matmul(a, b)
    forced.set_option("force_variant", 0)
    out = forced.batched_matmul(a, b)
    assert forced.last_variant() in (forced.Variant.SIMT, forced.Variant.SIMT_SPLITK)
    want = np.matmul(host(a).astype(np.float64), host(b).astype(np.float64))
    assert rel_to_max(host(out), want) <= F32_TOL


def test_non_finite_operands_propagate_like_fp32(forced):
    """Inf and NaN must come out where an fp32 product puts them (the split must not turn an
    infinite result into NaN through Inf - Inf or 0 x Inf in its correction terms)."""
    rng = np.random.default_rng(40)
    a = rng.uniform(0.5, 1.5, (1, 128, 96)).astype(np.float32)
    b = rng.uniform(0.5, 1.5, (1, 96, 160)).astype(np.float32)
    a[0, 3, 7] = np.inf           # row 3 of C becomes +Inf (all of b[7, :] is positive)
    a[0, 9, 11] = -np.inf         # row 9 becomes -Inf ...
    b[0, 11, 5] = 0.0             # ... except column 5: -Inf * 0 = NaN
    a[0, 20, 30] = np.nan         # row 20 becomes NaN
    b[0, 40, 100] = np.inf        # column 100 becomes +Inf (a[:, 40] positive), NaN in row 20
    with np.errstate(invalid="ignore", over="ignore"):
        want = np.matmul(a.astype(np.float64), b.astype(np.float64)).astype(np.float32)
    got = host(forced.batched_matmul(dev(a), dev(b)))
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(np.isposinf(got), np.isposinf(want))
    assert np.array_equal(np.isneginf(got), np.isneginf(want))
    finite = np.isfinite(want)
    assert np.abs(got[finite] - want[finite]).max() <= 1e-5 * np.abs(want[finite]).max()


def test_wait_that_runs_out_is_reported_and_the_context_survives(forced):
    """Failure detection without a GPU fault: a test switch makes the TMA producer arm its
    first stage but never load it, so nothing ever completes that barrier.  Every wait in the
    kernel is bounded (2 s): the roles give up, the kernel frees its TMEM and returns, the host
    reads the error word, and the next call on the same context works."""
    a = torch.randn((1, 256, 64), device="cuda")
    b = torch.randn((1, 64, 256), device="cuda")
    forced.check_device(0)
    forced.set_option("tc_debug", 16)
    forced.batched_matmul(a, b)
    with pytest.raises(forced.TTBError) as info:
        forced.check_device(0)
    assert info.value.status == -6  # TTB_ETIMEOUT
    assert "bounded wait" in str(info.value)
    forced.set_option("tc_debug", 0)
    forced.check_device(0)  # the error word was cleared by the read
    out = forced.batched_matmul(a, b)
    want = np.matmul(host(a).astype(np.float64), host(b).astype(np.float64))
    assert rel_to_max(host(out), want) <= F32_TOL
    forced.check_device(0)


# the last shape has whole waves of tiles plus a partial wave: only that one is cut by K blocks
@pytest.mark.parametrize("shape", [(1, 784, 4096, 1024), (1, 300, 1000, 260), (3, 256, 512, 384), (1, 128, 2048, 128),
                                   (1, 2560, 2048, 4096)])
def test_stream_k_distribution_matches_whole_tiles(forced, shape):
    """With stream-K the K blocks of all tiles are dealt out evenly over the SMs; tiles cut across
    units are completed from partial sums in a workspace.  Exact on small integers, inside the
    gate on normal data, in every operand layout, and repeatable from launch to launch."""
    B, N, K, M = shape
    rng = np.random.default_rng(43)
    ai = rng.integers(-9, 10, (B, N, K)).astype(np.float32)
    bi = rng.integers(-9, 10, (B, K, M)).astype(np.float32)
    wi = np.matmul(ai.astype(np.float64), bi.astype(np.float64)).astype(np.float32)
    a = rng.standard_normal((B, N, K)).astype(np.float32)
    b = rng.standard_normal((B, K, M)).astype(np.float32)
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    forced.set_option("streamk", 1)
    for name, (l, r) in layouts(dev(ai), dev(bi)).items():
        assert np.array_equal(host(forced.batched_matmul(l, r)), wi), name
    first = None
    for name, (l, r) in layouts(dev(a), dev(b)).items():
        got = host(forced.batched_matmul(l, r))
        assert rel_to_max(got, want) <= F32_TOL, name
        again = host(forced.batched_matmul(l, r))
        assert np.array_equal(got, again), name  # fixed summation order: bit-repeatable
        first = got if first is None else first
    forced.check_device(0)


def test_denormal_operands(forced):
    """fp32 denormals (|x| < 2^-126).  The tensor cores do not flush them, but a denormal has no
    full mantissa to split: its TF32 part keeps bits down to 2^-136 and the bf16 correction
    cannot represent anything below 2^-133, so a denormal operand contributes with an ABSOLUTE
    error of up to 2^-136 |b| per term instead of the relative 2^-22 of a normal one.
    (a) Mixed into ordinary data that is far below everything else: the 1e-5 gate holds.
    (b) A product whose every lhs entry is denormal: the error is bounded by that absolute
        term (about 1e-2 of such a result), while the CUDA-core kernel keeps fp32 accuracy --
        the documented deviation of the split-precision path."""
    rng = np.random.default_rng(47)
    K = 256
    a = rng.standard_normal((1, 128, K)).astype(np.float32)
    b = rng.standard_normal((1, K, 128)).astype(np.float32)
    a[0, ::3, ::5] = (rng.standard_normal(a[0, ::3, ::5].shape) * 1e-39).astype(np.float32)
    b[0, ::7, ::2] = (rng.standard_normal(b[0, ::7, ::2].shape) * 1e-40).astype(np.float32)
    assert (np.abs(a[a != 0]).min() < 1.1754944e-38) and (np.abs(b[b != 0]).min() < 1.1754944e-38)
    got = host(forced.batched_matmul(dev(a), dev(b)))
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    assert rel_to_max(got, want) <= F32_TOL
    a = (rng.standard_normal((1, 128, K)) * 1e-39).astype(np.float32)
    b = (rng.standard_normal((1, K, 128)) * 1e20).astype(np.float32)
    got = host(forced.batched_matmul(dev(a), dev(b)))
    want = np.matmul(a.astype(np.float64), b.astype(np.float64))
    assert np.count_nonzero(got) == got.size          # nothing was flushed to zero
    bound = 2.0 ** -136 * np.abs(b).astype(np.float64).sum(axis=1).max()  # 2^-136 |b| per term, worst column
    assert np.abs(got - want).max() <= bound
    assert rel_to_max(got, want) <= 5e-2


@pytest.mark.parametrize("option,value", [("a_tmem", 1), ("extra_conv", 0)])
@pytest.mark.parametrize("shape", [(2, 256, 512, 256), (1, 379, 1147, 635), (8, 128, 64, 128)])
def test_converter_variants_meet_f32_tolerance_all_layouts(forced, shape, option, value):
    """Two switches of the hybrid split's converters, all four operand majors, both kernel forms:
    `a_tmem` = 1 puts the A operands of the correction products into tensor memory (written by the
    converters with tcgen05.st, read by the MMAs in their A-from-TMEM form; the pair form then
    keeps one accumulator); `extra_conv` = 0 takes the two spare warps of the pair form out of the
    conversion (the default has them convert 5/8 of every B tile)."""
    rng = np.random.default_rng(77)
    B, N, K, M = shape
    a = dev(rng.standard_normal((B, N, K)).astype(np.float32))
    b = dev(rng.standard_normal((B, K, M)).astype(np.float32))
    want = np.matmul(host(a).astype(np.float64), host(b).astype(np.float64))
    forced.set_option(option, value)
    try:
        for name, (av, bv) in layouts(a, b).items():
            if forced.get_option("force_variant") == int(forced.Variant.TCGEN05_2CTA) and (N <= 128 or M <= 128):
                continue
            got = forced.batched_matmul(av, bv)
            assert rel_to_max(host(got), want) <= F32_TOL, (name, option)
        forced.check_device(0)
    finally:
        forced.set_option("a_tmem", 0)
        forced.set_option("extra_conv", 1)


@pytest.mark.parametrize("pieces", [2, 4, 8])
@pytest.mark.parametrize("shape", [(1, 1024, 2048, 768), (3, 300, 1504, 260), (1, 512, 4096, 512)])
def test_piece_schedule_meets_f32_tolerance_and_is_repeatable(forced, shape, pieces):
    """The piece schedule (every tile's K range cut into a power of two of parts that are dealt out
    round-robin; the part that draws a tile's last ticket adds all parts in part order): same
    tolerance as whole tiles, and the same bits on every run whichever part comes last."""
    rng = np.random.default_rng(91)
    B, N, K, M = shape
    a = dev(rng.standard_normal((B, N, K)).astype(np.float32))
    b = dev(rng.standard_normal((B, K, M)).astype(np.float32))
    want = np.matmul(host(a).astype(np.float64), host(b).astype(np.float64))
    if forced.get_option("force_variant") == int(forced.Variant.TCGEN05_2CTA) and (N <= 128 or M <= 128):
        pytest.skip("pair tiles need both extents above 128")
    forced.set_option("pieces", pieces)
    try:
        first = host(forced.batched_matmul(a, b))
        assert rel_to_max(first, want) <= F32_TOL
        for _ in range(3):
            again = host(forced.batched_matmul(a, b))
            assert np.array_equal(first, again)
        forced.check_device(0)
    finally:
        forced.set_option("pieces", -1)


@pytest.mark.parametrize("shape", [(1, 2048, 4096, 1024), (1, 3000, 2048, 2900), (2, 1100, 1536, 900)])
def test_paired_stream_k_meets_f32_tolerance_and_is_repeatable(forced, shape):
    """Paired stream-K (odd units walk their K-block range backwards; the two units that share a
    tile draw tickets, the second adds the first's sums to its own and stores): same tolerance as
    the plain cut, and the same bits on every run whichever unit comes second."""
    rng = np.random.default_rng(92)
    B, N, K, M = shape
    a = dev(rng.standard_normal((B, N, K)).astype(np.float32))
    b = dev(rng.standard_normal((B, K, M)).astype(np.float32))
    want = np.matmul(host(a).astype(np.float64), host(b).astype(np.float64))
    forced.set_option("streamk", 1)
    forced.set_option("sk_pair", 1)
    try:
        first = host(forced.batched_matmul(a, b))
        assert rel_to_max(first, want) <= F32_TOL
        for _ in range(3):
            assert np.array_equal(first, host(forced.batched_matmul(a, b)))
        forced.check_device(0)
    finally:
        forced.set_option("streamk", -1)
        forced.set_option("sk_pair", -1)


@pytest.mark.parametrize("level", [1, 2])
def test_profile_counters_do_not_change_results(forced, level):
    """`tc_profile` = 1 runs the instantiation with cycle counters in every role's loop, 2 records
    CTA lifetimes only: same bits as the plain kernel, and counters that make sense (a lifetime
    for every CTA that ran; with level 1 the converters' busy time inside it)."""
    import ctypes

    rng = np.random.default_rng(93)
    a = dev(rng.standard_normal((1, 1024, 2048)).astype(np.float32))
    b = dev(rng.standard_normal((1, 2048, 768)).astype(np.float32))
    plain = host(forced.batched_matmul(a, b))
    forced.set_option("tc_profile", level)
    try:
        got = host(forced.batched_matmul(a, b))
        torch.cuda.synchronize()
        out = (ctypes.c_int64 * (148 * 8))()
        assert forced.lib().ttb_tc_profile(0, out, 148) == 0
        prof = np.array(out[:], dtype=np.int64).reshape(148, 8)
    finally:
        forced.set_option("tc_profile", 0)
    assert np.array_equal(plain, got)
    total = prof[:, 7]
    assert total.max() > 0
    if level == 1:
        busy = prof[:, 5]
        assert busy.max() > 0 and np.all(busy <= total.max())
    forced.check_device(0)
