"""GPU parity tests of the matmul path, through the C ABI (tinytensor_b200 -> libttb.so).

Integer results must be bit-exact against the oracle (wrap-around included); f32 must be
within 1e-5 and f64 within 1e-12 of a float64 / long-double product, measured as
max|c - c_ref| / max|c_ref|.  The cases mirror the reference's tests/test_matmul.cpp and
add what it does not cover: strided, offset, broadcast and permuted views."""
import numpy as np
import pytest
import torch

import refcases
from gpu_util import TORCH_OF, dev, host, random_operands, rel_to_max

pytestmark = pytest.mark.gpu

F32_TOL = 1e-5   # north-star tolerance for f32, relative to max|c_ref|
F64_TOL = 1e-12  # and for f64


def check(got: np.ndarray, lhs: np.ndarray, rhs: np.ndarray, oracle=None):
    dt = lhs.dtype
    if dt.kind in "iu":
        want = refcases.expected(lhs, rhs)
        assert got.dtype == dt
        assert np.array_equal(got, want)
        if oracle is not None:
            assert np.array_equal(got, oracle.matmul(lhs, rhs))
    elif dt == np.float32:
        want = np.matmul(lhs.astype(np.float64), rhs.astype(np.float64))
        assert rel_to_max(got, want) <= F32_TOL
    else:
        want = np.matmul(lhs.astype(np.longdouble), rhs.astype(np.longdouble))
        assert rel_to_max(got, want) <= F64_TOL


# ---------------------------------------------------------------- reference's own cases
@pytest.mark.parametrize("dt", refcases.DTYPES)
def test_reference_matrix_matrix(ttb, oracle, dt):
    lhs, rhs = refcases.matrix_matrix(dt)
    got = host(ttb.matmul(dev(lhs), dev(rhs)))
    assert got.shape == (refcases.N_REF, refcases.K_REF)
    assert np.array_equal(got, refcases.expected(lhs, rhs))  # exact for floats too on this data
    assert np.array_equal(got, oracle.matmul(lhs[None], rhs[None])[0])


@pytest.mark.parametrize("dt", refcases.DTYPES)
def test_reference_batched(ttb, dt):
    lhs, rhs = refcases.batched(dt)
    got = host(ttb.matmul(dev(lhs), dev(rhs)))
    assert np.array_equal(got, refcases.expected(lhs, rhs))


@pytest.mark.parametrize("dt", refcases.DTYPES)
def test_reference_vector_forms(ttb, dt):
    for name, (a, b) in refcases.vector_cases(dt).items():
        got = host(ttb.matmul(dev(a), dev(b)))
        want = refcases.expected(a.reshape(1, -1) if a.ndim == 1 else a, b.reshape(-1, 1) if b.ndim == 1 else b)
        assert np.array_equal(got.reshape(-1), want.reshape(-1)), name
        assert got.ndim == 1, name


def test_bool_and_bad_shapes_raise(ttb):
    t = torch.ones(12, dtype=torch.bool, device="cuda")
    with pytest.raises(ttb.TTBError):
        ttb.matmul(t, t)
    with pytest.raises(ttb.TTBError):
        ttb.matmul(t.view(3, 4), t.view(4, 3))
    a = torch.ones(2, 3, 4, device="cuda")
    with pytest.raises(ttb.TTBError):
        ttb.matmul(a, torch.ones(2, 5, 3, device="cuda"))          # inner dims
    with pytest.raises(ttb.TTBError):
        ttb.batched_matmul(a, torch.ones(3, 4, 3, device="cuda"))  # batch sizes (not checked by the reference)
    with pytest.raises(ttb.TTBError):
        ttb.matmul(torch.ones(2, 2, 2, 2, device="cuda"), torch.ones(2, 2, 2, 2, device="cuda"))
    with pytest.raises(ttb.TTBError):
        ttb.matmul(a, torch.ones(4, 3, device="cuda"))             # no broadcasting of batch dims


def test_dtype_promotion_follows_reference_table(ttb):
    a = torch.arange(12, dtype=torch.uint8, device="cuda").view(3, 4)
    b = torch.arange(8, dtype=torch.int32, device="cuda").view(4, 2)
    out = ttb.matmul(a, b)
    assert out.dtype == torch.int32
    assert torch.equal(out.cpu(), a.cpu().to(torch.int32) @ b.cpu())
    out = ttb.matmul(a, b.to(torch.float32))
    assert out.dtype == torch.float32


# ---------------------------------------------------------------- views the reference clones
def _views(t3: torch.Tensor):
    """(name, lhs view builder) pairs exercised against contiguous truth."""
    return t3


@pytest.mark.parametrize("dt", refcases.DTYPES)
def test_strided_views_match_contiguous(ttb, oracle, dt, reset_options):
    rng = np.random.default_rng(21)
    B, N, K, M = 3, 45, 70, 38
    a, b = random_operands(rng, dt, B, N, K, M, 0, 120)
    want = oracle.matmul(a, b)
    A, Bm = dev(a), dev(b)

    def run(lv, rv):
        got = host(ttb.batched_matmul(lv, rv))
        if np.dtype(dt).kind in "iu":
            assert np.array_equal(got, want)
        else:
            tol = F32_TOL if dt == np.float32 else F64_TOL
            assert rel_to_max(got, want.astype(np.float64)) <= tol

    # transposed storage, viewed back (what backward's permute produces)
    run(A.permute(0, 2, 1).contiguous().permute(0, 2, 1), Bm)
    run(A, Bm.permute(0, 2, 1).contiguous().permute(0, 2, 1))
    # offset views into larger storage
    big = torch.zeros((B + 1, N + 3, K + 5), dtype=A.dtype, device="cuda")
    big[1:, 2:2 + N, 3:3 + K] = A
    run(big[1:, 2:2 + N, 3:3 + K], Bm)
    # positive-step slices on every dim
    wide = torch.zeros((B, 2 * N, 3 * K), dtype=A.dtype, device="cuda")
    wide[:, ::2, ::3] = A
    run(wide[:, ::2, ::3], Bm)
    # batch dim permuted to the middle of the storage
    mid = A.permute(1, 0, 2).contiguous().permute(1, 0, 2)
    run(mid, Bm)


@pytest.mark.parametrize("dt", [np.int32, np.float32, np.uint8])
def test_broadcast_views(ttb, oracle, dt):
    rng = np.random.default_rng(22)
    a, b = random_operands(rng, dt, 4, 20, 33, 17, 0, 50)
    A, Bm = dev(a), dev(b)
    # batch stride 0 on rhs
    got = host(ttb.batched_matmul(A, Bm[:1].expand(4, 33, 17)))
    want = oracle.matmul(a, np.broadcast_to(b[:1], b.shape))
    assert np.array_equal(got, want) if np.dtype(dt).kind in "iu" else rel_to_max(got, want.astype(np.float64)) <= F32_TOL
    # stride 0 on a matrix dim of lhs (every row the same)
    got = host(ttb.batched_matmul(A[:, :1, :].expand(4, 20, 33), Bm))
    want = oracle.matmul(np.broadcast_to(a[:, :1, :], a.shape), b)
    assert np.array_equal(got, want) if np.dtype(dt).kind in "iu" else rel_to_max(got, want.astype(np.float64)) <= F32_TOL


@pytest.mark.parametrize("dt", [np.int32, np.float32, np.int64, np.float64])
def test_small_shape_sweep(ttb, oracle, dt):
    """Every combination of small/ragged extents around the tile edges."""
    rng = np.random.default_rng(23)
    sizes = [1, 2, 7, 16, 17, 33, 64, 65, 129]
    for N in sizes[::2]:
        for K in sizes[1::2]:
            for M in sizes[::3]:
                a, b = random_operands(rng, dt, 2, N, K, M, -9, 10)
                got = host(ttb.batched_matmul(dev(a), dev(b)))
                check(got, a, b)


@pytest.mark.parametrize("dt", refcases.DTYPES)
def test_integer_wraparound_and_extremes(ttb, oracle, dt):
    if np.dtype(dt).kind not in "iu":
        pytest.skip("integers only")
    info = np.iinfo(dt)
    rng = np.random.default_rng(24)
    a = rng.integers(info.min, info.max, (2, 31, 257), dtype=dt, endpoint=True)
    b = rng.integers(info.min, info.max, (2, 257, 29), dtype=dt, endpoint=True)
    got = host(ttb.batched_matmul(dev(a), dev(b)))
    assert np.array_equal(got, oracle.matmul(a, b))


def test_splitk_scratch_path_matches_plain(ttb, oracle, reset_options):
    """Few output tiles and a long K: the SIMT kernel splits K over CTAs, writes partials
    to scratch and reduces them.  Integers stay bit-exact; floats stay in tolerance."""
    rng = np.random.default_rng(25)
    for dt in (np.int32, np.float32, np.float64, np.uint8):
        a, b = random_operands(rng, dt, 1, 130, 4096, 10, -8, 9)
        ttb.set_option("force_variant", int(ttb.Variant.SIMT_SPLITK))
        got = host(ttb.batched_matmul(dev(a), dev(b)))
        assert ttb.last_variant() == ttb.Variant.SIMT_SPLITK
        ttb.set_option("force_variant", int(ttb.Variant.SIMT))
        plain = host(ttb.batched_matmul(dev(a), dev(b)))
        assert ttb.last_variant() == ttb.Variant.SIMT
        check(got, a, b)
        check(plain, a, b)
        if np.dtype(dt).kind in "iu":
            assert np.array_equal(got, plain)


def test_strided_output_column_block(ttb):
    """The partitioner's write of an output-column block straight into row-major C."""
    rng = np.random.default_rng(26)
    a, b = random_operands(rng, np.int32, 1, 100, 64, 384, -8, 9)
    A, Bm = dev(a), dev(b)
    C = torch.full((1, 100, 384), -7, dtype=torch.int32, device="cuda")
    ttb.batched_matmul(A, Bm[:, :, 128:256], out=C[:, :, 128:256])
    want = refcases.expected(a, b)
    got = host(C)
    assert np.array_equal(got[:, :, 128:256], want[:, :, 128:256])
    assert (got[:, :, :128] == -7).all() and (got[:, :, 256:] == -7).all()


def test_host_buffer_entry_point(ttb, oracle):
    rng = np.random.default_rng(27)
    for dt in (np.int32, np.float32, np.int64):
        a, b = random_operands(rng, dt, 3, 65, 129, 70, -8, 9)
        got = ttb.batched_matmul_host(a, b.transpose(0, 2, 1).copy().transpose(0, 2, 1))
        check(got, a, b)


def test_host_buffer_pipeline_rows(ttb):
    """Products large enough to be pipelined through the host-buffer entry point, in blocks of
    lhs rows (every copy one contiguous span), agree with the device-resident call: integers bit
    for bit, f32 within the rounding of a different summation order.  lhs is a view into a wider
    matrix (row pitch > K)."""
    rng = np.random.default_rng(30)
    for dt, (N, K, M) in ((np.int32, (5000, 2048, 2048)), (np.float32, (4200, 4096, 2048))):
        wide, b = random_operands(rng, dt, 1, N, K + 72, M, -8, 9)
        b = b[:, :K]
        a = wide[:, :, 8:8 + K]
        got = ttb.batched_matmul_host(a, b)
        want = host(ttb.batched_matmul(dev(np.ascontiguousarray(a)), dev(np.ascontiguousarray(b))))
        if dt == np.int32:
            assert np.array_equal(got, want)
        else:
            assert rel_to_max(got, want) <= 2e-6


def test_host_buffer_pipeline_columns(ttb):
    """The same in blocks of output columns, taken when the lhs rows are not contiguous (here the
    lhs is stored transposed); rhs is a view into a wider matrix (row pitch > M)."""
    rng = np.random.default_rng(28)
    for dt, (N, K, M) in ((np.int32, (2048, 2048, 5000)), (np.float32, (2048, 4096, 4200))):
        a, wide = random_operands(rng, dt, 1, N, K, M + 72, -8, 9)
        a_t = np.ascontiguousarray(a.transpose(0, 2, 1)).transpose(0, 2, 1)
        b = wide[:, :, 8:8 + M]
        got = ttb.batched_matmul_host(a_t, b)
        want = host(ttb.batched_matmul(dev(a), dev(np.ascontiguousarray(b))))
        if dt == np.int32:
            assert np.array_equal(got, want)
        else:
            assert rel_to_max(got, want) <= 2e-6


def test_host_buffer_pipeline_batches(ttb):
    """Batched products large enough to be pipelined in groups of batches."""
    rng = np.random.default_rng(29)
    for dt, (B, N, K, M) in ((np.int32, (9, 1024, 2048, 1536)), (np.float32, (6, 2048, 2048, 1024))):
        a, b = random_operands(rng, dt, B, N, K, M, -8, 9)
        got = ttb.batched_matmul_host(a, b)
        want = host(ttb.batched_matmul(dev(a), dev(b)))
        if dt == np.int32:
            assert np.array_equal(got, want)
        else:
            assert rel_to_max(got, want) <= 2e-6


def test_multi_device_placement(ttb):
    """tests/test_multi_device_cuda.cpp:18-51: same-device work on device 1, cross-device throws."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    a0 = torch.ones(2, 8, 8, device="cuda:0")
    a1 = torch.ones(2, 8, 8, device="cuda:1")
    out = ttb.matmul(a1, a1)
    assert out.device == a1.device and torch.equal(out.cpu(), torch.full((2, 8, 8), 8.0))
    with pytest.raises(ttb.TTBError):
        ttb.matmul(a0, a1)


# ---------------------------------------------------------------- BASELINE configs
def test_config1_f32_512(ttb):
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    b = rng.uniform(-1, 1, (512, 512)).astype(np.float32)
    got = host(ttb.matmul(dev(a), dev(b)))
    assert rel_to_max(got, a.astype(np.float64) @ b.astype(np.float64)) <= F32_TOL


def test_config2_mlp_forward_and_backward_products(ttb):
    """X[4096,784].W1^T, H.W2^T and the four backward products, all through the rank-3
    entry with [1,.,.] views; transposed operands are permuted views, never copies."""
    rng = np.random.default_rng(1)
    X = rng.uniform(0, 1, (4096, 784)).astype(np.float32)
    W1 = rng.uniform(-1, 1, (1024, 784)).astype(np.float32) / np.sqrt(784).astype(np.float32)
    W2 = rng.uniform(-1, 1, (10, 1024)).astype(np.float32) / np.float32(32.0)
    dH = rng.uniform(-1, 1, (4096, 1024)).astype(np.float32)
    dC = rng.uniform(-1, 1, (4096, 10)).astype(np.float32)
    dX, dW1, dW2, ddH, ddC = map(lambda t: dev(t)[None], (X, W1, W2, dH, dC))
    f64 = lambda t: t.astype(np.float64)
    H = ttb.batched_matmul(dX, dW1.permute(0, 2, 1))
    Hn = host(H)[0]
    assert rel_to_max(Hn, f64(X) @ f64(W1).T) <= F32_TOL
    cases = {
        "fwd2": (H, dW2.permute(0, 2, 1), f64(Hn) @ f64(W2).T),
        "bwd_dX": (ddH, dW1, f64(dH) @ f64(W1)),
        "bwd_dW1": (dX.permute(0, 2, 1), ddH, f64(X).T @ f64(dH)),
        "bwd_dH": (ddC, dW2, f64(dC) @ f64(W2)),
        "bwd_dW2": (H.permute(0, 2, 1), ddC, f64(Hn).T @ f64(dC)),
    }
    for name, (l, r, want) in cases.items():
        got = host(ttb.batched_matmul(l, r))[0]
        assert rel_to_max(got, want) <= F32_TOL, name


def test_config3_attention_style_batched(ttb):
    rng = np.random.default_rng(2)
    Q, K, V = (rng.standard_normal((256, 128, 64)).astype(np.float32) for _ in range(3))
    dQ, dK, dV = dev(Q), dev(K), dev(V)
    S = ttb.batched_matmul(dQ, dK.permute(0, 2, 1))
    Sn = host(S)
    assert rel_to_max(Sn, np.matmul(Q.astype(np.float64), K.astype(np.float64).transpose(0, 2, 1))) <= F32_TOL
    O = host(ttb.batched_matmul(S, dV))
    assert rel_to_max(O, np.matmul(Sn.astype(np.float64), V.astype(np.float64))) <= F32_TOL


def test_config4_large_square_f32_sampled_rows(ttb):
    """8192^3 at full size; the float64 reference is computed for a sample of rows."""
    n = 8192
    g = torch.Generator(device="cuda").manual_seed(3)
    A = torch.randn((1, n, n), generator=g, device="cuda") * (n ** -0.5)
    B = torch.randn((1, n, n), generator=g, device="cuda") * (n ** -0.5)
    C = ttb.batched_matmul(A, B)
    rows = torch.tensor([0, 1, 127, 128, 4095, 4096, 8000, 8191], device="cuda")
    want = (A[0, rows].double() @ B[0].double()).cpu().numpy()
    got = C[0, rows].cpu().numpy()
    assert rel_to_max(got, want) <= F32_TOL
    # The column-block form used by the partitioner.  Not bit-identical to the full product: a
    # block's tile count need not fill the GPU, then K is dealt out differently (stream-K) and the
    # fp32 partial sums associate differently.  Both stay far inside the gate.
    C2 = torch.empty_like(C)
    for c0 in range(0, n, 2048):
        ttb.batched_matmul(A, B[:, :, c0:c0 + 2048], out=C2[:, :, c0:c0 + 2048])
    assert float((C - C2).abs().max() / C.abs().max()) <= 2e-6
    assert rel_to_max(C2[0, rows].cpu().numpy(), want) <= F32_TOL


def test_config4b_f64_4096(ttb):
    n = 4096
    g = torch.Generator(device="cuda").manual_seed(3)
    A = (torch.randn((1, n, n), generator=g, device="cuda", dtype=torch.float64) * (8192 ** -0.5))
    B = (torch.randn((1, n, n), generator=g, device="cuda", dtype=torch.float64) * (8192 ** -0.5))
    C = ttb.batched_matmul(A, B)
    rows = [0, 77, 2048, 4095]
    a = A[0, rows].cpu().numpy().astype(np.longdouble)
    b = B[0].cpu().numpy().astype(np.longdouble)
    assert rel_to_max(C[0, rows].cpu().numpy(), a @ b) <= F64_TOL


def test_config5_i32_batched_bit_exact(ttb):
    rng = np.random.default_rng(4)
    a = rng.integers(-8, 9, (64, 1024, 512)).astype(np.int32)
    b = rng.integers(-8, 9, (64, 512, 1024)).astype(np.int32)
    got = host(ttb.batched_matmul(dev(a), dev(b)))
    # |sum| <= 32768: float64 BLAS is exact here and fast enough at full size
    want = np.matmul(a.astype(np.float64), b.astype(np.float64)).astype(np.int32)
    assert np.array_equal(got, want)


def test_no_bounded_wait_gave_up(ttb):
    ttb.check_device(0)
