"""Pins the oracle (oracle/matmul_oracle.c) before anything trusts it: against the
reference's own known-answer tests, against the committed golden vectors produced by the
reference's kernel, and against that kernel itself when it has been compiled here."""
from pathlib import Path

import numpy as np
import pytest

import oracle_lib
import refcases

GOLDEN = Path(__file__).resolve().parent / "golden" / "matmul_golden.npz"


@pytest.mark.parametrize("dt", refcases.DTYPES)
def test_oracle_matches_reference_matrix_matrix_case(oracle, dt):
    lhs, rhs = refcases.matrix_matrix(dt)
    got = oracle.matmul(lhs[None], rhs[None])[0]
    assert np.array_equal(got, refcases.expected(lhs, rhs))


@pytest.mark.parametrize("dt", [np.uint8, np.int32, np.float32])
def test_oracle_matches_reference_batched_case(oracle, dt):
    lhs, rhs = refcases.batched(dt)
    got = oracle.matmul(lhs, rhs)
    assert np.array_equal(got, refcases.expected(lhs, rhs))


@pytest.mark.parametrize("dt", refcases.DTYPES)
def test_oracle_matches_reference_vector_cases(oracle, dt):
    for name, (a, b) in refcases.vector_cases(dt).items():
        a3 = a.reshape(1, 1, -1) if a.ndim == 1 else a[None]
        b3 = b.reshape(1, -1, 1) if b.ndim == 1 else b[None]
        got = oracle.matmul(a3, b3)
        assert np.array_equal(got.reshape(-1), refcases.expected(a3, b3).reshape(-1)), name


def test_oracle_loop_orders_are_bit_identical(oracle):
    rng = np.random.default_rng(5)
    for dt in (np.float32, np.float64, np.int16):
        a = (rng.standard_normal((3, 41, 150)) * 50).astype(dt)
        b = (rng.standard_normal((3, 150, 37)) * 50).astype(dt)
        assert np.array_equal(oracle.matmul(a, b, fast=True), oracle.matmul(a, b, fast=False))


def test_oracle_matches_golden_vectors(oracle):
    """Golden vectors were produced by the reference's own kernel (see make_golden.py).
    Integers and the no-contraction float build must match bit for bit; the float build
    with the compiler's default contraction within rounding."""
    g = np.load(GOLDEN)
    keys = sorted(k[:-4] for k in g.files if k.endswith("_lhs"))
    assert len(keys) == 24
    for key in keys:
        lhs, rhs, want = g[key + "_lhs"], g[key + "_rhs"], g[key + "_out"]
        got = oracle.matmul(lhs, rhs)
        assert np.array_equal(got, want), key
        if key + "_out_contracted" in g.files:
            c = g[key + "_out_contracted"]
            tol = 1e-5 if lhs.dtype == np.float32 else 1e-13
            assert np.abs(got - c).max() <= tol * max(1.0, np.abs(c).max()), key


def test_oracle_matches_compiled_reference(oracle):
    if oracle.ref is None or oracle.ref_strict is None:
        pytest.skip("oracle/_ref not built in this checkout (needs the reference tree)")
    rng = np.random.default_rng(11)
    for dt in refcases.DTYPES:
        B, N, K, M = 2, 77, 203, 91
        if np.issubdtype(dt, np.integer):
            a = rng.integers(0, 200, (B, N, K)).astype(dt)
            b = rng.integers(0, 200, (B, K, M)).astype(dt)
        else:
            a = rng.standard_normal((B, N, K)).astype(dt)
            b = rng.standard_normal((B, K, M)).astype(dt)
        assert np.array_equal(oracle.matmul(a, b), oracle.ref_matmul(a, b, strict=True)), dt
        if np.issubdtype(dt, np.integer):
            assert np.array_equal(oracle.matmul(a, b), oracle.ref_matmul(a, b)), dt


def test_oracle_large_scratch_path_of_reference(oracle):
    """The reference switches from static 1200x1200 scratch to heap buffers above that
    size (matmul.hpp:163-179); results must not depend on it."""
    if oracle.ref_strict is None:
        pytest.skip("oracle/_ref not built")
    rng = np.random.default_rng(12)
    a = rng.integers(-8, 9, (1, 1300, 130)).astype(np.int32)
    b = rng.integers(-8, 9, (1, 130, 1250)).astype(np.int32)
    assert np.array_equal(oracle.matmul(a, b), oracle.ref_matmul(a, b, strict=True))
    assert np.array_equal(oracle.matmul(a, b), oracle_lib.wrap_matmul(a, b))
