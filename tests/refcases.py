"""The known-answer cases of the reference's tests/test_matmul.cpp, restated as data
generators.  Inputs are the small integers (i+j)%100 the reference uses (:171,:176,
:210,:215); the expected value is the wrapping naive loop (:33-46), computed here with
numpy modular arithmetic.  With these inputs f32 sums stay below 2^24, so float results
are exact as well."""
import numpy as np

DTYPES = [np.uint8, np.int16, np.int32, np.int64, np.float32, np.float64]

# test_matmul.cpp:161-163, 199-202
N_REF, M_REF, K_REF = 256 + 123, 1024 + 123, 512 + 123


def _grid(rows, cols, fn):
    i = np.arange(rows)[:, None]
    j = np.arange(cols)[None, :]
    return fn(i, j)


def matrix_matrix(dt):
    """`Matrix Matrix product` (:154-188): lhs[N,M] . rhs[M,K]."""
    lhs = _grid(N_REF, M_REF, lambda i, j: (i + j) % 100).astype(dt)
    rhs = _grid(M_REF, K_REF, lambda i, j: (i + j) % 100).astype(dt)
    return lhs, rhs


def batched(dt, B=4):
    """`Batched Matrix Matrix product` (:191-237)."""
    lhs = np.stack([_grid(N_REF, M_REF, lambda i, j, b=b: (i * b + j + b) % 100) for b in range(B)]).astype(dt)
    rhs = np.stack([_grid(M_REF, K_REF, lambda i, j, b=b: (i + j + 2 * b) % 100) for b in range(B)]).astype(dt)
    return lhs, rhs


def vector_cases(dt):
    """Dot products of length 12 and 2048 (:50-86), vector.matrix and matrix.vector
    (:89-151) with the same (i+j)%100 style data, as 1-D / 2-D operands."""
    v12 = (np.arange(12) % 100).astype(dt)
    v2048 = (np.arange(2048) % 100).astype(dt)
    mat = _grid(N_REF, K_REF, lambda i, j: (i + j) % 100).astype(dt)
    vn = (np.arange(N_REF) % 100).astype(dt)
    vk = (np.arange(K_REF) % 100).astype(dt)
    return {"dot12": (v12, v12), "dot2048": (v2048, v2048), "vec_mat": (vn, mat), "mat_vec": (mat, vk)}


def expected(lhs, rhs):
    """Wrapping product for integer dtypes, float64-accumulated product for floats
    (exact for these inputs)."""
    dt = lhs.dtype
    if np.issubdtype(dt, np.integer):
        return np.matmul(lhs.astype(np.uint64), rhs.astype(np.uint64)).astype(dt)
    return np.matmul(lhs.astype(np.float64), rhs.astype(np.float64)).astype(dt)
