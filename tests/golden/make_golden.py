"""Generates tests/golden/matmul_golden.npz from the REFERENCE's own CPU kernel.

Run in a container that has the reference tree: `make -C oracle` compiles the
reference kernel (tinytensor/tensor/backend/cpu/kernel/matmul.hpp) into
oracle/_ref/libttref_strict.so, and this script feeds it small seeded inputs and stores
inputs and outputs.  The fixture travels with the repository; the reference does not.

    python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import oracle_lib  # noqa: E402

CASES = {
    # name: (B, N, K, M) -- ragged sizes, K crossing the reference's 64-wide K chunks
    "small": (2, 19, 70, 33),
    "vec_mat": (1, 1, 131, 45),
    "mat_vec": (1, 45, 131, 1),
    "dot": (1, 1, 200, 1),
}
DTYPES = [np.uint8, np.int16, np.int32, np.int64, np.float32, np.float64]


def main():
    o = oracle_lib.load()
    assert o.ref_strict is not None, "build oracle/_ref first: make -C oracle"
    out = {}
    for name, shape in CASES.items():
        for dt in DTYPES:
            # hash() of str is salted per process: derive the seed deterministically instead
            seed = sum(ord(c) for c in name) * 131 + np.dtype(dt).itemsize * 7 + int(np.dtype(dt).kind == "f")
            rng = np.random.default_rng(seed)
            B, N, K, M = shape
            if np.issubdtype(dt, np.integer):
                info = np.iinfo(dt)
                lo, hi = (0, 256) if dt == np.uint8 else (max(info.min, -(2**40)), min(info.max, 2**40))
                a = rng.integers(lo, hi, (B, N, K)).astype(dt)
                b = rng.integers(lo, hi, (B, K, M)).astype(dt)
            else:
                a = rng.standard_normal((B, N, K)).astype(dt)
                b = rng.standard_normal((B, K, M)).astype(dt)
            key = f"{name}_{np.dtype(dt).name}"
            out[key + "_lhs"] = a
            out[key + "_rhs"] = b
            out[key + "_out"] = o.ref_matmul(a, b, strict=True)
            if np.issubdtype(dt, np.floating):
                out[key + "_out_contracted"] = o.ref_matmul(a, b, strict=False)
    np.savez_compressed(HERE / "matmul_golden.npz", **out)
    print("wrote", HERE / "matmul_golden.npz", len(out), "arrays")


if __name__ == "__main__":
    main()
