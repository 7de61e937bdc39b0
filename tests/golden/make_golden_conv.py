"""Generates tests/golden/conv_golden.npz from the REFERENCE's own CPU conv2d kernels.

Run in a container that has the reference tree: `make -C oracle` compiles the reference's
unroll / matmul / col2im kernels (tinytensor/tensor/backend/cpu/kernel/conv.hpp, matmul.hpp),
driven in the order of its CPU runner (backend/cpu/conv.cpp), into
oracle/_ref/libttref_strict.so; this script feeds them small seeded inputs and stores inputs
and outputs.  The fixture travels with the repository; the reference does not.

    python tests/golden/make_golden_conv.py
"""
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import oracle_lib  # noqa: E402

CASES = {
    # name: (B, C_in, C_out, H, W, K, stride, padding)
    "s1p0": (2, 3, 5, 9, 8, 3, 1, 0),
    "s2p1": (2, 2, 4, 11, 7, 3, 2, 1),
    "k1": (1, 4, 3, 5, 5, 1, 1, 0),
    "s3p2k5": (1, 2, 3, 13, 9, 5, 3, 2),
}
DTYPES = [np.uint8, np.int16, np.int32, np.int64, np.float32, np.float64]


def main():
    o = oracle_lib.load()
    assert o.ref_strict is not None, "build oracle/_ref first: make -C oracle"
    out = {}
    for name, (B, C_in, C_out, H, W, K, S, P) in CASES.items():
        for dt in DTYPES:
            seed = sum(ord(c) for c in name) * 137 + np.dtype(dt).itemsize * 11 + int(np.dtype(dt).kind == "f")
            rng = np.random.default_rng(seed)
            if np.issubdtype(dt, np.integer):
                info = np.iinfo(dt)
                lo, hi = (0, 256) if dt == np.uint8 else (max(info.min, -(2**20)), min(info.max, 2**20))
                draw = lambda s: rng.integers(lo, hi, s).astype(dt)
            else:
                draw = lambda s: rng.standard_normal(s).astype(dt)
            x, w, bias = draw((B, C_in, H, W)), draw((C_out, C_in, K, K)), draw((C_out,))
            y = o.conv2d_forward(x, w, bias, S, P, which="ref_strict")
            g = draw(y.shape)
            gx, gw, _ = o.conv2d_backward(g, x, w, S, P, which="ref_strict")
            key = f"{name}_{np.dtype(dt).name}"
            out[key + "_geom"] = np.array([S, P], dtype=np.int64)
            for tag, arr in (("x", x), ("w", w), ("bias", bias), ("y", y), ("g", g), ("gx", gx), ("gw", gw)):
                out[f"{key}_{tag}"] = arr
    np.savez_compressed(HERE / "conv_golden.npz", **out)
    print("wrote", HERE / "conv_golden.npz", len(out), "arrays")


if __name__ == "__main__":
    main()
