"""Generates tests/golden/reference_api_golden.npz from the REFERENCE library itself.

Needs oracle/_ref/libttref_full.so (`make -f oracle/dropin.mk REF=<tinytensor tree> cpu`): the
unmodified reference, CPU backend, behind C entry points.  Stores
  * the first outputs of Generator(seed) for the configuration seeds, the first values of each
    seeded draw the benchmark configurations make, and a 64-bit digest of every full operand;
  * tinytensor::matmul on the five rank forms, with dtype promotion and permuted 3-D views;
  * the messages of the TTExceptions matmul throws for bool and mis-shaped operands;
  * lhs.grad / rhs.grad from backward() for the five rank forms and permuted views.
The fixture travels with the repository; the reference does not.

    python tests/golden/make_reference_api_golden.py
"""
import math
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent))
import ref_full  # noqa: E402

# (name, lhs shape, rhs shape, lhs perm, rhs perm): the perms are applied to the stored arrays
FORMS = [
    ("dot", (37,), (37,), None, None),
    ("vec_mat", (19,), (19, 11), None, None),
    ("mat_vec", (11, 19), (19,), None, None),
    ("mat_mat", (7, 19), (19, 5), None, None),
    ("batched", (2, 7, 19), (2, 19, 5), None, None),
    ("batched_rhs_t", (2, 7, 19), (2, 5, 19), None, (0, 2, 1)),
    ("batched_lhs_t", (2, 19, 7), (2, 19, 5), (0, 2, 1), None),
    ("batch_permuted", (7, 2, 19), (2, 19, 5), (1, 0, 2), None),
]
PROMOTIONS = [(np.uint8, np.int16), (np.int16, np.int32), (np.int32, np.int64), (np.int64, np.float32),
              (np.float32, np.float64), (np.uint8, np.float64), (np.int32, np.int32), (np.float32, np.float32)]
ERRORS = [
    ("bool", np.bool_, (4, 4), np.bool_, (4, 4)),
    ("dot_len", np.float32, (5,), np.float32, (6,)),
    ("vec_mat", np.float32, (5,), np.float32, (6, 3)),
    ("mat_vec", np.float32, (3, 5), np.float32, (6,)),
    ("mat_mat", np.float32, (3, 5), np.float32, (6, 3)),
    ("batched", np.float32, (2, 3, 5), np.float32, (2, 6, 3)),
    ("rank_3_2", np.float32, (2, 3, 5), np.float32, (5, 3)),
    ("rank_4", np.float32, (2, 2, 3, 5), np.float32, (2, 2, 5, 3)),
]


def digest(a: np.ndarray) -> np.uint64:
    """Order-sensitive 64-bit digest of the raw bits: sum over i of bits[i] * (2 i + 1), mod 2^64."""
    w = np.ascontiguousarray(a).reshape(-1)
    bits = w.view(np.uint32 if w.dtype.itemsize == 4 else np.uint64).astype(np.uint64)
    idx = np.arange(bits.size, dtype=np.uint64) * np.uint64(2) + np.uint64(1)
    with np.errstate(over="ignore"):
        return np.uint64((bits * idx).sum(dtype=np.uint64))


def draw(rng, dt, shape):
    dt = np.dtype(dt)
    if dt == np.bool_:
        return rng.integers(0, 2, shape).astype(dt)
    if dt.kind in "iu":
        return rng.integers(0, 100, shape).astype(dt)
    return rng.standard_normal(shape).astype(dt)


def config_draws(name, g):
    """The draws of one benchmark configuration, in order, from generator g."""
    if name == "c1":
        return [("A", g.uniform_real(-1, 1, (512, 512))), ("B", g.uniform_real(-1, 1, (512, 512)))]
    if name == "c2":
        b1, b2 = 1 / math.sqrt(784), 1 / math.sqrt(1024)
        return [("X", g.uniform_real(0, 1, (4096, 784))), ("W1", g.uniform_real(-b1, b1, (1024, 784))),
                ("W2", g.uniform_real(-b2, b2, (10, 1024))), ("dH", g.uniform_real(-1, 1, (4096, 1024))),
                ("dC", g.uniform_real(-1, 1, (4096, 10)))]
    if name == "c3":
        return [(k, g.normal(0, 1, (256, 128, 64))) for k in ("Q", "K", "V")]
    if name == "c4":
        return [(k, g.normal(0, 8192 ** -0.5, (8192, 8192))) for k in ("A", "B")]
    if name == "c4b":
        return [(k, g.normal(0, 8192 ** -0.5, (4096, 4096), np.float64)) for k in ("A", "B")]
    if name == "c5":
        return [("A", g.uniform_int(-8, 9, (64, 1024, 512))), ("B", g.uniform_int(-8, 9, (64, 512, 1024)))]
    raise ValueError(name)


CONFIG_SEEDS = {"c1": 0, "c2": 1, "c3": 2, "c4": 3, "c4b": 3, "c5": 4}


def main():
    assert ref_full.available(), "build oracle/_ref/libttref_full.so first (oracle/dropin.mk, target cpu)"
    out = {}
    for seed in range(5):
        g = ref_full.Gen(seed)
        out[f"gen_raw_{seed}"] = np.array([g.next() for _ in range(16)], dtype=np.uint64)
    for name, seed in CONFIG_SEEDS.items():
        g = ref_full.Gen(seed)
        for key, arr in config_draws(name, g):
            out[f"cfg_{name}_{key}_head"] = arr.reshape(-1)[:64].copy()
            out[f"cfg_{name}_{key}_digest"] = np.array([digest(arr)], dtype=np.uint64)
    rng = np.random.default_rng(2024)
    for name, ls, rs, lp, rp in FORMS:
        for dl, dr in PROMOTIONS:
            a, b = draw(rng, dl, ls), draw(rng, dr, rs)
            key = f"mm_{name}_{np.dtype(dl).name}_{np.dtype(dr).name}"
            out[key + "_lhs"], out[key + "_rhs"] = a, b
            out[key + "_out"] = ref_full.matmul(a, b, lp, rp)
        for dt in (np.float64, np.float32):
            a, b = draw(rng, dt, ls), draw(rng, dt, rs)
            r = ref_full.matmul(a, b, lp, rp)
            grad = draw(rng, dt, r.shape)
            ga, gb = ref_full.matmul_backward(a, b, grad, lp, rp)
            key = f"bw_{name}_{np.dtype(dt).name}"
            out[key + "_lhs"], out[key + "_rhs"], out[key + "_grad"] = a, b, grad
            out[key + "_glhs"], out[key + "_grhs"] = ga, gb
    for name, dl, ls, dr, rs in ERRORS:
        try:
            ref_full.matmul(draw(rng, dl, ls), draw(rng, dr, rs))
            msg = ""
        except ref_full.ReferenceError_ as e:
            # keep the message proper; the what() text starts with file, line and function
            msg = str(e).split("TinyTensor Error: ", 1)[-1].strip()
        assert msg, f"the reference did not throw for {name}"
        out[f"err_{name}"] = np.array(msg)
    np.savez_compressed(HERE / "reference_api_golden.npz", **out)
    print("wrote", HERE / "reference_api_golden.npz", len(out), "arrays")


if __name__ == "__main__":
    main()
