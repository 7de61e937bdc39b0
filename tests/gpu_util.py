"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

TORCH_OF = {
    np.dtype(np.uint8): torch.uint8,
    np.dtype(np.int16): torch.int16,
    np.dtype(np.int32): torch.int32,
    np.dtype(np.int64): torch.int64,
    np.dtype(np.float32): torch.float32,
    np.dtype(np.float64): torch.float64,
}


def dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def host(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def rel_to_max(got: np.ndarray, want64: np.ndarray) -> float:
    """max|c - c64| / max|c64|: the error measure of the f32/f64 gates.  An element-wise
    relative error is meaningless for sums that may land arbitrarily close to zero."""
    got = got.astype(np.float64 if want64.dtype != np.longdouble else np.longdouble)
    denom = float(np.abs(want64).max())
    return float(np.abs(got - want64).max()) / (denom if denom > 0 else 1.0)


def random_operands(rng, dt, B, N, K, M, int_lo=0, int_hi=100):
    dt = np.dtype(dt)
    if dt.kind in "iu":
        a = rng.integers(int_lo, int_hi, (B, N, K)).astype(dt)
        b = rng.integers(int_lo, int_hi, (B, K, M)).astype(dt)
    else:
        a = rng.standard_normal((B, N, K)).astype(dt)
        b = rng.standard_normal((B, K, M)).astype(dt)
    return a, b
