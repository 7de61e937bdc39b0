"""Seeded operands of the benchmark configurations, drawn the way a tinytensor program draws them.

``Generator`` mirrors tinytensor's ``Generator(seed)`` with its ``uniform_real`` / ``normal`` /
``uniform_int`` factory functions on the CPU backend (tinytensor/tensor/random.cpp:17-59,
include/tt/tensor.h:1964-2003 and :2204-2210); the arithmetic lives in libttb.so
(``ttb_generator_*``, csrc/generator.cpp) and is bit-identical to the reference library built
with the same compiler.  ``config_operands`` lists the tensors of each configuration in the
order they are drawn, one fresh generator per configuration seeded with the configuration's
seed.  Host (numpy) arrays: uploading them is the caller's business.
"""
from __future__ import annotations

import ctypes
import math

import numpy as np

from . import backend

_CODE = {np.dtype(np.float32): 5, np.dtype(np.float64): 6, np.dtype(np.int32): 3, np.dtype(np.int64): 4}


def _bind():
    L = backend.lib()
    if getattr(L, "_ttb_generator_bound", False):
        return L
    L.ttb_generator_seed.argtypes = [ctypes.c_uint64]
    L.ttb_generator_seed.restype = ctypes.c_uint64
    L.ttb_generator_next.argtypes = [ctypes.POINTER(ctypes.c_uint64)]
    L.ttb_generator_next.restype = ctypes.c_uint64
    for name in ("ttb_generator_uniform_real", "ttb_generator_normal"):
        f = getattr(L, name)
        f.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.c_double, ctypes.c_double, ctypes.c_int64, ctypes.c_int,
                      ctypes.c_void_p]
        f.restype = ctypes.c_int
    L.ttb_generator_uniform_int.argtypes = [ctypes.POINTER(ctypes.c_uint64), ctypes.c_int64, ctypes.c_int64,
                                            ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
    L.ttb_generator_uniform_int.restype = ctypes.c_int
    L._ttb_generator_bound = True
    return L


class Generator:
    """tinytensor::Generator: splitmix64 of the seed is the state, xorshift64 the outputs."""

    def __init__(self, seed: int):
        self._lib = _bind()
        self._state = ctypes.c_uint64(self._lib.ttb_generator_seed(int(seed)))

    def next(self) -> int:
        return int(self._lib.ttb_generator_next(ctypes.byref(self._state)))

    def _draw(self, fn, a, b, shape, dtype) -> np.ndarray:
        dt = np.dtype(dtype)
        if dt not in _CODE:
            raise backend.TTBError(f"unsupported dtype {dt} for a seeded draw")
        out = np.empty(shape, dtype=dt)
        rc = fn(ctypes.byref(self._state), a, b, out.size, _CODE[dt], ctypes.c_void_p(out.ctypes.data))
        if rc != 0:
            raise backend.TTBError(f"seeded draw failed with status {rc}", rc)
        return out

    def uniform_real(self, low: float, high: float, shape, dtype=np.float32) -> np.ndarray:
        """uniform_real(low, high, shape): [low, high)."""
        return self._draw(self._lib.ttb_generator_uniform_real, float(low), float(high), shape, dtype)

    def normal(self, mu: float, std: float, shape, dtype=np.float32) -> np.ndarray:
        return self._draw(self._lib.ttb_generator_normal, float(mu), float(std), shape, dtype)

    def uniform_int(self, low: int, high: int, shape, dtype=np.int32) -> np.ndarray:
        """uniform_int(low, high, shape): integers in [low, high)."""
        return self._draw(self._lib.ttb_generator_uniform_int, int(low), int(high), shape, dtype)


CONFIG_SEEDS = {"c1": 0, "c2": 1, "c3": 2, "c4": 3, "c4b": 3, "c5": 4}


def config_operands(name: str, batch_range=None) -> dict:
    """The operands of configuration `name` as host arrays, in draw order.

    c1   A, B [512,512] f32 U[-1,1)                                             seed 0
    c2   X [4096,784] U[0,1); W1 [1024,784] U[-1/sqrt(784), 1/sqrt(784));
         W2 [10,1024] U[-1/sqrt(1024), 1/sqrt(1024)); dH [4096,1024], dC [4096,10] U[-1,1)   seed 1
    c3   Q, K, V [256,128,64] f32 N(0,1)                                        seed 2
    c4   A, B [8192,8192] f32 N(0, 8192^-1/2)                                   seed 3
    c4b  A, B [4096,4096] f64 N(0, 8192^-1/2), a fresh generator                seed 3
    c5   A [64,1024,512], B [64,512,1024] i32 uniform integers in [-8, 8]       seed 4

    `batch_range` = (begin, end) keeps only those batches of c3 / c5 (the draw itself always
    covers the whole tensor, so a shard holds exactly the values the full tensor has there).
    """
    g = Generator(CONFIG_SEEDS[name])
    if name == "c1":
        return {"A": g.uniform_real(-1, 1, (512, 512)), "B": g.uniform_real(-1, 1, (512, 512))}
    if name == "c2":
        b1, b2 = 1 / math.sqrt(784), 1 / math.sqrt(1024)
        return {"X": g.uniform_real(0, 1, (4096, 784)), "W1": g.uniform_real(-b1, b1, (1024, 784)),
                "W2": g.uniform_real(-b2, b2, (10, 1024)), "dH": g.uniform_real(-1, 1, (4096, 1024)),
                "dC": g.uniform_real(-1, 1, (4096, 10))}
    if name in ("c3", "c5"):
        if name == "c3":
            ops = {k: g.normal(0, 1, (256, 128, 64)) for k in ("Q", "K", "V")}
        else:
            # the reference's uniform_int is half-open: [-8, 9) is "[-8, 8]"
            ops = {"A": g.uniform_int(-8, 9, (64, 1024, 512)), "B": g.uniform_int(-8, 9, (64, 512, 1024))}
        if batch_range is not None:
            ops = {k: np.ascontiguousarray(v[batch_range[0]:batch_range[1]]) for k, v in ops.items()}
        return ops
    if name == "c4":
        sd = 8192 ** -0.5
        return {"A": g.normal(0, sd, (8192, 8192)), "B": g.normal(0, sd, (8192, 8192))}
    if name == "c4b":
        sd = 8192 ** -0.5
        return {"A": g.normal(0, sd, (4096, 4096), np.float64), "B": g.normal(0, sd, (4096, 4096), np.float64)}
    raise backend.TTBError(f"unknown configuration {name!r}")
