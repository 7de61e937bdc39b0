"""Loads oracle/_ref/libttref_full.so: the UNMODIFIED reference library (CPU backend) behind C
entry points (oracle/ref_full_driver.cpp, built by oracle/dropin.mk).  Test infrastructure only.

    matmul(a, b, a_perm, b_perm)           tinytensor::matmul on permuted views of a and b
    matmul_backward(a, b, grad, ...)       gradients from Tensor::backward()
    Gen(seed).uniform_real / normal / uniform_int / next    the reference's Generator
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

PATH = Path(__file__).resolve().parent.parent / "oracle" / "_ref" / "libttref_full.so"

CODE = {np.dtype(np.bool_): 0, np.dtype(np.uint8): 1, np.dtype(np.int16): 2, np.dtype(np.int32): 3,
        np.dtype(np.int64): 4, np.dtype(np.float32): 5, np.dtype(np.float64): 6}
DTYPE = {v: k for k, v in CODE.items()}


class ReferenceError_(RuntimeError):
    """A TTException thrown by the reference."""


_lib = None


def available() -> bool:
    return PATH.exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        L = ctypes.CDLL(str(PATH))
        L.ttref_gen_new.restype = ctypes.c_void_p
        L.ttref_gen_new.argtypes = [ctypes.c_uint64]
        L.ttref_gen_free.argtypes = [ctypes.c_void_p]
        L.ttref_gen_next.restype = ctypes.c_uint64
        L.ttref_gen_next.argtypes = [ctypes.c_void_p]
        _lib = L
    return _lib


def _ints(v):
    return (ctypes.c_int * len(v))(*[int(x) for x in v]) if v is not None else None


def matmul(a: np.ndarray, b: np.ndarray, a_perm=None, b_perm=None) -> np.ndarray:
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    sa = [a.shape[i] for i in a_perm] if a_perm is not None else list(a.shape)
    sb = [b.shape[i] for i in b_perm] if b_perm is not None else list(b.shape)
    # rows of the (viewed) lhs times columns of the (viewed) rhs bounds every rank form
    cap = 8 * max(int(np.prod(sa[:-1], dtype=np.int64)) * (sb[-1] if len(sb) >= 2 else 1), 1)
    out = np.empty(cap, dtype=np.uint8)
    ndim, dtype = ctypes.c_int(), ctypes.c_int()
    shape = (ctypes.c_int * 3)()
    err = ctypes.create_string_buffer(1024)
    rc = lib().ttref_full_matmul(
        CODE[a.dtype], ctypes.c_void_p(a.ctypes.data), a.ndim, _ints(a.shape), _ints(a_perm),
        CODE[b.dtype], ctypes.c_void_p(b.ctypes.data), b.ndim, _ints(b.shape), _ints(b_perm),
        ctypes.c_void_p(out.ctypes.data), ctypes.c_int64(out.nbytes), ctypes.byref(ndim), shape, ctypes.byref(dtype),
        err, len(err))
    if rc == 1:
        raise ReferenceError_(err.value.decode())
    assert rc == 0, err.value
    dt = DTYPE[dtype.value]
    shp = tuple(shape[i] for i in range(ndim.value))
    n = int(np.prod(shp)) if shp else 1
    return out[: n * dt.itemsize].view(dt).reshape(shp).copy()


def matmul_backward(a: np.ndarray, b: np.ndarray, grad: np.ndarray, a_perm=None, b_perm=None):
    a, b, grad = np.ascontiguousarray(a), np.ascontiguousarray(b), np.ascontiguousarray(grad)
    assert a.dtype == b.dtype == grad.dtype
    ga, gb = np.empty_like(a), np.empty_like(b)
    err = ctypes.create_string_buffer(1024)
    rc = lib().ttref_full_matmul_backward(
        CODE[a.dtype], ctypes.c_void_p(a.ctypes.data), a.ndim, _ints(a.shape), _ints(a_perm),
        ctypes.c_void_p(b.ctypes.data), b.ndim, _ints(b.shape), _ints(b_perm),
        ctypes.c_void_p(grad.ctypes.data), ctypes.c_void_p(ga.ctypes.data), ctypes.c_void_p(gb.ctypes.data),
        err, len(err))
    if rc == 1:
        raise ReferenceError_(err.value.decode())
    assert rc == 0, err.value
    return ga, gb


class Gen:
    def __init__(self, seed: int):
        self._g = ctypes.c_void_p(lib().ttref_gen_new(int(seed)))

    def __del__(self):
        try:
            lib().ttref_gen_free(self._g)
        except Exception:
            pass

    def next(self) -> int:
        return int(lib().ttref_gen_next(self._g))

    def _draw(self, name, a, b, shape, dtype, int_args=False):
        out = np.empty(shape, dtype=dtype)
        err = ctypes.create_string_buffer(1024)
        ca = (ctypes.c_int64 if int_args else ctypes.c_double)
        rc = getattr(lib(), name)(self._g, ca(a), ca(b), ctypes.c_int(out.size), CODE[out.dtype],
                                  ctypes.c_void_p(out.ctypes.data), err, len(err))
        if rc != 0:
            raise ReferenceError_(err.value.decode())
        return out

    def uniform_real(self, lo, hi, shape, dtype=np.float32):
        return self._draw("ttref_uniform_real", lo, hi, shape, dtype)

    def normal(self, mu, sd, shape, dtype=np.float32):
        return self._draw("ttref_normal", mu, sd, shape, dtype)

    def uniform_int(self, lo, hi, shape, dtype=np.int32):
        return self._draw("ttref_uniform_int", lo, hi, shape, dtype, int_args=True)
