"""Loads the test oracle: oracle/liboracle.so (C restatement of the reference's CPU
matmul) and, when present, oracle/_ref/libttref.so (the reference's own kernel compiled
from its sources).  Test infrastructure only."""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent.parent
ORACLE_DIR = ROOT / "oracle"

_NAMES = {
    np.dtype(np.uint8): "u8",
    np.dtype(np.int16): "i16",
    np.dtype(np.int32): "i32",
    np.dtype(np.int64): "i64",
    np.dtype(np.float32): "f32",
    np.dtype(np.float64): "f64",
}


class Oracle:
    def __init__(self, port: ctypes.CDLL, ref: ctypes.CDLL | None, ref_strict: ctypes.CDLL | None = None):
        self.port = port
        self.ref = ref
        self.ref_strict = ref_strict  # same sources, floating-point contraction forbidden

    @staticmethod
    def _prep(lhs, rhs):
        # The reference makes both operands contiguous first (backend/cpu/matmul.cpp:37-38).
        lhs = np.ascontiguousarray(lhs)
        rhs = np.ascontiguousarray(rhs)
        assert lhs.ndim == 3 and rhs.ndim == 3 and lhs.dtype == rhs.dtype
        assert lhs.shape[0] == rhs.shape[0] and lhs.shape[2] == rhs.shape[1]
        B, N, K = lhs.shape
        M = rhs.shape[2]
        return lhs, rhs, B, N, K, M

    def matmul(self, lhs: np.ndarray, rhs: np.ndarray, fast: bool = True) -> np.ndarray:
        """The C restatement.  `fast` picks the loop order that streams over columns;
        both orders are bit-identical."""
        lhs, rhs, B, N, K, M = self._prep(lhs, rhs)
        out = np.empty((B, N, M), dtype=lhs.dtype)
        name = _NAMES[lhs.dtype]
        if fast:
            fn = getattr(self.port, f"oracle_matmul_fast_{name}")
            scratch = np.empty(M, dtype=lhs.dtype)
            fn(ctypes.c_void_p(lhs.ctypes.data), ctypes.c_void_p(rhs.ctypes.data), ctypes.c_void_p(out.ctypes.data),
               ctypes.c_int64(B), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int64(M),
               ctypes.c_void_p(scratch.ctypes.data))
        else:
            fn = getattr(self.port, f"oracle_matmul_{name}")
            fn(ctypes.c_void_p(lhs.ctypes.data), ctypes.c_void_p(rhs.ctypes.data), ctypes.c_void_p(out.ctypes.data),
               ctypes.c_int64(B), ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int64(M))
        return out

    def ref_matmul(self, lhs: np.ndarray, rhs: np.ndarray, strict: bool = False) -> np.ndarray:
        """The reference's own kernel (oracle/_ref/libttref.so; `strict` = the build
        without floating-point contraction)."""
        lib = self.ref_strict if strict else self.ref
        assert lib is not None, "oracle/_ref/libttref*.so has not been built"
        lhs, rhs, B, N, K, M = self._prep(lhs, rhs)
        out = np.empty((B, N, M), dtype=lhs.dtype)
        fn = getattr(lib, f"ref_matmul_{_NAMES[lhs.dtype]}")
        fn(ctypes.c_void_p(lhs.ctypes.data), ctypes.c_void_p(rhs.ctypes.data), ctypes.c_void_p(out.ctypes.data),
           ctypes.c_int64(B), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(M))
        return out


class RefCuda:
    """The reference's own CUDA matmul kernel (oracle/_ref/libttref_cuda.so), launched the way
    its runner launches it: contiguous operands, default stream."""

    def __init__(self, lib: ctypes.CDLL):
        self.lib = lib

    def matmul(self, lhs, rhs):
        import torch

        names = {torch.uint8: "u8", torch.int16: "i16", torch.int32: "i32", torch.int64: "i64",
                 torch.float32: "f32", torch.float64: "f64"}
        lhs, rhs = lhs.contiguous(), rhs.contiguous()  # backend/cuda/matmul.cu:40-41
        B, N, K = lhs.shape
        M = rhs.shape[2]
        out = torch.empty((B, N, M), dtype=lhs.dtype, device=lhs.device)
        fn = getattr(self.lib, f"ref_cuda_matmul_{names[lhs.dtype]}")
        fn.restype = ctypes.c_int
        rc = fn(ctypes.c_void_p(lhs.data_ptr()), ctypes.c_void_p(rhs.data_ptr()), ctypes.c_void_p(out.data_ptr()),
                ctypes.c_int(B), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(M),
                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, f"reference CUDA kernel launch failed: cudaError {rc}"
        return out


def load_ref_cuda():
    """None when the library was not built (no reference tree at build time)."""
    path = ORACLE_DIR / "_ref" / "libttref_cuda.so"
    return RefCuda(ctypes.CDLL(str(path))) if path.exists() else None


def load() -> Oracle:
    port = ORACLE_DIR / "liboracle.so"
    if not port.exists():
        subprocess.run(["make", "-C", str(ORACLE_DIR), str(port)], check=True, capture_output=True)
    ref = ORACLE_DIR / "_ref" / "libttref.so"
    strict = ORACLE_DIR / "_ref" / "libttref_strict.so"
    return Oracle(ctypes.CDLL(str(port)), ctypes.CDLL(str(ref)) if ref.exists() else None,
                  ctypes.CDLL(str(strict)) if strict.exists() else None)


def wrap_matmul(lhs: np.ndarray, rhs: np.ndarray) -> np.ndarray:
    """Integer matmul with wrap-around mod 2^w, the semantics of the naive loop in the
    reference's tests/test_matmul.cpp:33-46 (accumulation in T)."""
    dt = lhs.dtype
    wide = np.matmul(lhs.astype(np.uint64), rhs.astype(np.uint64))  # wraps mod 2^64
    return wide.astype(dt)  # truncation keeps the low bits
