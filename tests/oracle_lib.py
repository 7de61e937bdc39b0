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


    # ---- conv2d (oracle/conv_oracle.c; the reference's kernels in oracle/_ref/libttref*.so)
    @staticmethod
    def _conv_dims(x, w, stride, padding):
        B, C_in, H_in, W_in = x.shape
        C_out, c2, K, k2 = w.shape
        assert c2 == C_in and K == k2 and x.dtype == w.dtype
        H_out = (H_in + 2 * padding - K) // stride + 1
        W_out = (W_in + 2 * padding - K) // stride + 1
        ints = [ctypes.c_int(v) for v in (B, C_in, H_in, W_in, C_out, K, stride, padding)]
        return ints, (B, C_out, H_out, W_out)

    def _conv_lib(self, which: str):
        lib = {"port": self.port, "ref": self.ref, "ref_strict": self.ref_strict}[which]
        assert lib is not None, f"oracle library '{which}' has not been built"
        return lib, ("oracle" if which == "port" else "ref")

    def conv2d_forward(self, x, w, bias=None, stride=1, padding=0, which="port"):
        lib, prefix = self._conv_lib(which)
        x, w = np.ascontiguousarray(x), np.ascontiguousarray(w)
        ints, oshape = self._conv_dims(x, w, stride, padding)
        y = np.empty(oshape, dtype=x.dtype)
        bptr = None
        if bias is not None:
            bias = np.ascontiguousarray(bias)
            bptr = ctypes.c_void_p(bias.ctypes.data)
        fn = getattr(lib, f"{prefix}_conv2d_forward_{_NAMES[x.dtype]}")
        fn(ctypes.c_void_p(x.ctypes.data), ctypes.c_void_p(w.ctypes.data), bptr, ctypes.c_void_p(y.ctypes.data), *ints)
        return y

    def conv2d_backward(self, g, x, w, stride=1, padding=0, which="port", with_bias=True):
        """-> (grad_input, grad_weight, grad_bias or None).  The reference libraries return no
        bias gradient (the reference computes it with tensor reductions outside the runner's
        kernels, backend/cpu/conv.cpp:283)."""
        lib, prefix = self._conv_lib(which)
        g, x, w = np.ascontiguousarray(g), np.ascontiguousarray(x), np.ascontiguousarray(w)
        ints, oshape = self._conv_dims(x, w, stride, padding)
        assert g.shape == oshape and g.dtype == x.dtype
        gx, gw = np.empty_like(x), np.empty_like(w)
        fn = getattr(lib, f"{prefix}_conv2d_backward_{_NAMES[x.dtype]}")
        if which == "port":
            gb = np.empty(w.shape[0], dtype=x.dtype) if with_bias else None
            fn(ctypes.c_void_p(g.ctypes.data), ctypes.c_void_p(x.ctypes.data), ctypes.c_void_p(w.ctypes.data),
               ctypes.c_void_p(gx.ctypes.data), ctypes.c_void_p(gw.ctypes.data),
               ctypes.c_void_p(gb.ctypes.data) if gb is not None else None, *ints)
            return gx, gw, gb
        fn(ctypes.c_void_p(g.ctypes.data), ctypes.c_void_p(x.ctypes.data), ctypes.c_void_p(w.ctypes.data),
           ctypes.c_void_p(gx.ctypes.data), ctypes.c_void_p(gw.ctypes.data), *ints)
        return gx, gw, None


def conv2d_direct(x: np.ndarray, w: np.ndarray, stride: int, padding: int) -> np.ndarray:
    """The direct definition the reference's test uses as its expected value
    (tests/test_conv.cpp:28-73): Y[b,m,h,w] += T(X * W) over c, p, q, accumulated in T.
    Integers wrap (computed mod 2^64, truncated); floats are summed in float64."""
    B, C_in, H_in, W_in = x.shape
    C_out, _, K, _ = w.shape
    H_out = (H_in + 2 * padding - K) // stride + 1
    W_out = (W_in + 2 * padding - K) // stride + 1
    wide = np.uint64 if x.dtype.kind in "iu" else np.float64
    xp = np.zeros((B, C_in, H_in + 2 * padding, W_in + 2 * padding), dtype=wide)
    xp[:, :, padding:padding + H_in, padding:padding + W_in] = x.astype(wide)
    y = np.zeros((B, C_out, H_out, W_out), dtype=wide)
    ww = w.astype(wide)
    for p in range(K):
        for q in range(K):
            patch = xp[:, :, p:p + stride * (H_out - 1) + 1:stride, q:q + stride * (W_out - 1) + 1:stride]
            y += np.einsum("bchw,mc->bmhw", patch, ww[:, :, p, q])
    return y.astype(x.dtype) if x.dtype.kind in "iu" else y


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
