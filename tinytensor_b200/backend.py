"""ctypes binding of libttb.so and the host-side mirror of tinytensor's matmul entry.

Mirrors (reference paths relative to the tinytensor tree):
  * ``matmul``            -> tinytensor::matmul, tinytensor/tensor/tensor.cpp:2390-2484
  * ``batched_matmul``    -> BackendCUDA::batched_matmul / cuda::batched_matmul_runner,
                             tinytensor/tensor/backend/cuda/matmul.cu:26-78
  * ``TTBError``          -> TTException, include/tt/exception.h:15-25
"""
from __future__ import annotations

import ctypes
import enum
import os
from pathlib import Path

import numpy as np
import torch

_PKG = Path(__file__).resolve().parent
_LIB_NAME = "libttb.so"


class TTBError(RuntimeError):
    """Raised for every error the reference reports with TTException, and for any
    non-zero status of the C ABI."""

    def __init__(self, message: str, status: int = -1):
        super().__init__(message)
        self.status = status


class Variant(enum.IntEnum):
    AUTO = 0
    SIMT = 1
    TCGEN05_3XTF32 = 2
    DMMA_F64 = 3
    SIMT_SPLITK = 4
    TCGEN05_2CTA = 5
    TCGEN05_I8LIMB = 6
    SIMT_SKINNY = 7


class _View(ctypes.Structure):
    _fields_ = [
        ("data", ctypes.c_void_p),
        ("offset", ctypes.c_int64),
        ("size", ctypes.c_int64 * 3),
        ("stride", ctypes.c_int64 * 3),
    ]


# tinytensor::ScalarType values (include/tt/scalar.h:21-29).
_DTYPE_CODE = {
    torch.bool: 0,
    torch.uint8: 1,
    torch.int16: 2,
    torch.int32: 3,
    torch.int64: 4,
    torch.float32: 5,
    torch.float64: 6,
}
_NP_DTYPE_CODE = {
    np.dtype(np.bool_): 0,
    np.dtype(np.uint8): 1,
    np.dtype(np.int16): 2,
    np.dtype(np.int32): 3,
    np.dtype(np.int64): 4,
    np.dtype(np.float32): 5,
    np.dtype(np.float64): 6,
}
# promote_type_map of the reference (tinytensor/common/scalar.cpp:17-26): the
# promoted type is the one with the larger enum value.
_CODE_DTYPE = {v: k for k, v in _DTYPE_CODE.items()}
# to_string(ScalarType) of the reference (include/tt/scalar.h:76-93), used in its error messages.
_CODE_NAME = ("bool8", "uint8", "int16", "int32", "int64", "float32", "float64")


def _shape_str(t) -> str:
    """A shape as the reference prints it: (3, 5)."""
    return "(" + ", ".join(str(int(d)) for d in t.shape) + ")"

_lib = None


def lib_path() -> Path:
    override = os.environ.get("TTB_LIBRARY")
    return Path(override) if override else _PKG / _LIB_NAME


def lib() -> ctypes.CDLL:
    """Loads libttb.so (once).  Raises if it has not been built: there is no fallback."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not path.exists():
        raise TTBError(
            f"{path} not found: build it with `python -m tinytensor_b200.build` "
            "(this package has no CPU or eager fallback)"
        )
    L = ctypes.CDLL(str(path))
    vp = ctypes.POINTER(_View)
    L.ttb_batched_matmul.argtypes = [vp, vp, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    L.ttb_batched_matmul.restype = ctypes.c_int
    L.ttb_batched_matmul_strided_out.argtypes = [
        vp, vp, ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64), ctypes.c_int, ctypes.c_int,
        ctypes.c_void_p,
    ]
    L.ttb_batched_matmul_strided_out.restype = ctypes.c_int
    L.ttb_batched_matmul_fused.argtypes = [
        vp, vp, ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64), vp, ctypes.c_int, ctypes.c_int,
        ctypes.c_int, ctypes.c_void_p]
    L.ttb_batched_matmul_fused.restype = ctypes.c_int
    L.ttb_conv2d_forward.argtypes = [ctypes.c_void_p] * 4 + [ctypes.POINTER(_ConvDesc), ctypes.c_int, ctypes.c_int,
                                     ctypes.c_void_p]
    L.ttb_conv2d_forward.restype = ctypes.c_int
    L.ttb_conv2d_backward.argtypes = [ctypes.c_void_p] * 6 + [ctypes.POINTER(_ConvDesc), ctypes.c_int, ctypes.c_int,
                                      ctypes.c_void_p]
    L.ttb_conv2d_backward.restype = ctypes.c_int
    L.ttb_matmul_allgather.argtypes = [
        vp, vp, ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_void_p),
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    L.ttb_matmul_allgather.restype = ctypes.c_int
    L.ttb_matmul_allgather_multicast.argtypes = [
        vp, vp, ctypes.c_void_p, ctypes.c_int64, ctypes.POINTER(ctypes.c_int64), ctypes.c_void_p, ctypes.c_int,
        ctypes.c_int, ctypes.c_void_p]
    L.ttb_matmul_allgather_multicast.restype = ctypes.c_int
    L.ttb_batched_matmul_static_scratch.argtypes = [vp, vp, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                                                    ctypes.c_void_p]
    L.ttb_batched_matmul_static_scratch.restype = ctypes.c_int
    L.ttb_batched_matmul_host.argtypes = [vp, vp, ctypes.c_void_p, ctypes.c_int, ctypes.c_int]
    L.ttb_batched_matmul_host.restype = ctypes.c_int
    L.ttb_partition.argtypes = [ctypes.c_int64] * 4 + [ctypes.c_int, ctypes.c_int, ctypes.c_int64,
                                                      ctypes.POINTER(ctypes.c_int64), ctypes.POINTER(ctypes.c_int64)]
    L.ttb_partition.restype = ctypes.c_int
    L.ttb_last_error.restype = ctypes.c_char_p
    L.ttb_last_variant.restype = ctypes.c_int
    L.ttb_launch_count.restype = ctypes.c_int64
    L.ttb_variant_name.argtypes = [ctypes.c_int]
    L.ttb_variant_name.restype = ctypes.c_char_p
    L.ttb_set_option.argtypes = [ctypes.c_char_p, ctypes.c_int64]
    L.ttb_set_option.restype = ctypes.c_int
    L.ttb_get_option.argtypes = [ctypes.c_char_p]
    L.ttb_get_option.restype = ctypes.c_int64
    L.ttb_device_count.restype = ctypes.c_int
    L.ttb_check_device.argtypes = [ctypes.c_int]
    L.ttb_check_device.restype = ctypes.c_int
    L.ttb_device_alloc.argtypes = [ctypes.POINTER(ctypes.c_void_p), ctypes.c_uint64, ctypes.c_int, ctypes.c_void_p]
    L.ttb_device_alloc.restype = ctypes.c_int
    L.ttb_device_free.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p]
    L.ttb_device_free.restype = ctypes.c_int
    L.ttb_device_memory_stats.argtypes = [ctypes.c_int] + [ctypes.POINTER(ctypes.c_uint64)] * 3
    L.ttb_device_memory_stats.restype = ctypes.c_int
    L.ttb_device_trim.argtypes = [ctypes.c_int]
    L.ttb_device_trim.restype = ctypes.c_int
    L.ttb_copy_device_to_device.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                            ctypes.c_uint64, ctypes.c_void_p]
    L.ttb_copy_device_to_device.restype = ctypes.c_int
    L.ttb_view_tma_eligible.argtypes = [vp, ctypes.c_int, ctypes.c_int]
    L.ttb_view_tma_eligible.restype = ctypes.c_int
    L.ttb_version.restype = ctypes.c_int
    _lib = L
    return L


def _raise(status: int) -> None:
    msg = lib().ttb_last_error().decode("utf-8", "replace")
    raise TTBError(msg or f"ttb status {status}", status)


def _make_view(data_ptr: int, offset: int, sizes, strides) -> _View:
    v = _View()
    v.data = data_ptr
    v.offset = int(offset)
    for i in range(3):
        v.size[i] = int(sizes[i])
        v.stride[i] = int(strides[i])
    return v


def view_of(t: torch.Tensor) -> _View:
    """The (storage base, element offset, shape, element strides) of a rank-3 torch
    tensor, i.e. the fields a tinytensor Tensor carries (include/tt/tensor.h:1570-1577)."""
    if t.dim() != 3:
        raise TTBError(f"expected a rank-3 tensor, got rank {t.dim()}")
    return _make_view(t.untyped_storage().data_ptr(), t.storage_offset(), t.shape, t.stride())


def set_option(key: str, value: int) -> None:
    rc = lib().ttb_set_option(key.encode(), int(value))
    if rc != 0:
        _raise(rc)


def get_option(key: str) -> int:
    return int(lib().ttb_get_option(key.encode()))


def last_variant() -> Variant:
    return Variant(lib().ttb_last_variant())


def launch_count() -> int:
    return int(lib().ttb_launch_count())


def check_device(device: int = 0) -> None:
    """Synchronises `device` and raises if a bounded wait inside a kernel gave up."""
    rc = lib().ttb_check_device(int(device))
    if rc != 0:
        _raise(rc)


def measure_fp64_tensor_peak(device: int = 0) -> float:
    """FP64 tensor-core rate of `device` in TFLOP/s from a register-only loop of the f64 kernel's MMA."""
    L = lib()
    L.ttb_measure_fp64_tensor_peak.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    L.ttb_measure_fp64_tensor_peak.restype = ctypes.c_int
    out = ctypes.c_double()
    rc = L.ttb_measure_fp64_tensor_peak(int(device), ctypes.byref(out))
    if rc != 0:
        _raise(rc)
    return out.value


def tma_eligible(t: torch.Tensor, operand: int) -> bool:
    v = view_of(t)
    return bool(lib().ttb_view_tma_eligible(ctypes.byref(v), _DTYPE_CODE[t.dtype], operand))


def _stream_ptr(stream) -> int:
    if stream is None:
        stream = torch.cuda.current_stream()
    return int(stream.cuda_stream)


def batched_matmul(lhs: torch.Tensor, rhs: torch.Tensor, out: torch.Tensor | None = None, stream=None) -> torch.Tensor:
    """lhs[B,N,K] . rhs[B,K,M] -> [B,N,M] on the operands' CUDA device.

    The backend operator of the reference (backend_base.h:130): rank-3 operands of one
    dtype on one device, any strides; the result is a fresh contiguous tensor unless
    `out` (rank 3, any strides) is given.  Queued on the current torch stream; does not
    synchronise.
    """
    if lhs.dim() != 3 or rhs.dim() != 3:
        raise TTBError(f"batched_matmul expects rank-3 operands, got {lhs.dim()} and {rhs.dim()}")
    if lhs.device != rhs.device:
        raise TTBError(f"Expected tensors to be on the same device. Given {lhs.device} and {rhs.device}")
    if lhs.device.type != "cuda":
        raise TTBError("tinytensor_b200 only runs on CUDA devices (no CPU fallback)")
    if lhs.dtype != rhs.dtype:
        raise TTBError(f"operands must share a dtype after promotion, got {lhs.dtype} and {rhs.dtype}")
    if lhs.dtype not in _DTYPE_CODE:
        raise TTBError(f"unsupported dtype {lhs.dtype}")
    code = _DTYPE_CODE[lhs.dtype]
    dev = lhs.device.index if lhs.device.index is not None else torch.cuda.current_device()
    lv, rv = view_of(lhs), view_of(rhs)
    L = lib()
    if out is None:
        if lhs.shape[0] != rhs.shape[0] or lhs.shape[2] != rhs.shape[1] or code == 0:
            # Let the library produce the message; nothing is allocated or launched.
            dummy = ctypes.c_void_p(8)
            rc = L.ttb_batched_matmul(ctypes.byref(lv), ctypes.byref(rv), dummy, code, dev, None)
            _raise(rc if rc != 0 else -1)
        with torch.cuda.device(dev):
            out = torch.empty((lhs.shape[0], lhs.shape[1], rhs.shape[2]), dtype=lhs.dtype, device=lhs.device)
        rc = L.ttb_batched_matmul(ctypes.byref(lv), ctypes.byref(rv), ctypes.c_void_p(out.data_ptr()), code, dev,
                                  ctypes.c_void_p(_stream_ptr(stream)))
    else:
        if out.dim() != 3 or tuple(out.shape) != (lhs.shape[0], lhs.shape[1], rhs.shape[2]):
            raise TTBError(f"out has shape {tuple(out.shape)}, expected "
                           f"{(lhs.shape[0], lhs.shape[1], rhs.shape[2])}")
        if out.dtype != lhs.dtype or out.device != lhs.device:
            raise TTBError("out must have the operands' dtype and device")
        strides = (ctypes.c_int64 * 3)(*out.stride())
        rc = L.ttb_batched_matmul_strided_out(
            ctypes.byref(lv), ctypes.byref(rv), ctypes.c_void_p(out.untyped_storage().data_ptr()),
            out.storage_offset(), strides, code, dev, ctypes.c_void_p(_stream_ptr(stream)))
    if rc != 0:
        _raise(rc)
    return out


class PreparedMatmul:
    """``lhs . rhs -> out`` with the C ABI's argument structures built once.

    ``batched_matmul`` checks its tensors and fills two ``ttb_view`` structures on every call,
    which in Python costs far more than the call itself; a C++ host (the tinytensor-side adapter)
    fills the same two structures in nanoseconds.  A prepared product is that host's view of the
    cost: calling it is one foreign call into ``ttb_batched_matmul_strided_out`` with the very
    same arguments.  The tensors must stay alive and in place; the stream is the one current at
    preparation unless one is passed to the call."""

    def __init__(self, lhs: torch.Tensor, rhs: torch.Tensor, out: torch.Tensor, stream=None):
        if lhs.dim() != 3 or rhs.dim() != 3 or out.dim() != 3:
            raise TTBError("PreparedMatmul expects rank-3 tensors")
        if not (lhs.device == rhs.device == out.device) or lhs.device.type != "cuda":
            raise TTBError("PreparedMatmul: operands and result must share a CUDA device")
        if not (lhs.dtype == rhs.dtype == out.dtype) or lhs.dtype not in _DTYPE_CODE:
            raise TTBError("PreparedMatmul: operands and result must share a supported dtype")
        if tuple(out.shape) != (lhs.shape[0], lhs.shape[1], rhs.shape[2]):
            raise TTBError(f"out has shape {tuple(out.shape)}, expected {(lhs.shape[0], lhs.shape[1], rhs.shape[2])}")
        self._keep = (lhs, rhs, out)
        self._lv, self._rv = view_of(lhs), view_of(rhs)
        self._strides = (ctypes.c_int64 * 3)(*out.stride())
        dev = lhs.device.index if lhs.device.index is not None else torch.cuda.current_device()
        self._fn = lib().ttb_batched_matmul_strided_out
        self._stream = ctypes.c_void_p(_stream_ptr(stream))
        self._args = (ctypes.byref(self._lv), ctypes.byref(self._rv), ctypes.c_void_p(out.untyped_storage().data_ptr()),
                      out.storage_offset(), self._strides, _DTYPE_CODE[lhs.dtype], dev)

    def __call__(self, stream=None) -> torch.Tensor:
        rc = self._fn(*self._args, self._stream if stream is None else ctypes.c_void_p(_stream_ptr(stream)))
        if rc != 0:
            _raise(rc)
        return self._keep[2]


def tensor_map_cache_stats():
    """(hits, misses) of this thread's tensor-map cache (ttb_tensor_map_cache_stats)."""
    L = lib()
    L.ttb_tensor_map_cache_stats.argtypes = [ctypes.POINTER(ctypes.c_uint64)] * 2
    L.ttb_tensor_map_cache_stats.restype = None
    h, m = ctypes.c_uint64(), ctypes.c_uint64()
    L.ttb_tensor_map_cache_stats(ctypes.byref(h), ctypes.byref(m))
    return h.value, m.value


class Activation(enum.IntEnum):
    NONE = 0
    RELU = 1


def batched_matmul_fused(lhs: torch.Tensor, rhs: torch.Tensor, addend: torch.Tensor | None = None,
                         activation: Activation = Activation.NONE, out: torch.Tensor | None = None,
                         stream=None) -> torch.Tensor:
    """``ttb_batched_matmul_fused``: act(lhs . rhs + addend) in one kernel.

    `addend` is anything that expands to the result shape [B,N,M] without a copy: a bias over
    columns ([M]), over rows ([N,1]), a full tensor, or `out` itself (accumulation,
    out += lhs . rhs).  Replaces the reference's matmul + expand + add (nn/linear.cpp:45-48),
    conv2d's per-image bias add (backend/cuda/conv.cu:163-183) and add_grad's second kernel
    (tensor/tensor.cpp:1137-1160)."""
    if lhs.dim() != 3 or rhs.dim() != 3 or lhs.dtype != rhs.dtype or lhs.device != rhs.device:
        raise TTBError("operands must be rank-3 tensors of one dtype on one device")
    if lhs.device.type != "cuda":
        raise TTBError("tinytensor_b200 only runs on CUDA devices (no CPU fallback)")
    if lhs.dtype not in _DTYPE_CODE:
        raise TTBError(f"unsupported dtype {lhs.dtype}")
    shape = (lhs.shape[0], lhs.shape[1], rhs.shape[2])
    dev = lhs.device.index if lhs.device.index is not None else torch.cuda.current_device()
    if out is None:
        if lhs.shape[0] != rhs.shape[0] or lhs.shape[2] != rhs.shape[1]:
            raise TTBError(f"shapes {tuple(lhs.shape)} and {tuple(rhs.shape)} do not multiply")
        with torch.cuda.device(dev):
            out = torch.empty(shape, dtype=lhs.dtype, device=lhs.device)
    elif tuple(out.shape) != shape or out.dtype != lhs.dtype or out.device != lhs.device:
        raise TTBError(f"out must be a {shape} tensor of the operands' dtype and device")
    av = None
    if addend is not None:
        if addend.dtype != lhs.dtype or addend.device != lhs.device:
            raise TTBError("addend must have the operands' dtype and device")
        try:
            av = view_of(addend.expand(shape))
        except RuntimeError as e:
            raise TTBError(f"addend of shape {tuple(addend.shape)} does not expand to {shape}") from e
    lv, rv = view_of(lhs), view_of(rhs)
    strides = (ctypes.c_int64 * 3)(*out.stride())
    rc = lib().ttb_batched_matmul_fused(
        ctypes.byref(lv), ctypes.byref(rv), ctypes.c_void_p(out.untyped_storage().data_ptr()), out.storage_offset(),
        strides, ctypes.byref(av) if av is not None else None, int(activation), _DTYPE_CODE[lhs.dtype], dev,
        ctypes.c_void_p(_stream_ptr(stream)))
    if rc != 0:
        _raise(rc)
    return out


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None,
           activation: Activation = Activation.NONE) -> torch.Tensor:
    """tinytensor's Linear.forward (nn/linear.cpp:41-50): x[..., in] . weight[in, out] + bias[out],
    as one fused kernel (the reference runs matmul, expand and a binary add)."""
    if weight.dim() != 2 or x.shape[-1] != weight.shape[0]:
        raise TTBError(f"linear: x[..., {x.shape[-1]}] does not match weight {tuple(weight.shape)}")
    x2 = x.reshape(1, -1, x.shape[-1])
    out = batched_matmul_fused(x2, weight.unsqueeze(0), bias, activation)
    return out.reshape(*x.shape[:-1], weight.shape[1])


class _ConvDesc(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int64) for n in ("batch", "c_in", "h_in", "w_in", "c_out", "kernel", "stride", "padding")]


def _conv_desc(input: torch.Tensor, weight: torch.Tensor, stride: int, padding: int):
    if input.dim() != 4 or weight.dim() != 4:
        raise TTBError(f"conv2d expects rank-4 input and weight, got {input.dim()} and {weight.dim()}")
    if input.shape[1] != weight.shape[1] or weight.shape[2] != weight.shape[3]:
        raise TTBError(f"conv2d: input {tuple(input.shape)} does not match weight {tuple(weight.shape)} "
                       "(channels must agree, kernels are square)")
    if input.dtype != weight.dtype or input.device != weight.device or input.device.type != "cuda":
        raise TTBError("conv2d: input and weight must share a dtype and a CUDA device")
    if input.dtype not in _DTYPE_CODE:
        raise TTBError(f"unsupported dtype {input.dtype}")
    B, C_in, H_in, W_in = input.shape
    d = _ConvDesc(B, C_in, H_in, W_in, weight.shape[0], weight.shape[2], int(stride), int(padding))
    h_out = (H_in + 2 * padding - weight.shape[2]) // stride + 1 if stride > 0 else 0
    w_out = (W_in + 2 * padding - weight.shape[2]) // stride + 1 if stride > 0 else 0
    return d, (B, weight.shape[0], h_out, w_out)


def conv2d(input: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None = None, stride: int = 1,
           padding: int = 0, stream=None) -> torch.Tensor:
    """tinytensor's conv2d forward (backend/cuda/conv.cu:37-197) through ``ttb_conv2d_forward``:
    input [B,C_in,H,W], weight [C_out,C_in,K,K], bias [C_out] -> [B,C_out,H_out,W_out]."""
    d, oshape = _conv_desc(input, weight, stride, padding)
    input, weight = input.contiguous(), weight.contiguous()  # conv.cu:77
    if bias is not None:
        if bias.shape != (weight.shape[0],) or bias.dtype != input.dtype or bias.device != input.device:
            raise TTBError("conv2d: bias must be [C_out] of the input's dtype and device")
        bias = bias.contiguous()
    dev = input.device.index if input.device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(dev):
        out = torch.empty([max(v, 0) for v in oshape], dtype=input.dtype, device=input.device)
    rc = lib().ttb_conv2d_forward(ctypes.c_void_p(input.data_ptr()), ctypes.c_void_p(weight.data_ptr()),
                                  ctypes.c_void_p(bias.data_ptr()) if bias is not None else None,
                                  ctypes.c_void_p(out.data_ptr()), ctypes.byref(d), _DTYPE_CODE[input.dtype], dev,
                                  ctypes.c_void_p(_stream_ptr(stream)))
    if rc != 0:
        _raise(rc)
    return out


def conv2d_backward(grad_output: torch.Tensor, input: torch.Tensor, weight: torch.Tensor, stride: int = 1,
                    padding: int = 0, with_bias: bool = True, stream=None):
    """conv2d backward (backend/cuda/conv.cu:199-403) through ``ttb_conv2d_backward``:
    -> (grad_input, grad_weight, grad_bias or None)."""
    d, oshape = _conv_desc(input, weight, stride, padding)
    if tuple(grad_output.shape) != tuple(oshape) or grad_output.dtype != input.dtype or grad_output.device != input.device:
        raise TTBError(f"conv2d backward: grad_output must be {tuple(oshape)} of the input's dtype and device")
    grad_output, input, weight = grad_output.contiguous(), input.contiguous(), weight.contiguous()
    dev = input.device.index if input.device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(dev):
        gx, gw = torch.empty_like(input), torch.empty_like(weight)
        gb = torch.empty(weight.shape[0], dtype=input.dtype, device=input.device) if with_bias else None
    rc = lib().ttb_conv2d_backward(ctypes.c_void_p(grad_output.data_ptr()), ctypes.c_void_p(input.data_ptr()),
                                   ctypes.c_void_p(weight.data_ptr()), ctypes.c_void_p(gx.data_ptr()),
                                   ctypes.c_void_p(gw.data_ptr()),
                                   ctypes.c_void_p(gb.data_ptr()) if gb is not None else None, ctypes.byref(d),
                                   _DTYPE_CODE[input.dtype], dev, ctypes.c_void_p(_stream_ptr(stream)))
    if rc != 0:
        _raise(rc)
    return gx, gw, gb


def matmul_allgather(lhs: torch.Tensor, rhs: torch.Tensor, out: torch.Tensor, peer_bases, stream=None) -> torch.Tensor:
    """``ttb_matmul_allgather``: lhs . rhs into `out` (a rank-3, possibly strided view of this
    rank's full C) and, tile by tile from inside the GEMM kernel, into the same place of every
    peer's C.  `peer_bases` are device pointers to the START of the peers' C storages, mapped
    into this process (e.g. ``symmetric_memory`` buffer pointers); the peers' buffers must be laid
    out like this rank's.  f32 on the tensor-core kernel only.  The caller synchronises the
    ranks afterwards."""
    if lhs.dtype != torch.float32 or rhs.dtype != torch.float32 or out.dtype != torch.float32:
        raise TTBError("matmul_allgather: f32 only")
    if out.dim() != 3 or tuple(out.shape) != (lhs.shape[0], lhs.shape[1], rhs.shape[2]):
        raise TTBError("matmul_allgather: out has the wrong shape")
    dev = lhs.device.index if lhs.device.index is not None else torch.cuda.current_device()
    lv, rv = view_of(lhs), view_of(rhs)
    strides = (ctypes.c_int64 * 3)(*out.stride())
    peers = (ctypes.c_void_p * max(len(peer_bases), 1))(*[ctypes.c_void_p(int(p)) for p in peer_bases])
    rc = lib().ttb_matmul_allgather(ctypes.byref(lv), ctypes.byref(rv), ctypes.c_void_p(out.untyped_storage().data_ptr()),
                                out.storage_offset(), strides, peers, len(peer_bases), _DTYPE_CODE[lhs.dtype], dev,
                                ctypes.c_void_p(_stream_ptr(stream)))
    if rc != 0:
        _raise(rc)
    return out


def matmul_allgather_multicast(lhs: torch.Tensor, rhs: torch.Tensor, out: torch.Tensor, multicast_base: int,
                               stream=None) -> torch.Tensor:
    """``ttb_matmul_allgather_multicast``: like matmul_allgather, but every finished tile is stored
    once to the NVSwitch multicast address of C (`multicast_base`: the multicast pointer of the
    symmetric buffer that holds `out`), which delivers it to every GPU."""
    if lhs.dtype != torch.float32 or rhs.dtype != torch.float32 or out.dtype != torch.float32:
        raise TTBError("matmul_allgather_multicast: f32 only")
    if out.dim() != 3 or tuple(out.shape) != (lhs.shape[0], lhs.shape[1], rhs.shape[2]):
        raise TTBError("matmul_allgather_multicast: out has the wrong shape")
    dev = lhs.device.index if lhs.device.index is not None else torch.cuda.current_device()
    lv, rv = view_of(lhs), view_of(rhs)
    strides = (ctypes.c_int64 * 3)(*out.stride())
    rc = lib().ttb_matmul_allgather_multicast(
        ctypes.byref(lv), ctypes.byref(rv), ctypes.c_void_p(out.untyped_storage().data_ptr()), out.storage_offset(),
        strides, ctypes.c_void_p(int(multicast_base)), _DTYPE_CODE[lhs.dtype], dev, ctypes.c_void_p(_stream_ptr(stream)))
    if rc != 0:
        _raise(rc)
    return out


def batched_matmul_static_scratch(lhs: torch.Tensor, rhs: torch.Tensor, out: torch.Tensor, stream=None) -> torch.Tensor:
    """The product through ``ttb_batched_matmul_static_scratch``: for callers that own all device
    memory themselves (or cannot take cudaMalloc's device-wide synchronisation) the library
    allocates nothing -- the caller passes `out` (contiguous [B,N,M]) and the K-split partial
    sums live in a fixed 16 MiB device array.  Results above that limit raise TTBError.  Calls
    that may overlap on the GPU race on the shared array; keep them on one stream."""
    if lhs.dim() != 3 or rhs.dim() != 3 or lhs.dtype != rhs.dtype or lhs.device != rhs.device:
        raise TTBError("operands must be rank-3 tensors of one dtype on one device")
    if lhs.dtype not in _DTYPE_CODE:
        raise TTBError(f"unsupported dtype {lhs.dtype}")
    want = (lhs.shape[0], lhs.shape[1], rhs.shape[2])
    if tuple(out.shape) != want or not out.is_contiguous() or out.dtype != lhs.dtype or out.device != lhs.device:
        raise TTBError(f"out must be a contiguous {want} tensor of the operands' dtype and device")
    dev = lhs.device.index if lhs.device.index is not None else torch.cuda.current_device()
    lv, rv = view_of(lhs), view_of(rhs)
    rc = lib().ttb_batched_matmul_static_scratch(ctypes.byref(lv), ctypes.byref(rv), ctypes.c_void_p(out.data_ptr()),
                                                 _DTYPE_CODE[lhs.dtype], dev, ctypes.c_void_p(_stream_ptr(stream)))
    if rc != 0:
        _raise(rc)
    return out


def _stream_ptr_on(stream, device: int) -> int:
    if stream is None:
        stream = torch.cuda.current_stream(int(device))
    return int(stream.cuda_stream)


def device_alloc(nbytes: int, device: int = 0, stream=None) -> int:
    """Stream-ordered cached allocation (ttb_device_alloc): the address of `nbytes` bytes on `device`,
    usable by work enqueued on `stream` from now on.  Replaces the cudaMalloc of the reference's
    DeviceMemory<T> (tinytensor/tensor/backend/cuda/data_types.cu:38-50)."""
    p = ctypes.c_void_p()
    rc = lib().ttb_device_alloc(ctypes.byref(p), int(nbytes), int(device), _stream_ptr_on(stream, device))
    if rc != 0:
        _raise(rc)
    return p.value or 0


def device_free(ptr: int, device: int = 0, stream=None) -> None:
    """Give a block of device_alloc back to the pool, in stream order (ttb_device_free; the
    reference's cudaFree, data_types.cu:102-116)."""
    rc = lib().ttb_device_free(ctypes.c_void_p(ptr), int(device), _stream_ptr_on(stream, device))
    if rc != 0:
        _raise(rc)


def device_memory_stats(device: int = 0) -> dict:
    """Byte counters of device_alloc: `current`, `total` (as StorageCUDA::current_bytes_allocated and
    total_bytes_allocated, backend/cuda/storage_cuda.h:66) and `reserved` (held by the pool)."""
    cur, tot, res = ctypes.c_uint64(), ctypes.c_uint64(), ctypes.c_uint64()
    rc = lib().ttb_device_memory_stats(int(device), ctypes.byref(cur), ctypes.byref(tot), ctypes.byref(res))
    if rc != 0:
        _raise(rc)
    return {"current": cur.value, "total": tot.value, "reserved": res.value}


def device_trim(device: int = 0) -> None:
    rc = lib().ttb_device_trim(int(device))
    if rc != 0:
        _raise(rc)


def to_device(t: torch.Tensor, device: int, stream=None) -> torch.Tensor:
    """Tensor::to(Device) between GPUs as one peer copy (ttb_copy_device_to_device) instead of the
    reference's bounce through a host vector (tinytensor/autograd/unary_ops.cpp:67-83).  The
    source is made contiguous first, as to_vec does."""
    if not t.is_cuda:
        raise TTBError("to_device: the source must be a CUDA tensor")
    src = t.contiguous()
    out = torch.empty(src.shape, dtype=src.dtype, device=f"cuda:{int(device)}")
    if src.device.index != int(device) and stream is None:
        # the copy runs on the destination's stream: order it after the source's pending work
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(src.device))
        torch.cuda.current_stream(int(device)).wait_event(ready)
    rc = lib().ttb_copy_device_to_device(out.data_ptr(), int(device), src.data_ptr(), src.device.index,
                                         src.numel() * src.element_size(), _stream_ptr_on(stream, device))
    if rc != 0:
        _raise(rc)
    return out


def _promote(lhs: torch.Tensor, rhs: torch.Tensor):
    if lhs.dtype not in _DTYPE_CODE or rhs.dtype not in _DTYPE_CODE:
        raise TTBError("Unknown ScalarType")
    code = max(_DTYPE_CODE[lhs.dtype], _DTYPE_CODE[rhs.dtype])
    if code == 0:
        raise TTBError("matmul does not support boolean tensors. Given "
                       f"{_CODE_NAME[_DTYPE_CODE[lhs.dtype]]}, {_CODE_NAME[_DTYPE_CODE[rhs.dtype]]}")
    dt = _CODE_DTYPE[code]
    # A cast yields a contiguous tensor in the reference too (backend/cuda/cast.cu:25-32).
    return (lhs if lhs.dtype == dt else lhs.to(dt)), (rhs if rhs.dtype == dt else rhs.to(dt))


def matmul(lhs: torch.Tensor, rhs: torch.Tensor) -> torch.Tensor:
    """tinytensor::matmul (tensor.cpp:2390-2484): dtype promotion, bool rejected, and the
    five rank forms funnelled into one rank-3 batched product.  No broadcasting of batch
    dims.  Unlike the reference, 2-D strided operands are passed as views (the reference's
    reshape clones them first, tensor.cpp:1386); the values are the same."""
    if lhs.device != rhs.device:
        raise TTBError(f"Expected tensors to be on the same device. Given {lhs.device} and {rhs.device}")
    lhs, rhs = _promote(lhs, rhs)
    ld, rd = lhs.dim(), rhs.dim()
    if ld == 1 and rd == 1:
        if lhs.shape[0] != rhs.shape[0]:
            raise TTBError(f"Invalid shapes for dot product. Both LHS and RHS must have same dimensions: "
                           f"LHS={_shape_str(lhs)} and RHS={_shape_str(rhs)}")
        return batched_matmul(lhs.view(1, 1, -1) if lhs.is_contiguous() else lhs.unsqueeze(0).unsqueeze(0),
                              rhs.unsqueeze(0).unsqueeze(2)).flatten()
    if ld == 1 and rd == 2:
        if lhs.shape[0] != rhs.shape[0]:
            raise TTBError(f"Invalid shape for matrix multiplication. Length of LHS should equal size of RHS "
                           f"dimension 0: LHS={_shape_str(lhs)} and RHS={_shape_str(rhs)}")
        return batched_matmul(lhs.unsqueeze(0).unsqueeze(0), rhs.unsqueeze(0)).flatten()
    if ld == 2 and rd == 1:
        if lhs.shape[1] != rhs.shape[0]:
            raise TTBError(f"Invalid shape for matrix multiplication. Length of RHS should equal size of LHS "
                           f"dimension 1: LHS={_shape_str(lhs)} and RHS={_shape_str(rhs)}")
        return batched_matmul(lhs.unsqueeze(0), rhs.unsqueeze(0).unsqueeze(2)).flatten()
    if ld == 2 and rd == 2:
        if lhs.shape[1] != rhs.shape[0]:
            raise TTBError(f"Invalid shape for matrix multiplication. Size of LHS dimension 1 should equal size "
                           f"of RHS dimension 0: LHS={_shape_str(lhs)} and RHS={_shape_str(rhs)}")
        return batched_matmul(lhs.unsqueeze(0), rhs.unsqueeze(0)).squeeze(0)
    if ld == 3 and rd == 3:
        if lhs.shape[2] != rhs.shape[1]:
            raise TTBError(f"Invalid shape for batched matrix multiplication. Size of LHS dimension 2 should "
                           f"equal size of RHS dimension 1: LHS={_shape_str(lhs)} and RHS={_shape_str(rhs)}")
        return batched_matmul(lhs, rhs)
    raise TTBError("Unsupported sizes. Try reshaping or broadcasting. Expected dimensions of: "
                   "\n\t(LHS=1, RHS=1) for dot product,"
                   "\n\t(LHS=1, RHS=2) for vector-matrix product,"
                   "\n\t(LHS=2, RHS=1) for matrix-vector product,"
                   "\n\t(LHS=2, RHS=2) for matrix-matrix multiplication, or"
                   "\n\t(LHS=3, RHS=3) for batched matrix multiplication.")


def matmul_backward(lhs: torch.Tensor, rhs: torch.Tensor, grad_output: torch.Tensor):
    """Gradients of ``matmul(lhs, rhs)`` as tinytensor's autograd computes them: the rank
    plumbing of tensor.cpp:2403-2472 undone around TensorBatchedMatmul::backward
    (autograd/binary_ops.cpp:172-179), i.e. two more products on PERMUTED VIEWS,
    ``grad . rhs^T`` and ``lhs^T . grad``, which go to the kernels uncopied.
    -> (grad_lhs, grad_rhs), shaped like the operands."""
    ld, rd = lhs.dim(), rhs.dim()
    if (ld, rd) == (1, 1):
        l3, r3, g3 = lhs.reshape(1, 1, -1), rhs.reshape(1, -1, 1), grad_output.reshape(1, 1, 1)
    elif (ld, rd) == (1, 2):
        l3, r3, g3 = lhs.reshape(1, 1, -1), rhs.unsqueeze(0), grad_output.reshape(1, 1, -1)
    elif (ld, rd) == (2, 1):
        l3, r3, g3 = lhs.unsqueeze(0), rhs.reshape(1, -1, 1), grad_output.reshape(1, -1, 1)
    elif (ld, rd) == (2, 2):
        l3, r3, g3 = lhs.unsqueeze(0), rhs.unsqueeze(0), grad_output.unsqueeze(0)
    elif (ld, rd) == (3, 3):
        l3, r3, g3 = lhs, rhs, grad_output
    else:
        raise TTBError("Unsupported sizes. Try reshaping or broadcasting.")
    if tuple(g3.shape) != (l3.shape[0], l3.shape[1], r3.shape[2]):
        raise TTBError(f"grad_output has shape {tuple(grad_output.shape)}, which is not the shape of matmul(lhs, rhs)")
    grad_l = batched_matmul(g3, r3.permute(0, 2, 1))
    grad_r = batched_matmul(l3.permute(0, 2, 1), g3)
    return grad_l.reshape(lhs.shape), grad_r.reshape(rhs.shape)


def _np_view(a: np.ndarray) -> _View:
    if a.ndim != 3:
        raise TTBError(f"expected a rank-3 array, got rank {a.ndim}")
    es = a.dtype.itemsize
    if any(s % es or s < 0 for s in a.strides):
        raise TTBError("array strides must be non-negative multiples of the element size")
    return _make_view(a.ctypes.data, 0, a.shape, [s // es for s in a.strides])


def batched_matmul_host(lhs: np.ndarray, rhs: np.ndarray, out: np.ndarray | None = None, device: int = 0) -> np.ndarray:
    """Host-buffer form (ttb_batched_matmul_host): operands and result live in host memory;
    the library copies in, multiplies on `device`, copies out and synchronises."""
    if lhs.dtype != rhs.dtype:
        raise TTBError("operands must share a dtype")
    if lhs.dtype not in _NP_DTYPE_CODE:
        raise TTBError(f"unsupported dtype {lhs.dtype}")
    lv, rv = _np_view(lhs), _np_view(rhs)
    shape = (lhs.shape[0], lhs.shape[1], rhs.shape[2])
    if out is None:
        out = np.empty(shape, dtype=lhs.dtype)
    elif out.shape != shape or out.dtype != lhs.dtype or not out.flags.c_contiguous:
        raise TTBError("out must be a C-contiguous array of the result shape and dtype")
    rc = lib().ttb_batched_matmul_host(ctypes.byref(lv), ctypes.byref(rv), ctypes.c_void_p(out.ctypes.data),
                                       _NP_DTYPE_CODE[lhs.dtype], int(device))
    if rc != 0:
        _raise(rc)
    return out
