"""B200-native matmul backend for tinytensor: host-side mirror of the reference interface.

The product is ``libttb.so`` (hand-written sm_100a CUDA behind a C ABI, see
``include/ttb.h``).  This package is the thin host layer used by the tests and the
benchmark: it loads the library with ctypes and mirrors the names, argument
meaning and error behaviour of the reference's matmul path
(``tinytensor::matmul`` -> ``BackendBase::batched_matmul``).  torch is used only
for device memory, streams and ``torch.distributed``.

There is no CPU or eager fallback: importing works without the library, but any
compute call raises if ``libttb.so`` is missing.
"""
from .backend import (  # noqa: F401
    Activation,
    PreparedMatmul,
    TTBError,
    Variant,
    batched_matmul,
    batched_matmul_fused,
    conv2d,
    conv2d_backward,
    linear,
    batched_matmul_host,
    batched_matmul_static_scratch,
    check_device,
    device_alloc,
    device_free,
    device_memory_stats,
    device_trim,
    to_device,
    get_option,
    last_variant,
    launch_count,
    lib,
    lib_path,
    matmul,
    matmul_backward,
    matmul_allgather,
    matmul_allgather_multicast,
    measure_fp64_tensor_peak,
    tensor_map_cache_stats,
    set_option,
    tma_eligible,
    view_of,
)
from .inputs import CONFIG_SEEDS, Generator, config_operands  # noqa: F401
from .partition import Partition, ShardedMatmul, partition  # noqa: F401

__all__ = [
    "Activation", "TTBError", "Variant", "batched_matmul", "batched_matmul_fused", "conv2d", "conv2d_backward", "linear", "batched_matmul_host", "batched_matmul_static_scratch",
    "check_device", "device_alloc", "device_free", "device_memory_stats", "device_trim", "to_device", "get_option",
    "last_variant", "launch_count", "lib", "lib_path", "matmul", "matmul_allgather", "matmul_allgather_multicast", "matmul_backward", "set_option", "tma_eligible",
    "view_of", "Partition", "ShardedMatmul", "partition", "Generator", "config_operands", "CONFIG_SEEDS", "measure_fp64_tensor_peak", "PreparedMatmul", "tensor_map_cache_stats",
]
