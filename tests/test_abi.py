"""CPU-side checks of the C ABI: the library loads, exports every symbol the header
declares, and the host-only entry points behave.  No compute call is made here."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent


def declared_symbols():
    text = (ROOT / "include" / "ttb.h").read_text()
    return sorted(set(re.findall(r"TTB_API\s+[\w\s\*]+?\b(ttb_\w+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_symbols()
    assert "ttb_batched_matmul" in names and "ttb_batched_matmul_host" in names
    assert len(names) >= 12


def test_library_exports_every_declared_symbol(ttb):
    L = ttb.lib()
    for name in declared_symbols():
        assert hasattr(L, name), f"libttb.so does not export {name}"


def test_version_and_variant_names(ttb):
    L = ttb.lib()
    assert L.ttb_version() >= 100
    assert L.ttb_variant_name(1) == b"simt"
    assert L.ttb_variant_name(2) == b"tcgen05_3xtf32"
    assert L.ttb_variant_name(99) == b"unknown"


def test_options_round_trip_and_reject_bad_values(ttb, reset_options):
    ttb.set_option("force_variant", 1)
    assert ttb.get_option("force_variant") == 1
    with pytest.raises(ttb.TTBError):
        ttb.set_option("force_variant", 77)
    with pytest.raises(ttb.TTBError):
        ttb.set_option("tf32_terms", 4)
    with pytest.raises(ttb.TTBError):
        ttb.set_option("no_such_option", 1)


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_partition_batch_ranges_cover_exactly(ttb, world):
    for B in (2, 7, 64, 256):
        covered = []
        for r in range(world):
            p = ttb.partition(B, 128, 64, 128, world, r)
            assert p.kind == "batch"
            covered.extend(range(p.begin, p.end))
        assert covered == list(range(B))
        sizes = [ttb.partition(B, 128, 64, 128, world, r).size for r in range(world)]
        assert max(sizes) - min(sizes) <= 1


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_partition_column_blocks_cover_exactly(ttb, world):
    for M in (8192, 1000, 130, 64):
        covered = []
        for r in range(world):
            p = ttb.partition(1, 4096, 512, M, world, r)
            assert p.kind == "columns"
            assert p.begin % 128 == 0 or p.begin == M
            covered.extend(range(p.begin, p.end))
        assert covered == list(range(M))
    p = ttb.partition(1, 8192, 8192, 8192, 8, 3)
    assert (p.begin, p.end) == (3072, 4096)


def test_partition_rejects_bad_arguments(ttb):
    with pytest.raises(ttb.TTBError):
        ttb.partition(1, 8, 8, 8, 0, 0)
    with pytest.raises(ttb.TTBError):
        ttb.partition(1, 8, 8, 8, 2, 2)
    with pytest.raises(ttb.TTBError):
        ttb.partition(0, 8, 8, 8, 2, 0)


def test_tma_eligibility_table(ttb):
    """Host-only classification of views: which ones the tensor-core kernels can read
    through a tensor map built from their strides."""
    base = torch.zeros(4 * 64 * 96 + 8, dtype=torch.float32)
    t = base[:4 * 64 * 96].view(4, 64, 96)
    assert ttb.tma_eligible(t, 0)                       # contiguous
    assert ttb.tma_eligible(t.permute(0, 2, 1), 1)      # transposed view (backward's operand)
    assert ttb.tma_eligible(t[:, :, 32:64], 1)          # column block: strided, aligned
    assert ttb.tma_eligible(t[1:2], 0)                  # offset batch
    assert ttb.tma_eligible(t[:1].expand(4, 64, 96), 0)  # broadcast batch (stride 0)
    assert not ttb.tma_eligible(t[:, :, ::2], 0)        # step on the inner dim
    assert not ttb.tma_eligible(base[1:1 + 64 * 96].view(1, 64, 96), 0)  # 4-byte offset
    assert not ttb.tma_eligible(t[:, :, :10].contiguous(), 0)  # 40-byte rows
    assert not ttb.tma_eligible(t[:, :1, :].expand(4, 64, 96), 0)  # stride 0 on a matrix dim


def test_compute_call_without_gpu_fails_loudly(ttb):
    """No CPU fallback: on a box without CUDA the call reports an error."""
    if torch.cuda.is_available():
        pytest.skip("CUDA present")
    a = np.ones((1, 4, 4), dtype=np.float32)
    with pytest.raises(ttb.TTBError):
        ttb.batched_matmul_host(a, a)
    with pytest.raises(ttb.TTBError):
        ttb.batched_matmul(torch.ones(1, 4, 4), torch.ones(1, 4, 4))


def test_missing_library_fails_loudly(ttb, monkeypatch, tmp_path):
    from tinytensor_b200 import backend

    monkeypatch.setenv("TTB_LIBRARY", str(tmp_path / "nope.so"))
    monkeypatch.setattr(backend, "_lib", None)
    with pytest.raises(ttb.TTBError):
        backend.lib()


def test_conv2d_and_fused_argument_checks_need_no_gpu(ttb):
    """Shape, dtype and limit errors of the conv2d and fused entry points are found on the host,
    before any CUDA call: they come back as status codes with a message (the tinytensor-side
    adapter turns them into TTException)."""
    from tinytensor_b200.backend import _ConvDesc, _View

    L = ttb.lib()
    one = ctypes.c_void_p(64)  # never dereferenced: every call below fails validation first

    def conv(desc, dtype=5):
        return L.ttb_conv2d_forward(one, one, None, one, ctypes.byref(desc), dtype, 0, None)

    assert conv(_ConvDesc(1, 3, 8, 8, 4, 9, 1, 0)) == -2          # kernel larger than the image: TTB_ESHAPE
    assert b"does not fit" in L.ttb_last_error()
    assert conv(_ConvDesc(1, 3, 8, 8, 4, 3, 0, 0)) == -2          # stride 0
    assert conv(_ConvDesc(1, 3, 8, 8, 4, 3, 1, -1)) == -2         # negative padding
    assert conv(_ConvDesc(1, 3, 8, 8, 4, 3, 1, 0), dtype=0) == -3  # bool8: TTB_EDTYPE
    assert conv(_ConvDesc(1, 70000, 8, 8, 4, 3, 1, 0)) == -9       # more than 65535 channels: TTB_ELIMIT
    assert conv(_ConvDesc(4096, 64, 512, 512, 64, 3, 1, 1)) == -9  # beyond the reference's int indexing
    assert L.ttb_conv2d_forward(one, one, None, one, None, 5, 0, None) == -1  # null description
    assert L.ttb_conv2d_backward(one, one, one, one, None, None, ctypes.byref(_ConvDesc(1, 3, 8, 8, 4, 3, 1, 0)), 5,
                                 0, None) == -1                    # null grad_weight

    def view(shape, stride=None):
        stride = stride or (shape[1] * shape[2], shape[2], 1)
        return _View(ctypes.c_void_p(64), 0, (ctypes.c_int64 * 3)(*shape), (ctypes.c_int64 * 3)(*stride))

    a, b = view((2, 8, 4)), view((2, 4, 6))
    fused = lambda addend, act, dtype=5: L.ttb_batched_matmul_fused(
        ctypes.byref(a), ctypes.byref(b), one, 0, None, ctypes.byref(addend) if addend is not None else None, act, dtype,
        0, None)
    assert fused(view((2, 8, 7)), 0) == -2                        # addend shape
    assert b"addend" in L.ttb_last_error()
    assert fused(None, 5) == -1                                   # unknown activation
    assert fused(None, 1, dtype=3) == -3                          # relu on i32
    assert fused(view((2, 8, 6), (48, 6, -1)), 0) == -1           # negative stride in the addend


def test_allgather_peer_arguments_are_checked_on_the_host(ttb):
    """ttb_matmul_allgather validates its peer pointers before it touches a device: null peers,
    too many peers, and a peer buffer whose 16-byte alignment differs from this rank's C (the
    kernel chooses vector or scalar stores from its own C and uses them for every peer)."""
    from tinytensor_b200.backend import _View

    L = ttb.lib()

    def view(ptr, shape):
        return _View(ctypes.c_void_p(ptr), 0, (ctypes.c_int64 * 3)(*shape),
                     (ctypes.c_int64 * 3)(shape[1] * shape[2], shape[2], 1))

    a, b = view(1 << 20, (1, 256, 128)), view(2 << 20, (1, 128, 256))
    strides = (ctypes.c_int64 * 3)(256 * 256, 256, 1)
    out = 3 << 20

    def call(peers, n=None):
        arr = (ctypes.c_void_p * max(len(peers), 1))(*[ctypes.c_void_p(p) for p in peers])
        return L.ttb_matmul_allgather(ctypes.byref(a), ctypes.byref(b), ctypes.c_void_p(out), 0, strides, arr,
                                      len(peers) if n is None else n, 5, 0, None)

    assert call([(4 << 20) + 4]) == -1                 # 4-byte aligned peer, 16-byte aligned C: TTB_EINVAL
    assert b"not aligned like out" in L.ttb_last_error()
    assert call([0]) == -1                             # null peer
    assert call([4 << 20] * 16) == -9                  # more than 15 peers: TTB_ELIMIT
    assert call([4 << 20], n=-1) == -1                 # negative count
