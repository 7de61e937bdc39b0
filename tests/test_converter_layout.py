"""Host-side restatement of the index math of the f32 kernel's converter warps
(tinytensor_b200/csrc/gemm_f32_tcgen05.cu, hybrid split): where a 16-byte chunk of a raw fp32
operand tile (128 x 32 fp32, as TMA delivers it) goes in the 64-byte-swizzled bf16 tiles the
correction MMAs read.  The kernel computes the offset of a thread's first chunk once and adds
u * NCT * 8 bytes for its u-th chunk; these tests pin the facts that shortcut relies on."""
import pytest


def dst_offset(ci: int, mn_major: bool) -> int:
    """Byte offset in the bf16 tile of raw chunk `ci` (16 bytes = 4 fp32 -> 8 bytes = 4 bf16)."""
    if not mn_major:
        # K-major raw tile: row = 128 B = 8 chunks, chunk position XORed with (row & 7);
        # bf16 row = 64 B = 4 chunks of 16 B XORed with ((row >> 1) & 3)
        r, cp = ci >> 3, ci & 7
        return r * 64 + (cp >> 1) * 16 + (((cp ^ r) & 1) << 3)
    # MN-major raw tile: four boxes of 32 (MN) x 32 (K); a row is one K index, 32-byte chunks XORed
    # with (k & 3); bf16 row = 64 B, 16-byte chunks XORed with ((k >> 1) & 3)
    box, kr, c16 = ci >> 8, (ci & 255) >> 3, ci & 7
    lc = (c16 >> 1) ^ (kr & 3)
    return box * 2048 + kr * 64 + ((lc ^ ((kr >> 1) & 3)) << 4) + ((c16 & 1) << 3)


@pytest.mark.parametrize("mn_major", [False, True])
def test_chunks_fill_the_bf16_tile_exactly_once(mn_major):
    offsets = sorted(dst_offset(ci, mn_major) for ci in range(1024))
    assert offsets == list(range(0, 8192, 8))  # 1024 chunks x 8 bytes = one 8 KiB bf16 tile


@pytest.mark.parametrize("mn_major", [False, True])
@pytest.mark.parametrize("converter_threads", [128, 256])  # CTA-pair form, one-CTA form
def test_offset_of_later_chunks_is_the_first_plus_a_constant(mn_major, converter_threads):
    per_thread = 1024 // converter_threads
    for tid in range(converter_threads):
        first = dst_offset(tid, mn_major)
        for u in range(per_thread):
            assert dst_offset(tid + u * converter_threads, mn_major) == first + u * converter_threads * 8


def test_k_major_chunk_keeps_its_row_and_k_range():
    """K-major: chunk (row r, stored position cp) holds k = 4 * (cp ^ (r & 7)) .. + 3 of row r;
    its bf16 copy must sit in row r of the bf16 tile at k * 2 bytes, in the bf16 tile's swizzle."""
    for r in range(128):
        for cp in range(8):
            k0 = 4 * (cp ^ (r & 7))                      # logical first k of the stored chunk
            logical = r * 64 + k0 * 2                     # unswizzled bf16 byte offset
            chunk16, within = logical // 16 % 4, logical % 16
            swizzled = r * 64 + ((chunk16 ^ ((r >> 1) & 3)) * 16) + within
            assert dst_offset(r * 8 + cp, False) == swizzled


@pytest.mark.parametrize("mn_major", [False, True])
def test_split_of_the_rhs_tile_between_warpgroup_and_spare_warps(mn_major):
    """Pair form: the converter warpgroup (128 threads) takes chunks [0, 384) of the B tile, thread
    t its chunks t + 128 u (u < 3); the two spare warps (64 threads) take [384, 1024), thread e its
    chunks 384 + e + 64 u (u < 10), 512 bytes apart in the bf16 tile.  Together: every chunk once,
    every destination once, and the spare warps' constant step holds across box boundaries."""
    seen, dsts = [], []
    for t in range(128):
        for u in range(3):
            ci = t + 128 * u
            seen.append(ci)
            dsts.append(dst_offset(t, mn_major) + u * 128 * 8)
            assert dsts[-1] == dst_offset(ci, mn_major)
    for e in range(64):
        first = dst_offset(384 + e, mn_major)
        for u in range(10):
            ci = 384 + e + 64 * u
            seen.append(ci)
            dsts.append(first + u * 512)
            assert dsts[-1] == dst_offset(ci, mn_major)
    assert sorted(seen) == list(range(1024))
    assert sorted(dsts) == list(range(0, 8192, 8))
