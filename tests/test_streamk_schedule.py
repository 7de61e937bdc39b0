"""Host-side restatement of the stream-K schedule of the f32 tensor-core kernel
(tinytensor_b200/csrc/gemm_f32_tcgen05.cu: the segment table built in the kernel's prologue, the
owner's fix-up loop, and the launcher's choice of how many waves of tiles stay whole).  The
protocol has one partial-sum slot and one flag per unit, so these must hold for every shape:
every K block of every tile is computed exactly once, every tile has exactly one owner (the unit
whose range starts at its K block 0), a unit hands over at most one partial tile, and the units
an owner waits for are exactly those that computed the rest of its tile.  The launcher only cuts
when every unit gets at least four K blocks of the cut (a unit with an empty range would never
raise its flag), so the checks run on the shapes it lets through."""
import random

import pytest

K_MAX_SEGMENTS = 32


def segments(unit, units, total_tiles, sk_tile0, nkb):
    """The (tile, kb0, kb1) list of one unit: whole tiles first, then its share of the cut tiles."""
    segs = [(t, 0, nkb) for t in range(unit, sk_tile0, units)]
    all_kb = (total_tiles - sk_tile0) * nkb
    pos, end = all_kb * unit // units, all_kb * (unit + 1) // units
    while pos < end:
        rel, k0 = divmod(pos, nkb)
        stop = min(pos + (nkb - k0), end)
        segs.append((sk_tile0 + rel, k0, k0 + (stop - pos)))
        pos = stop
    return segs


def waited_for(owner, units, total_tiles, sk_tile0, nkb, tile):
    """Units the owner of `tile` reads partial sums from (the kernel's loop over q > unit)."""
    all_kb = (total_tiles - sk_tile0) * nkb
    out = []
    for q in range(owner + 1, units):
        if all_kb * q // units >= (tile - sk_tile0 + 1) * nkb:
            break
        out.append(q)
    return out


def check(units, total_tiles, sk_tile0, nkb):
    done = {}
    owner, helpers = {}, {}
    for u in range(units):
        segs = segments(u, units, total_tiles, sk_tile0, nkb)
        partial = [s for s in segs if s[1] != 0]
        assert len(partial) <= 1                       # one slot per unit is enough
        if partial:
            assert partial[0] == [s for s in segs if s[0] >= sk_tile0][0]  # and it is its first cut segment
        for t, k0, k1 in segs:
            assert 0 <= k0 < k1 <= nkb
            for kb in range(k0, k1):
                assert (t, kb) not in done
                done[(t, kb)] = u
            if k0 == 0:
                assert t not in owner
                owner[t] = u
            else:
                helpers.setdefault(t, []).append(u)
    assert len(done) == total_tiles * nkb              # nothing missing
    assert sorted(owner) == list(range(total_tiles))
    for t in range(sk_tile0, total_tiles):
        assert waited_for(owner[t], units, total_tiles, sk_tile0, nkb, t) == sorted(helpers.get(t, []))


def launcher_choice(units, total_tiles, nkb, exchange=False):
    """waves_full / sk_tile0 and whether the cut is possible, as launch_cg decides them."""
    waves_full, rem = divmod(total_tiles, units)
    if exchange and waves_full < 3 and total_tiles * nkb // units >= 16:
        waves_full = 0
    cut_tiles = rem if waves_full > 0 else total_tiles
    cut_kb_per_unit = cut_tiles * nkb // units
    possible = (cut_tiles > 0 and cut_kb_per_unit >= 4 and waves_full + 3 <= K_MAX_SEGMENTS
                and total_tiles // units + 3 <= K_MAX_SEGMENTS)
    return waves_full * units, possible


@pytest.mark.parametrize("units,total_tiles,nkb", [
    (148, 160, 98),    # conv2d grad_w: one whole wave + 12 tiles cut
    (74, 80, 128),     # 2560 x 2048 x 4096 on CTA pairs
    (74, 1024, 256),   # 8192^3: 13 whole waves + 62 tiles cut
    (64, 16, 16),      # 512^3: fewer tiles than units, every tile cut
    (148, 1, 600),     # one tile over all SMs
    (148, 149, 7),     # a single extra tile of a short K
    (3, 7, 5), (5, 5, 1), (7, 3, 2),
])
def test_named_shapes(units, total_tiles, nkb):
    for exchange in (False, True):
        sk_tile0, possible = launcher_choice(units, total_tiles, nkb, exchange)
        if possible:
            check(units, total_tiles, sk_tile0, nkb)
    if total_tiles * nkb // units >= 4:
        check(units, total_tiles, 0, nkb)               # pure stream-K of the same shape


def test_random_shapes():
    rng = random.Random(7)
    checked = 0
    for _ in range(600):
        units = rng.choice([1, 2, 3, 7, 16, 64, 74, 148])
        total_tiles = rng.randint(1, 6 * units + 5)
        nkb = rng.randint(1, 300)
        sk_tile0, possible = launcher_choice(units, total_tiles, nkb, rng.random() < 0.3)
        if possible:  # what the launcher lets through is consistent and fits the kernel's segment table
            checked += 1
            check(units, total_tiles, sk_tile0, nkb)
            assert max(len(segments(u, units, total_tiles, sk_tile0, nkb)) for u in range(units)) <= K_MAX_SEGMENTS
    assert checked > 100


def test_a_cut_thinner_than_the_launcher_allows_would_leave_units_without_work():
    """Why the four-K-block floor exists: 149 tiles of 7 K blocks on 148 units, one tile cut."""
    sk_tile0, possible = launcher_choice(148, 149, 7)
    assert sk_tile0 == 148 and not possible
    assert sum(1 for u in range(148) if len(segments(u, 148, 149, sk_tile0, 7)) == 1) > 100  # whole tile only
