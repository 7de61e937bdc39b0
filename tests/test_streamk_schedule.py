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


# ---------------------------------------------------------------- paired stream-K
def paired_segments(unit, units, total_tiles, sk_tile0, nkb):
    """Odd units walk the cut part of their list backwards (the kernel's prologue, sk_pair)."""
    segs = segments(unit, units, total_tiles, sk_tile0, nkb)
    if unit & 1:
        first = next((i for i, s in enumerate(segs) if s[0] >= sk_tile0), len(segs))
        segs = segs[:first] + segs[first:][::-1]
    return segs


def pair_slot(unit, seg, nkb):
    """Slot a cut segment's sums go to: two per unit, 0 for a tail, 1 for a head."""
    _, k0, k1 = seg
    assert (k0 != 0) != (k1 != nkb)                    # a cut segment is a tail or a head, never a middle
    return unit * 2 + (0 if k0 != 0 else 1)


def other_slot(unit, seg):
    """Where the second of the two contributors looks for the first one's sums."""
    _, k0, _ = seg
    return (unit - 1) * 2 + 1 if k0 != 0 else (unit + 1) * 2 + 0


@pytest.mark.parametrize("units,total_tiles,nkb", [
    (74, 128, 256),    # the 8-GPU column block of 8192^3 on CTA pairs: every tile cut
    (74, 100, 256), (74, 80, 64), (148, 300, 40), (3, 7, 5), (2, 3, 9),
])
def test_paired_schedule(units, total_tiles, nkb):
    """With every unit's range at least one tile long (the launcher's condition for the pairing):
    every K block once, every cut tile has exactly two contributors, each writes to a slot of its
    own and finds the other's, and the tiles that complete at the very end are shared by an even
    unit and the odd one after it -- one completion for two units."""
    all_kb = total_tiles * nkb
    assert all_kb // units >= nkb + 1
    done, contributors, slots = {}, {}, {}
    last_tile_of = {}
    for u in range(units):
        segs = paired_segments(u, units, total_tiles, 0, nkb)
        assert len(segs) <= K_MAX_SEGMENTS
        last_tile_of[u] = segs[-1][0]
        for seg in segs:
            t, k0, k1 = seg
            for kb in range(k0, k1):
                assert (t, kb) not in done
                done[(t, kb)] = u
            if k0 != 0 or k1 != nkb:
                s = pair_slot(u, seg, nkb)
                assert s not in slots                  # a slot is written once per launch
                slots[s] = (t, u)
                contributors.setdefault(t, []).append((u, seg))
    assert len(done) == all_kb
    for t, cs in contributors.items():
        assert len(cs) == 2                            # the ticket counts to two
        (ua, sa), (ub, sb) = cs
        assert slots[other_slot(ua, sa)] == (t, ub) and slots[other_slot(ub, sb)] == (t, ua)
    # completions at the end: an even unit ends on the head of the tile its odd neighbour ends on
    # (unless their ranges happen to meet exactly on a tile boundary: then there is no shared tile)
    aligned = 0
    for u in range(0, units - 1, 2):
        if (all_kb * (u + 1) // units) % nkb == 0:
            aligned += 1
        else:
            assert last_tile_of[u] == last_tile_of[u + 1]
    assert len(set(last_tile_of.values())) <= (units + 1) // 2 + aligned


# ---------------------------------------------------------------- piece schedule
def piece_segments(unit, units, total_tiles, pieces_log2, piece_len, nkb):
    out = []
    g = unit
    while g < (total_tiles << pieces_log2):
        k0 = (g & ((1 << pieces_log2) - 1)) * piece_len
        out.append((g >> pieces_log2, k0, min(k0 + piece_len, nkb)))
        g += units
    return out


def piece_plan(want, nkb, kc, total_tiles, units):
    """The launcher's choice: the largest power of two of equal, non-empty parts (whole
    accumulation chunks each) not above `want` whose per-unit list fits the segment table."""
    lg = 0
    while (2 << lg) <= want:
        lg += 1
    while lg > 0:
        length = -(-nkb // (1 << lg))
        length = -(-length // kc) * kc
        parts = -(-nkb // length)
        if parts == (1 << lg) and -(-(total_tiles * parts) // units) <= K_MAX_SEGMENTS:
            return lg, length
        lg -= 1
    return 0, 0


@pytest.mark.parametrize("units,total_tiles,nkb,want", [
    (74, 128, 256, 4), (74, 256, 256, 4), (74, 512, 256, 4), (74, 128, 256, 8), (148, 20, 47, 4), (74, 9, 63, 2),
])
def test_piece_schedule(units, total_tiles, nkb, want):
    """Every K block once; every tile has exactly `pieces` parts; the slot a part is written to
    (two per unit, by the parity of the part's position in the unit's list) is not reused before
    the tile it belongs to can have been completed, i.e. not by the unit's next part."""
    lg, length = piece_plan(want, nkb, 8, total_tiles, units)
    if lg == 0:
        pytest.skip("no equal power-of-two split of this K range")
    pieces = 1 << lg
    done, parts = {}, {}
    for u in range(min(units, total_tiles * pieces)):
        segs = piece_segments(u, units, total_tiles, lg, length, nkb)
        assert len(segs) <= K_MAX_SEGMENTS
        for i, (t, k0, k1) in enumerate(segs):
            assert 0 <= k0 < k1 <= nkb
            for kb in range(k0, k1):
                assert (t, kb) not in done
                done[(t, kb)] = u
            parts.setdefault(t, []).append((u, i))
            # the reader of part g = t * pieces + j finds it at unit g % units, list position g // units
            g = t * pieces + k0 // length
            assert (g % units, g // units) == (u, i)
    assert len(done) == total_tiles * nkb
    assert all(len(p) == pieces for p in parts.values())
