"""The seeded input generator (ttb_generator_*, tinytensor_b200/inputs.py) against the
reference's own Generator: the committed golden vectors the reference library produced
(tests/golden/reference_api_golden.npz, script beside it), and, when it has been built,
the reference library itself (oracle/_ref/libttref_full.so), bit for bit."""
import math
import sys
from pathlib import Path

import numpy as np
import pytest

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import ref_full  # noqa: E402
from make_reference_api_golden import CONFIG_SEEDS, config_draws, digest  # noqa: E402

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_api_golden.npz")


def bits(a):
    return np.ascontiguousarray(a).view(np.uint8)


@pytest.mark.parametrize("seed", range(5))
def test_raw_outputs_match_the_reference(ttb, seed):
    g = ttb.Generator(seed)
    got = np.array([g.next() for _ in range(16)], dtype=np.uint64)
    assert np.array_equal(got, GOLDEN[f"gen_raw_{seed}"])


@pytest.mark.parametrize("name", list(CONFIG_SEEDS))
def test_configuration_operands_match_the_reference(ttb, name):
    """Every operand of every benchmark configuration, full size: first 64 values and a digest of
    all bits equal what the reference's uniform_real / normal / uniform_int drew."""
    ops = ttb.config_operands(name)
    assert ttb.CONFIG_SEEDS[name] == CONFIG_SEEDS[name]
    keys = [k[len(f"cfg_{name}_"):-len("_head")] for k in GOLDEN.files if k.startswith(f"cfg_{name}_") and k.endswith("_head")]
    assert list(ops) == keys  # same tensors in the same draw order
    for key, arr in ops.items():
        want = GOLDEN[f"cfg_{name}_{key}_head"]
        assert arr.dtype == want.dtype
        assert np.array_equal(bits(arr.reshape(-1)[:64]), bits(want)), key
        assert digest(arr) == GOLDEN[f"cfg_{name}_{key}_digest"][0], key


def test_batch_range_is_a_slice_of_the_full_draw(ttb):
    full = ttb.config_operands("c3")
    part = ttb.config_operands("c3", batch_range=(96, 128))
    for k in full:
        assert np.array_equal(part[k], full[k][96:128])


def test_config_draws_helper_agrees_with_inputs_module(ttb):
    """The helper the golden script drives the reference with makes the same calls, in the same
    order, as tinytensor_b200.inputs.config_operands."""
    for name in ("c1", "c2"):
        got = dict(config_draws(name, ttb.Generator(CONFIG_SEEDS[name])))
        want = ttb.config_operands(name)
        assert list(got) == list(want)
        for k in want:
            assert np.array_equal(bits(got[k]), bits(want[k]))


def test_argument_errors(ttb):
    g = ttb.Generator(0)
    with pytest.raises(ttb.TTBError):
        g.uniform_real(1.0, 1.0, (4,))          # low < high required, as the reference asserts
    with pytest.raises(ttb.TTBError):
        g.uniform_int(0, 5, (4,), np.int16)     # the reference samples integers in i32 / i64 only
    with pytest.raises(ttb.TTBError):
        g.normal(0, 1, (4,), np.int32)


@pytest.mark.skipif(not ref_full.available(), reason="oracle/_ref/libttref_full.so not built")
@pytest.mark.parametrize("seed", [0, 3, 4, 987654321])
def test_against_the_reference_library(ttb, seed):
    """Interleaved draws of all three distributions and both float widths from one generator on
    each side: values and generator state stay identical throughout."""
    ours, ref = ttb.Generator(seed), ref_full.Gen(seed)
    n = 70001
    for lo, hi in ((-1.0, 1.0), (0.0, 1.0), (-1 / math.sqrt(784), 1 / math.sqrt(784)), (3.0, 1e6)):
        for dt in (np.float32, np.float64):
            assert np.array_equal(bits(ours.uniform_real(lo, hi, (n,), dt)), bits(ref.uniform_real(lo, hi, (n,), dt)))
    for mu, sd in ((0.0, 1.0), (0.0, 8192 ** -0.5), (-3.5, 0.25)):
        for dt in (np.float32, np.float64):
            assert np.array_equal(bits(ours.normal(mu, sd, (n,), dt)), bits(ref.normal(mu, sd, (n,), dt)))
    for lo, hi in ((-8, 9), (0, 2), (-2 ** 31, 2 ** 31 - 1), (5, 1000003)):
        assert np.array_equal(ours.uniform_int(lo, hi, (n,), np.int32), ref.uniform_int(lo, hi, (n,), np.int32))
    assert np.array_equal(ours.uniform_int(-2 ** 40, 2 ** 41, (n,), np.int64),
                          ref.uniform_int(-2 ** 40, 2 ** 41, (n,), np.int64))
    assert ours.next() == ref.next()
