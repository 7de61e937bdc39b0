"""The mirror of tinytensor::matmul's host logic (tinytensor_b200/backend.py::matmul: rank
plumbing, dtype promotion, refusals) against the reference's own compiled matmul
(tinytensor/tensor/tensor.cpp:2390-2484): the messages of its TTExceptions, taken from the golden
fixture the reference library produced.  Runs without a GPU: every refusal happens before a
kernel could be launched.  The values and gradients are compared on the GPU in
test_matmul_api_vs_reference_gpu.py."""
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parent / "golden"))
import ref_full  # noqa: E402
from make_reference_api_golden import ERRORS  # noqa: E402

GOLDEN = np.load(Path(__file__).resolve().parent / "golden" / "reference_api_golden.npz")


def _operand(dt, shape):
    return torch.zeros(shape, dtype=torch.bool if dt == np.bool_ else torch.float32)


@pytest.mark.parametrize("case", ERRORS, ids=[e[0] for e in ERRORS])
def test_refusals_carry_the_references_message(ttb, case):
    name, dl, ls, dr, rs = case
    with pytest.raises(ttb.TTBError) as info:
        ttb.matmul(_operand(dl, ls), _operand(dr, rs))
    assert str(info.value) == str(GOLDEN[f"err_{name}"])


@pytest.mark.skipif(not ref_full.available(), reason="oracle/_ref/libttref_full.so not built")
@pytest.mark.parametrize("case", ERRORS, ids=[e[0] for e in ERRORS])
def test_refusals_against_the_reference_library(ttb, case):
    name, dl, ls, dr, rs = case
    with pytest.raises(ref_full.ReferenceError_) as ref_info:
        ref_full.matmul(np.zeros(ls, dl), np.zeros(rs, dr))
    with pytest.raises(ttb.TTBError) as info:
        ttb.matmul(_operand(dl, ls), _operand(dr, rs))
    assert str(ref_info.value).split("TinyTensor Error: ", 1)[-1].strip() == str(info.value)


def test_cross_device_operands_are_refused(ttb):
    """CHECK_SAME_DEVICE (tensor.cpp:180-185, :2393) comes first in the reference too."""
    if not torch.cuda.is_available():
        a, b = torch.zeros(2, 2), torch.zeros(2, 2, device="meta")
    else:
        a, b = torch.zeros(2, 2), torch.zeros(2, 2, device="cuda")
    with pytest.raises(ttb.TTBError):
        ttb.matmul(a, b)
