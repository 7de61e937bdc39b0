"""The reference's OWN doctest executables, run on a tinytensor build whose CUDA matmul path is
this library: oracle/dropin.mk compiles the reference tree with its CUDA backend for sm_100a,
with backend/cuda/matmul.cu replaced by csrc/tt_runner_shim.cu, conv.cu's two conv2d runners by
csrc/tt_conv_shim.cu, DeviceMemory<T>'s cudaMalloc / cudaFree sent to the library's memory pool
(csrc/tt_alloc_shim.h) and Tensor::to(Device) between GPUs made one peer copy
(csrc/tt_to_device_shim.cpp), links libttb.so, and builds the tests unchanged.  Each executable
runs every case on kCPU and, through tests/test_util.h:5-11, again on kCUDA -- i.e. on this
backend:

  test_matmul           tests/test_matmul.cpp:50-237   6 dtypes x 5 rank forms, wrapping ints
  test_matmul_autograd  tests/test_matmul_autograd.cpp:43-261 (vs libtorch)  transposed-view products
  test_conv, test_conv_autograd   conv2d forward / backward on the matmul path (vs libtorch)
  test_rnn, test_lstm, test_gru   matmul's callers with offset views
  test_to, test_to_autograd, test_clone, test_multi_device_cuda   storage, copies, device moves

The executables are built where the reference tree is and travel with the repository snapshot
(git-ignored); without them the tests are skipped with that reason."""
import os
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
BIN = ROOT / "oracle" / "_ref" / "tt_dropin" / "bin"
TESTS = ["test_matmul", "test_matmul_autograd", "test_conv", "test_conv_autograd", "test_rnn", "test_lstm",
         "test_gru", "test_to", "test_to_autograd", "test_clone", "test_multi_device_cuda"]


def _need(name: str) -> Path:
    exe = BIN / name
    if not exe.exists():
        pytest.skip(f"{exe.relative_to(ROOT)} has not been built (make -f oracle/dropin.mk REF=<tinytensor tree> dropin)")
    return exe


def _loaded_objects(exe: Path) -> str:
    env = dict(os.environ, LD_TRACE_LOADED_OBJECTS="1")
    return subprocess.run([str(exe)], env=env, capture_output=True, text=True, timeout=60).stdout


def test_the_executables_load_this_library(ttb):
    """The dynamic loader resolves libttb.so to the in-tree build for the test executable and
    for the tinytensor library it links."""
    exe = _need("test_matmul")
    objs = _loaded_objects(exe)
    lines = [l for l in objs.splitlines() if "libttb.so" in l]
    assert lines, objs
    resolved = Path(lines[0].split("=>")[-1].split("(")[0].strip()).resolve()
    assert resolved == ttb.lib_path().resolve()
    assert "libtinytensor_dropin.so" in objs


@pytest.mark.parametrize("name", TESTS)
def test_reference_test_passes_on_this_backend(name):
    exe = _need(name)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=900)
    tail = (r.stdout + r.stderr)[-3000:]
    assert r.returncode == 0, f"{name} exited {r.returncode}:\n{tail}"
    # doctest's summary line: every assertion passed, and the run was not empty
    assert "Status: SUCCESS" in r.stdout, tail
    summary = [l for l in r.stdout.splitlines() if "assertions:" in l]
    assert summary, tail
    if name != "test_multi_device_cuda":   # needs two GPUs to assert anything
        assert " 0 passed" not in summary[0], tail
