import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def ttb():
    """The package, with libttb.so built if it is missing (nvcc cross-compiles without a GPU)."""
    import tinytensor_b200 as pkg
    from tinytensor_b200 import build

    if not pkg.lib_path().exists():
        build.build()
    pkg.lib()
    return pkg


@pytest.fixture(scope="session")
def oracle():
    import oracle_lib

    return oracle_lib.load()


@pytest.fixture()
def reset_options(ttb):
    """Restores the library's dispatch options after a test that forces a variant."""
    yield
    for key, value in (("force_variant", 0), ("tf32_terms", 2), ("k_chunk", 0), ("splitk", 1), ("two_cta", -1),
                       ("mask_big", 0), ("tc_debug", 0), ("tc_profile", 0), ("streamk", -1),
                       ("conv_columns_mb", 2048), ("int_tensor", 1), ("peer_tma", 1), ("a_tmem", 0), ("extra_conv", 1), ("pieces", -1), ("sk_pair", -1)):
        ttb.set_option(key, value)
