import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_dir():
    return GOLDEN


@pytest.fixture(scope="session")
def selftest_lib():
    """The test-suite's own kernels (tests/csrc/selftest_kernels.cu), built into tests/libesp_selftest.so when missing
    or stale.  They are not part of the product library."""
    import ctypes as C
    from loongserve_b200 import build
    lib = C.CDLL(build.build_selftest(force=False))
    vp, i32, i64 = C.c_void_p, C.c_int32, C.c_int64
    lib.esp_selftest_umma.argtypes = [vp, vp, vp, i32, i32, vp]
    lib.esp_selftest_umma.restype = i32
    lib.esp_selftest_bounded_wait.argtypes = [i64, vp, vp]
    lib.esp_selftest_bounded_wait.restype = i32
    return lib
