import os
import sys
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]
for p in (REPO, REPO / "ai-compiler-framework_b200" / "python"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def _gpu_count() -> int:
    try:
        import aicf_cuda
        return int(aicf_cuda.lib.aicf_b200_device_count())
    except Exception:
        return 0


@pytest.fixture(scope="session")
def gpu():
    """Skips when no device is visible; the CUDA library itself must always load."""
    import aicf_cuda  # noqa: F401  (raises if the library was not built: no fallback)
    if _gpu_count() < 1:
        pytest.skip("no CUDA device visible")
    return True


@pytest.fixture(scope="session")
def ref_lib(gpu):
    """The reference's own CUDA backend, built by oracle/ref_build.py (None if it was never built)."""
    import ctypes
    path = REPO / "oracle" / "_ref" / "libaicf_ref.so"
    if not path.exists():
        pytest.skip("oracle/_ref/libaicf_ref.so not built")
    lib = ctypes.CDLL(str(path))
    lib.ref_op_call.restype = ctypes.c_int
    lib.ref_op_call.argtypes = [ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                ctypes.c_void_p, ctypes.c_uint64]
    lib.ref_launch_by_id.restype = ctypes.c_int
    lib.ref_launch_by_id.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                     ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64]
    assert lib.ref_tensor_desc_size() == 96
    return lib
