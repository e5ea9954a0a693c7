import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

GOLDEN = ROOT / "tests" / "golden" / "qpath_golden.npz"
# where the reference project is checked out (only the tests that build or import it need it)
REFERENCE_ROOT = Path(os.environ.get("DISC_REFERENCE_ROOT", "/root/reference"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(GOLDEN)


@pytest.fixture(scope="session")
def built_lib():
    """Path of libdisc_b200_ral.so, built on demand (nvcc cross-compiles without a GPU)."""
    from bladedisc_b200 import build
    return build.build()


@pytest.fixture(scope="session")
def ref_ral():
    """The reference's own RAL core + recording shim, when it could be built here."""
    import ctypes
    import subprocess
    so = ROOT / "oracle" / "_ref" / "libref_ral.so"
    if not so.exists() and (REFERENCE_ROOT / "tao_compiler/mlir/ral/ral_api.cc").exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "ref"], check=False,
                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    if not so.exists():
        pytest.skip("reference RAL library not built (reference tree absent)")
    lib = ctypes.CDLL(str(so))
    lib.ref_name.restype = ctypes.c_char_p
    lib.ref_recorded.restype = ctypes.c_int64
    lib.ref_dispatch.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p)]
    return lib


@pytest.fixture(scope="session")
def ref_host():
    """The reference's own host runtime (contexts, constants, host buffers, input / output binding),
    when it could be built here."""
    import ctypes
    import subprocess
    so = ROOT / "oracle" / "_ref" / "libref_host.so"
    if not so.exists() and (REFERENCE_ROOT / "tao_compiler/mlir/ral/ral_api.cc").exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "ref"], check=False,
                       stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    if not so.exists():
        pytest.skip("reference host runtime not built (reference tree absent)")
    return ctypes.CDLL(str(so))
