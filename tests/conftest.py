import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 GPU (run with -m gpu)")
    # The C-ABI library is built in-tree; compile it when it is not there yet
    # (nvcc cross-compiles for sm_100a without a GPU).  A missing nvcc is not
    # hidden: the tests that load the library then fail loudly.
    from oxmera_b200 import capi
    if not os.path.exists(capi.library_path()):
        try:
            from oxmera_b200.build import build_library
            build_library()
        except Exception as e:  # reported by the tests that need the library
            sys.stderr.write(f"could not build {capi.LIB_NAME}: {e}\n")


@pytest.fixture(scope="session")
def oracle():
    """The CPU oracle (built on demand with gcc)."""
    from tests.oracle_lib import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def backend():
    """The B200 backend on cuda:0, registered for dispatch.  Fails loudly when
    the CUDA library is missing or no B200 is visible: there is no fallback."""
    import oxmera_b200 as ox
    b = ox.B200Backend(0)
    ox.register_backend(b)
    yield b
    b.synchronize()
