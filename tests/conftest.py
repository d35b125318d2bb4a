import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def built_library():
    """The in-tree shared library; built on demand (nvcc cross-compiles without a GPU)."""
    from vte_b200 import build
    build.build_library()
    return build.LIB


@pytest.fixture(scope="session")
def cuda_runtime(built_library):
    """A live runtime on device 0.  GPU tests fail loudly (no skip, no fallback)
    when the device or the library is missing."""
    from vte_b200 import build
    from vte_b200.bridge import CudaRuntime
    build.build_cubins()
    rt = CudaRuntime(device_index=int(os.environ.get("VTE_DEVICE_INDEX", "0")))
    rt.initialize()
    yield rt
    rt.cleanup()


@pytest.fixture(scope="session")
def codegen():
    from vte_b200.compiler import CodegenEngine
    return CodegenEngine()
