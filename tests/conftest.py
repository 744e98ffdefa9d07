import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def built_lib():
    """The in-tree CUDA library; building it needs nvcc but no GPU."""
    from mini_llm_cuda_b200 import build
    build.build()
    from mini_llm_cuda_b200 import api
    return api.lib()
