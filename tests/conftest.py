import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line('markers', 'gpu: needs a CUDA device (run with -m gpu on a B200)')


@pytest.fixture(scope='session')
def built_library():
    """the C-ABI shared library, built if missing (nvcc works without a GPU)"""
    from vesta_gpu_b200 import build
    return build.build_library()
