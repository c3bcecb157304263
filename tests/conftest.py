import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import jq_oracle

    jq_oracle.build()
    return jq_oracle


@pytest.fixture(scope="session")
def native_lib():
    """The built C-ABI library; building is attempted once if it is missing."""
    lib_path = os.path.join(ROOT, "jjjetson_ops_b200", "libjq_b200.so")
    if not os.path.exists(lib_path):
        from jjjetson_ops_b200 import _build

        _build.build_all()
    from jjjetson_ops_b200 import capi

    return capi


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")
