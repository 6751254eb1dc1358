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
    from oracle import gs_oracle

    gs_oracle.build()
    return gs_oracle


@pytest.fixture(scope="session")
def gsb():
    """The package with its native libraries; GPU tests fail loudly if they are missing."""
    import torch

    assert torch.cuda.is_available(), "GPU test collected on a machine without CUDA"
    import gsampler_b200

    return gsampler_b200
