import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "exllamav3-rs_b200"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")


@pytest.fixture(scope="session")
def ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import exl3b200
    c = exl3b200.Ctx(0)
    yield c
    c.close()


@pytest.fixture(scope="session")
def ref():
    """The reference's own CUDA ops (oracle/_ref/libexl3ref.so), when that library was built; else None."""
    from tests import helpers
    return helpers.load_ref()
