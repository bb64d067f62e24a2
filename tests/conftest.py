import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")
    # The native library is part of what is under test: (re)build it when nvcc is
    # around and the sources are newer; otherwise the prebuilt in-tree .so is used.
    from humming_b200 import build as hm_build

    try:
        hm_build.build()
    except Exception as exc:  # pragma: no cover - surfaced by the import in the tests
        sys.stderr.write(f"[conftest] could not build libhumming_b200.so: {exc}\n")


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    return torch.device("cuda:0")
