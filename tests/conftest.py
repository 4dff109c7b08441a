import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as o
    o.load()
    return o


@pytest.fixture(scope="session")
def cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from raft_b200 import _lib
    _lib.load()  # raises if the extension is not built: GPU tests never run on a fallback
    return torch.device("cuda:0")


@pytest.fixture
def knobs(monkeypatch):
    """Sets B2R_* launch-shape knobs for one test: the library reads its environment once, so every
    change is followed by reload_tuning(), and the defaults are restored (and re-read) afterwards."""
    from raft_b200 import linalg

    def set_knobs(**kv):
        for k, v in kv.items():
            if v is None:
                monkeypatch.delenv(k, raising=False)  # back to the built-in default
            else:
                monkeypatch.setenv(k, str(v))
        linalg.reload_tuning()

    yield set_knobs
    monkeypatch.undo()
    linalg.reload_tuning()
