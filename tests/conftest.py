import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "flash-linear-attention_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "ref_vectors.npz"))


@pytest.fixture(scope="session", autouse=True)
def tc_error_word_stays_clear():
    """After the whole session: no tcgen05 kernel may have recorded a timed-out wait."""
    yield
    import torch
    if torch.cuda.is_available():
        from fla_b200 import _lib
        lib = _lib.load()
        torch.cuda.synchronize()
        assert lib.flab_tc_error_state() == 0, f"a bounded device-side wait ran out: id {lib.flab_tc_error_state()}"
