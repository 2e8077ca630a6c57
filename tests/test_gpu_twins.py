"""GPU: the mma.sync twins of the tcgen05 kernels. The library picks the tcgen05 kernels for K = V = 128 on its own, so
the chunk-op parity tests are run once more in a child process with FLA_B200_NO_TC=1 (the switch is read once per
process), which sends the same shapes through the mma.sync kernels."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def test_chunk_ops_with_tensor_core_kernels_disabled():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, FLA_B200_NO_TC="1")
    sel = "test_chunk_simple_gla or test_chunk_delta_rule or test_chunk_gated_delta_rule or test_chunk_retention"
    r = subprocess.run([sys.executable, "-m", "pytest", os.path.join(here, "test_gpu_ops.py"), "-m", "gpu", "-q", "-x", "-k", sel],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-2000:]
    assert " passed" in r.stdout
