"""The range-checked debug build of the library (-DMINF_BOUNDS) on tiny and ragged cases."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_range_checked_build_runs_clean_on_small_and_ragged_cases():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    lib = os.path.join(ROOT, "minference_b200", "libminfer_b200_bounds.so")
    if not os.path.exists(lib):
        pytest.skip("the range-checked build is not present (python -m minference_b200.build --bounds)")
    env = dict(os.environ, MINFER_B200_LIB=lib)
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "bounds_build_check.py")], env=env, capture_output=True,
                       text=True, timeout=600)
    assert p.returncode == 0 and "BOUNDS_OK" in p.stdout, p.stdout[-2000:] + p.stderr[-2000:]
