"""The vLLM hook inside a running engine (tests/vllm_engine_check.py in a child process; about two minutes, most of it
engine start-up)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sparse_prefill_hook_inside_a_vllm_engine():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    try:
        import vllm  # noqa: F401
    except Exception as e:
        pytest.skip(f"vLLM cannot be imported here: {type(e).__name__}")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "vllm_engine_check.py")], capture_output=True, text=True,
                       timeout=900)
    out = p.stdout + p.stderr
    if "engine up" not in out:          # the engine itself did not start on this machine: nothing of this library ran
        pytest.skip("the vLLM engine did not come up: " + out[-400:].replace("\n", " | "))
    print("\n".join(line for line in out.splitlines() if "tokens" in line or "logprob" in line or "ENGINE_" in line))
    assert p.returncode == 0, out[-3000:]
    assert "ENGINE_OK" in out and "sparse prefill calls 2" in out
