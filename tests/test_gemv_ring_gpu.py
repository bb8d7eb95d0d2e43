"""The TMA-fed GEMV kernels (opt-in, IRON_GEMV_RING) against the same references as the
register-streamed ones: the GEMV tests re-run in a child process with every shape routed
through them (the switch is read once per process)."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


def test_every_gemv_shape_through_the_tma_fed_kernels():
    root = Path(__file__).resolve().parents[1]
    env = dict(os.environ, IRON_GEMV_RING="15")
    run = subprocess.run(
        [sys.executable, "-m", "pytest", "tests/test_kernels_gpu.py", "tests/test_engine_gpu.py", "-q", "-x",
         "-m", "gpu", "-k", "gemv or swiglu or qkv or decode or golden", "-p", "no:cacheprovider"],
        cwd=root, env=env, capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-3000:] + run.stderr[-2000:]
    assert " passed" in run.stdout
