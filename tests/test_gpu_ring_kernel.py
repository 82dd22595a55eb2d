"""The bulk-copy-ring kernel on the cases the plain-load kernel serves by default.

Which streaming kernel runs is fixed when the library first launches, so the parity tests are
run again in a child process with MANTLE_SAMPLER_KERNEL=tma."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_parity_suite_with_the_ring_kernel():
    env = dict(os.environ, MANTLE_SAMPLER_KERNEL="tma")
    cmd = [sys.executable, "-m", "pytest", os.path.join(ROOT, "tests", "test_gpu_parity.py"), "-m", "gpu", "-x", "-q",
           "-k", "not long_shortlist and not full_vocab and not full_size"]
    res = subprocess.run(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert res.returncode == 0, res.stdout[-3000:]
