"""The checked build of the kernels (PAE_BOUNDS=1; csrc/common.cuh): it stands in for a memory
checker, which is not to be had on every machine. The build is chosen when the package is
imported, so the checks run in a process of their own: tests/bounds_probe.py replays mixed
traces on it (no index may be out of range, and the logits must be the plain model's) and then
feeds the kernels indices that are out of range, which must be caught and skipped."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu


def test_the_engine_on_the_checked_build():
    probe = Path(__file__).resolve().parent / "bounds_probe.py"
    env = dict(os.environ, PAE_BOUNDS="1")
    done = subprocess.run([sys.executable, str(probe)], capture_output=True, text=True, timeout=1500, env=env)
    assert done.returncode == 0, (done.stdout[-3000:] + "\n" + done.stderr[-3000:])
    assert "BOUNDS PROBE OK" in done.stdout
    assert "indices out of range were caught and skipped" in done.stdout
