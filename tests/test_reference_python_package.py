"""The reference's own Python package, built against the shared-memory GaspiCxx stand-in by
baseline/install_reference_python.py, runs its Python tests (two processes each) and they end with
PASSED.  Needs ``COMPREX_REFERENCE``; skipped without it."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("COMPREX_REFERENCE")
pytestmark = pytest.mark.skipif(not REF or not os.path.exists(os.path.join(REF or "", "allreduce.py")),
                                reason="COMPREX_REFERENCE does not point at the reference's tree")


@pytest.mark.parametrize("script", ["test/BigRingAllreduce.py", "test/RingAllreduce.py", "test/AllToOneAllreduce.py",
                                    "examples/comprEx.py"])
def test_reference_python_tests_pass_on_the_stand_in(script):
    res = subprocess.run([sys.executable, os.path.join(ROOT, "baseline", "install_reference_python.py"),
                          "--reference", REF, "--run", script, "--ranks", "2"], capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "PASSED" in res.stdout and "FAILED" not in res.stdout, res.stdout[-2000:]
