"""The host back end under AddressSanitizer + UBSan and under ThreadSanitizer
(csrc/selftest/host_selftest.cpp): edge sizes, capacity limits, canaries around every
slot, the two-parity slot protocol between two threads, a bounded wait that runs out."""
import subprocess

import pytest

from comprex_b200 import build as B


@pytest.mark.parametrize("sanitizer,args", [("address,undefined", []), ("thread", ["--protocol"])])
def test_host_backend_under_sanitizers(sanitizer, args):
    try:
        exe = B.build_selftest(sanitizer)
    except RuntimeError as e:
        if "cannot find" in str(e) or "unrecognized" in str(e):
            pytest.skip("no compiler with the sanitizer runtime on this machine")
        raise
    res = subprocess.run([str(exe)] + args, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "host selftest passed" in res.stdout
