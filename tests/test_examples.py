"""The examples as tests, like the reference's README asks (README.md:57-67): two ranks, each
script must end with PASSED.  CPU ranks over gloo and shared memory."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _torchrun(script, *args, timeout=600):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", OMP_NUM_THREADS="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), os.path.join(ROOT, "examples", script), *args]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)


@pytest.mark.parametrize("script", ["gaspiEx.py", "comprEx.py"])
def test_two_rank_examples_pass(script):
    res = _torchrun(script)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "PASSED" in res.stdout and "FAILED" not in res.stdout, res.stdout + res.stderr


def test_ddp_hook_example_runs():
    res = _torchrun("ddp_hook_train.py", "--steps", "20")
    assert res.returncode == 0, res.stdout + res.stderr
    assert "mean final loss" in res.stdout
