"""The native (C/C++) collectives: the C++ example program run as a test, the reference's C symbol
names, and bit-for-bit agreement of the native schedules with the Python classes on real ranks."""
import ctypes as C
import os
import re
import subprocess

import pytest
import torch
import torch.distributed as dist

import comprex_b200 as cx
from comprex_b200 import _lib, build
from comprex_b200.native import NativeAllreduce

from test_multiprocess import gpu_world, run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("COMPREX_REFERENCE")


@pytest.fixture(scope="module")
def example_exe(tmp_path_factory):
    lib = build.build()
    exe = tmp_path_factory.mktemp("native") / "native_allreduce"
    cmd = [os.environ.get("CXX", "g++"), "-std=c++17", "-O2", os.path.join(ROOT, "examples", "native_allreduce.cpp"),
           "-I" + os.path.join(ROOT, "comprex_b200", "csrc"), "-L" + str(lib.parent), "-lcomprex_b200",
           "-Wl,-rpath," + str(lib.parent), "-o", str(exe)]
    res = subprocess.run(cmd, capture_output=True, text=True)
    assert res.returncode == 0, res.stdout + res.stderr
    return str(exe)


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4, 5])
@pytest.mark.parametrize("ranks", [2, 3])
def test_cpp_example_host_ranks(example_exe, kind, ranks):
    res = subprocess.run([example_exe, "--host", "--ranks", str(ranks), "--kind", str(kind), "--size", "5003",
                          "--runs", "8", "--ratio", "0.05"], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0 and "+++ PASSED +++" in res.stdout, res.stdout + res.stderr


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("kind", [5, 3, 4])
def test_cpp_example_gpu_ranks(example_exe, kind):
    env = dict(os.environ, COMPREX_TIMEOUT_MS="5000")
    res = subprocess.run([example_exe, "--ranks", "2", "--kind", str(kind), "--size", "100003", "--runs", "6",
                          "--ratio", "0.01"], capture_output=True, text=True, timeout=300, env=env)
    assert res.returncode == 0 and "+++ PASSED +++" in res.stdout, res.stdout + res.stderr


def test_library_exports_the_reference_c_names():
    """Every function of the reference's allreduce and environment C ABI is exported under the same
    name (src/allreduce_C.cpp:12-122, src/GPI_C.cpp:44-73)."""
    lib = _lib.load()
    names = ["GaspiEnvironment_new", "GaspiEnvironment_del", "GaspiEnvironment_get_rank", "GaspiEnvironment_get_ranks",
             "GaspiEnvironment_barrier", "GaspiEnvironment_flush", "Gaspi_Printf"]
    for cls in ("AllToOneAllreduce", "RingAllreduce", "BigRingAllreduce"):
        names += [f"{cls}_{m}" for m in ("new", "del", "setupConnections", "apply")]
        names += [f"Comprex_{cls}_{m}" for m in ("new", "del", "setupConnections", "apply", "flush", "reset",
                                                  "set_compression_ratio")]
    if REF and os.path.exists(os.path.join(REF, "src", "allreduce_C.cpp")):
        src = open(os.path.join(REF, "src", "allreduce_C.cpp")).read()
        found = set(re.findall(r"\b((?:Comprex_)?\w+Allreduce_\w+)\s*\(", src))
        assert found and found <= set(names), found - set(names)
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def scenario_native_matches_python(rank, world, device):
    """The C++ schedules against the Python ones: same inputs, several calls, then flush; every
    vector must agree bit for bit (both drive the same primitives in the same order)."""
    env = cx.GaspiEnvironment(16 << 20, device=device, timeout_ms=5000)
    n = 20011
    cases = [("comprex_bigring", dict(consistent=False)), ("comprex_bigring", dict(consistent=True)),
             ("comprex_ring", dict()), ("comprex_ring", dict(consistent=True, chunk_align=4)),
             ("comprex_alltoone", dict()), ("bigring", dict()), ("ring", dict()), ("alltoone", dict())]
    py_cls = {"comprex_bigring": cx.Comprex_BigRingAllreduce, "comprex_ring": cx.Comprex_RingAllreduce,
              "comprex_alltoone": cx.Comprex_AllToOneAllreduce, "bigring": cx.BigRingAllreduce,
              "ring": cx.RingAllreduce, "alltoone": cx.AllToOneAllreduce}
    for kind, kw in cases:
        py = py_cls[kind](env)
        if kind == "comprex_alltoone":
            py.setup_connections(n, 1, 0, 0.03, 2.5)
        elif kind.startswith("comprex"):
            py.setup_connections(n, 1, 0.03, 2.5, **kw)
        elif kind == "alltoone":
            py.setup_connections(n, 1, 0)
        else:
            py.setup_connections(n, 1)
        nat = NativeAllreduce(env, kind, n, 0.03, 2.5, **kw)
        for step in range(4):
            torch.manual_seed(100 * step + rank)
            x = torch.randn(n, device=device)
            a, b = x.clone(), x.clone()
            py.apply(a)
            nat.apply(b)
            env.flush()
            nat.check()
            assert torch.equal(a, b), f"{kind} {kw}: call {step} differs"
        if kind.startswith("comprex"):
            a, b = torch.zeros(n, device=device), torch.zeros(n, device=device)
            py.flush(a)
            nat.flush(b)
            env.flush()
            nat.check()
            assert torch.equal(a, b), f"{kind} {kw}: flush differs"
            sd = nat.state_dict()
            assert sd["step"] > 4 and float(sd["residual"].abs().sum()) == 0.0
            assert nat.stats()["n"] > 0
        env.barrier()
    env.barrier()
    env.close()
    return True


@pytest.mark.parametrize("world", [2, 3])
def test_native_schedules_match_python_cpu(world):
    assert all(run_ranks(world, "test_native_collectives:scenario_native_matches_python"))


@pytest.mark.gpu
@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_native_schedules_match_python_gpus():
    assert all(run_ranks(gpu_world(), "test_native_collectives:scenario_native_matches_python", backend="nccl"))
