"""The compressed allreduce classes against the reference's own classes, call by call.

When ``COMPREX_REFERENCE`` names the reference's source tree, its ``Comprex_BigRingAllreduce``,
``Comprex_RingAllreduce`` and ``Comprex_AllToOneAllreduce`` (compiled unmodified against the
shared-memory GaspiCxx stand-in under ``baseline/``) run as P processes on the same float inputs as
this package's classes on P virtual ranks, configured for the reference's semantics
(``consistent=False``; Ring ``schedule="hops"``; AllToOne ``stale=True``).  Every rank's vector
after every call must agree bit for bit.  Skipped without the variable."""
import os
import subprocess
import sys
import uuid
import glob

import numpy as np
import pytest
import torch

import comprex_b200 as cx

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.environ.get("COMPREX_REFERENCE")
pytestmark = pytest.mark.skipif(not REF or not os.path.exists(os.path.join(REF or "", "src", "allreduce.tpp")),
                                reason="COMPREX_REFERENCE does not point at the reference's tree")


@pytest.fixture(scope="module")
def driver(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("refdrv") / "reference_allreduce_driver")
    cmd = [os.environ.get("CXX", "g++"), "-O2", "-std=c++14", "-fpermissive", "-w", "-ffp-contract=off"]
    for inc in (os.path.join(ROOT, "baseline", "gaspicxx_shim", "include"), os.path.join(REF, "include"),
                os.path.join(REF, "src")):
        cmd += ["-I", inc]
    cmd += [os.path.join(ROOT, "tests", "reference_allreduce_driver.cpp"), "-o", exe, "-lrt", "-lpthread"]
    subprocess.run(cmd, check=True)
    return exe


def run_reference(exe, variant, P, n, ratio, size_factor, runs, prefix_in, prefix_out):
    job = uuid.uuid4().hex[:10]
    ctl = f"/dev/shm/cxshim_{job}_ctl"
    with open(ctl, "wb") as f:
        f.truncate(2 << 20)
    try:
        procs = [subprocess.Popen([exe, variant, str(n), repr(ratio), repr(size_factor), str(runs), prefix_in, prefix_out],
                                  env=dict(os.environ, CXSHIM_RANK=str(r), CXSHIM_SIZE=str(P), CXSHIM_JOB=job),
                                  stdout=subprocess.DEVNULL, stderr=subprocess.PIPE) for r in range(P)]
        for p in procs:
            _, err = p.communicate(timeout=300)
            assert p.returncode == 0, err.decode()
    finally:
        for path in glob.glob(f"/dev/shm/cxshim_{job}_*"):
            os.unlink(path)


@pytest.mark.parametrize("variant", ["bigring", "ring", "alltoone"])
@pytest.mark.parametrize("P", [2, 3, 4])
@pytest.mark.parametrize("n,ratio", [(20011, 0.05), (100003, 0.01)])
def test_allreduce_matches_reference_call_by_call(driver, tmp_path, variant, P, n, ratio):
    runs, size_factor = 4, 3.0
    pin, pout = str(tmp_path / "in"), str(tmp_path / "out")
    inputs = {}
    for r in range(P):
        for k in range(runs + 1):                  # the last one goes through flush
            x = torch.randn(n, generator=torch.Generator().manual_seed(1000 * r + k))
            inputs[(r, k)] = x
            x.numpy().tofile(f"{pin}_r{r}_k{k}.bin")
    run_reference(driver, variant, P, n, ratio, size_factor, runs, pin, pout)

    world = cx.LoopbackWorld(P, device="cpu", timeout_ms=2000)
    if variant == "bigring":
        ars = [cx.Comprex_BigRingAllreduce(e) for e in world.envs]
        for a in ars:
            a.setup_connections(n, 1, ratio, size_factor, consistent=False)
    elif variant == "ring":
        ars = [cx.Comprex_RingAllreduce(e) for e in world.envs]
        for a in ars:
            a.setup_connections(n, 1, ratio, size_factor, schedule="hops")
    else:
        ars = [cx.Comprex_AllToOneAllreduce(e) for e in world.envs]
        for a in ars:
            a.setup_connections(n, 1, 0, ratio, size_factor, stale=True)
    changed = 0
    for k in range(runs):
        xs = [inputs[(r, k)].clone() for r in range(P)]
        world.run(ars, "apply", [(x,) for x in xs])
        changed += sum(int((xs[r] != inputs[(r, k)]).sum()) for r in range(P))
        for r in range(P):
            ref = torch.from_numpy(np.fromfile(f"{pout}_r{r}_k{k}.bin", dtype=np.float32))
            same = torch.equal(xs[r], ref)
            assert same, (f"rank {r}, call {k}: {int((xs[r] != ref).sum())} of {n} elements differ, "
                          f"max |diff| {float((xs[r] - ref).abs().max())}")
    assert changed > 0          # the calls did exchange something
    # flush: everything still held back arrives.  BigRing adds the peers' residuals in ring order
    # on both sides (bit for bit); the chief of AllToOne adds its workers in rank order (bit for
    # bit); the Ring's owners sum in ring order there and in rank order here (to rounding, and only
    # the chunk a rank owns is exact in the reference, test/RingAllreduce.cpp:87-100).
    xs = [inputs[(r, runs)].clone() for r in range(P)]
    world.run(ars, "flush", [(x,) for x in xs])
    for r in range(P):
        ref = torch.from_numpy(np.fromfile(f"{pout}_r{r}_k{runs}.bin", dtype=np.float32))
        if variant == "ring":
            a = ars[r]
            c = (r + 1) % P
            sl = slice(a.segment_starts[c], a.segment_starts[c] + a.segment_sizes[c])
            torch.testing.assert_close(xs[r][sl], ref[sl], rtol=1e-5, atol=1e-5)
        elif variant == "alltoone" and r != 0:
            continue                                   # workers' vectors are not defined by a flush
        else:
            assert torch.equal(xs[r], ref), f"flush, rank {r}: {int((xs[r] != ref).sum())} elements differ"
    world.close()


@pytest.mark.parametrize("variant", ["dense_bigring", "dense_ring", "dense_alltoone"])
@pytest.mark.parametrize("P", [2, 3, 4])
def test_dense_allreduce_matches_reference(driver, tmp_path, variant, P):
    """The dense classes: same sums as the reference's (bit for bit where the order of the
    additions is the same - BigRing, AllToOne; to rounding for the Ring, whose direct
    reduce-scatter adds in rank order instead of ring order)."""
    n, runs = 30011, 2
    pin, pout = str(tmp_path / "in"), str(tmp_path / "out")
    inputs = {}
    for r in range(P):
        for k in range(runs):
            x = torch.randn(n, generator=torch.Generator().manual_seed(77 * r + k))
            inputs[(r, k)] = x
            x.numpy().tofile(f"{pin}_r{r}_k{k}.bin")
    run_reference(driver, variant, P, n, 1.0, 1.0, runs, pin, pout)
    world = cx.LoopbackWorld(P, device="cpu", timeout_ms=2000)
    cls = {"dense_bigring": cx.BigRingAllreduce, "dense_ring": cx.RingAllreduce, "dense_alltoone": cx.AllToOneAllreduce}[variant]
    ars = [cls(e) for e in world.envs]
    for a in ars:
        if variant == "dense_alltoone":
            a.setup_connections(n, 1, 0)
        else:
            a.setup_connections(n, 1)
    for k in range(runs):
        xs = [inputs[(r, k)].clone() for r in range(P)]
        world.run(ars, "apply", [(x,) for x in xs])
        for r in range(P):
            ref = torch.from_numpy(np.fromfile(f"{pout}_r{r}_k{k}.bin", dtype=np.float32))
            if variant == "dense_ring" and P > 2:
                torch.testing.assert_close(xs[r], ref, rtol=1e-5, atol=1e-5)
            else:
                assert torch.equal(xs[r], ref), f"rank {r}, call {k}"
    world.close()
