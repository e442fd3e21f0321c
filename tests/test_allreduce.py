"""The six allreduce variants on P virtual ranks of one device.

The compressed tests follow the reference's pattern (test/AllToOneAllreduce.cpp,
test/RingAllreduce.cpp, test/BigRingAllreduce.cpp): one rank keeps accumulating
across runs while the others reset their input; after ``flush`` the accumulator
must equal ``(runs*(P-1)+1) * values`` exactly, i.e. nothing is lost to
thresholding, residuals and flush together conserve the sum.
"""
import pytest
import torch

import comprex_b200 as cx

from helpers import alt_ramp

RANKS = [1, 2, 3, 4, 8]


@pytest.fixture(params=RANKS)
def world(request, device):
    w = cx.LoopbackWorld(request.param, device=device, timeout_ms=500)
    yield w
    w.close()


@pytest.mark.parametrize("cls,kw", [(cx.AllToOneAllreduce, dict(chiefRank=0)), (cx.RingAllreduce, {}),
                                    (cx.BigRingAllreduce, {})])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense_allreduce(world, cls, kw, dtype):
    n, P = 10007, world.size
    ars = [cls(e) for e in world.envs]
    for a in ars:
        a.setup_connections(n, 1, dtype=dtype, **kw)
    for step in range(3):
        torch.manual_seed(step)
        xs = [torch.randn(n).to(dtype).to(world.device) for _ in range(P)]
        ref = sum(x.double() for x in xs)
        world.run(ars, "apply", [(x,) for x in xs])
        tol = 1e-5 if dtype == torch.float32 else 0.1
        for x in xs:
            assert (x.double() - ref).abs().max().item() < tol
        if cls is not cx.BigRingAllreduce:   # one reducer per element: identical bits everywhere
            for x in xs[1:]:
                assert torch.equal(x, xs[0])


@pytest.mark.parametrize("cls,kw", [(cx.Comprex_BigRingAllreduce, {}), (cx.Comprex_RingAllreduce, {}),
                                    (cx.Comprex_RingAllreduce, dict(schedule="hops")),
                                    (cx.Comprex_AllToOneAllreduce, dict(chiefRank=0)),
                                    (cx.Comprex_AllToOneAllreduce, dict(chiefRank=0, stale=True))])
@pytest.mark.parametrize("n,ratio", [(50, 0.01), (1000, 0.01), (20011, 0.05)])
def test_compressed_allreduce_conserves_sum(world, cls, kw, n, ratio):
    P, dev = world.size, world.device
    ars = [cls(e) for e in world.envs]
    for a in ars:
        a.setup_connections(n, 1, compression_ratio=ratio, size_factor=3.0, **kw)
    vals = alt_ramp(n, dev)
    runs = 6
    acc = vals.clone()
    for _ in range(runs):
        xs = [acc] + [vals.clone() for _ in range(P - 1)]
        world.run(ars, "apply", [(x,) for x in xs])
    xs = [acc] + [torch.zeros(n, device=dev) for _ in range(P - 1)]
    world.run(ars, "flush", [(x,) for x in xs])
    expect = (runs * (P - 1) + 1) * vals
    if cls is cx.Comprex_RingAllreduce and P > 1:
        a = ars[0]
        c = 1 % P   # rank 0 owns chunk 1 and keeps it dense (test/RingAllreduce.cpp:87-100)
        sl = slice(a.segment_starts[c], a.segment_starts[c] + a.segment_sizes[c])
        assert torch.equal(acc[sl], expect[sl])
    else:
        assert torch.equal(acc, expect)
    for a in ars:
        for r in a._residuals():
            assert float(r.abs().sum()) == 0.0


def test_stale_alltoone_is_one_call_late(device):
    """stale=True (the reference's FastComprEx legs): what a call compresses arrives with the next
    call.  With a zero vector on the chief, its result of call s equals the fresh mode's result of
    call s-1 bit for bit, and the first call delivers nothing."""
    n, P = 6000, 3
    outs = {}
    for stale in (False, True):
        w = cx.LoopbackWorld(P, device=device, timeout_ms=500)
        ars = [cx.Comprex_AllToOneAllreduce(e) for e in w.envs]
        for a in ars:
            a.setup_connections(n, 1, 0, 0.05, 3.0, stale=stale)
        chief_after, worker_after = [], []
        for step in range(5):
            xs = [torch.zeros(n, device=device)] + [
                torch.randn(n, generator=torch.Generator().manual_seed(10 * step + r)).to(device) for r in range(1, P)]
            w.run(ars, "apply", [(x,) for x in xs])
            chief_after.append(xs[0].cpu().clone())
            worker_after.append(xs[1].cpu().clone())
        outs[stale] = (chief_after, worker_after)
        w.close()
    fresh, stale = outs[False][0], outs[True][0]
    assert float(stale[0].abs().sum()) == 0.0 and float(fresh[0].abs().sum()) > 0.0
    for s in range(1, 5):
        assert torch.equal(stale[s], fresh[s - 1])
    assert float(outs[True][1][0].abs().sum()) == 0.0          # first broadcast is empty too


def test_ring_schedules_agree_on_two_ranks(device):
    """With two ranks the direct schedule is the hop-by-hop ring of the reference: same bits."""
    results = []
    for schedule in ("direct", "hops"):
        w = cx.LoopbackWorld(2, device=device, timeout_ms=500)
        ars = [cx.Comprex_RingAllreduce(e) for e in w.envs]
        for a in ars:
            a.setup_connections(20011, 1, compression_ratio=0.05, size_factor=3.0, schedule=schedule)
        outs = []
        for step in range(4):
            xs = [torch.randn(20011, generator=torch.Generator().manual_seed(10 * step + r)).to(device) for r in range(2)]
            w.run(ars, "apply", [(x,) for x in xs])
            outs += [x.cpu() for x in xs]
        outs += [r.cpu().clone() for a in ars for r in a._residuals()]
        results.append(outs)
        w.close()
    for a, b in zip(*results):
        assert torch.equal(a, b)


def test_consistent_bigring_replicas_identical_and_conserving(world):
    P, dev, n = world.size, world.device, 30011
    ars = [cx.Comprex_BigRingAllreduce(e) for e in world.envs]
    for a in ars:
        a.setup_connections(n, 1, compression_ratio=0.02, size_factor=3.0, consistent=True)
    total = torch.zeros(n, dtype=torch.float64)
    inputs = torch.zeros(n, dtype=torch.float64)
    for step in range(8):
        torch.manual_seed(step)
        xs = [torch.randn(n).to(dev) for _ in range(P)]
        inputs += sum(x.double().cpu() for x in xs)
        world.run(ars, "apply", [(x,) for x in xs])
        for x in xs[1:]:
            assert torch.equal(x, xs[0])
        frac = float((xs[0] != 0).float().mean())
        assert frac <= min(1.0, 0.02 * 1.6 * P)
        total += xs[0].double().cpu()
    xs = [torch.zeros(n, device=dev) for _ in range(P)]
    world.run(ars, "flush", [(x,) for x in xs])
    total += xs[0].double().cpu()
    assert (total - inputs).abs().max().item() < 1e-4


def test_ring_result_is_topk_of_reduced_chunk(world):
    """Non-owners receive exactly the entries of the owner's reduced chunk that pass its threshold."""
    P, dev, n = world.size, world.device, 40000
    if P < 2:
        pytest.skip("needs peers")
    ars = [cx.Comprex_RingAllreduce(e) for e in world.envs]
    for a in ars:
        a.setup_connections(n, 1, compression_ratio=0.05, size_factor=2.5)
    torch.manual_seed(3)
    xs = [torch.randn(n).to(dev) for _ in range(P)]
    world.run(ars, "apply", [(x,) for x in xs])
    a = ars[0]
    for owner in range(P):
        c = (owner + 1) % P
        sl = slice(a.segment_starts[c], a.segment_starts[c] + a.segment_sizes[c])
        dense = xs[owner][sl]
        for r in range(P):
            if r == owner:
                continue
            got = xs[r][sl]
            nz = got != 0
            assert torch.equal(got[nz], dense[nz])
            assert 0 < int(nz.sum()) < 0.2 * dense.numel()


def test_set_compression_ratio_and_state_dict(world):
    P, dev, n = world.size, world.device, 20000
    ars = [cx.Comprex_BigRingAllreduce(e) for e in world.envs]
    for a in ars:
        a.setup_connections(n, 1, compression_ratio=0.01, size_factor=2.5, consistent=True)
    xs = [torch.randn(n).to(dev) for _ in range(P)]
    world.run(ars, "apply", [(x.clone(),) for x in xs])
    lo = ars[0].stats()["nnz"]
    for a in ars:
        a.set_compression_ratio(0.1)
    world.run(ars, "apply", [(x.clone(),) for x in xs])
    assert ars[0].stats()["nnz"] > 3 * lo
    sd = ars[0].state_dict()
    assert sd["ratio"] == pytest.approx(0.1) and sd["residuals"][0].abs().sum() > 0
    saved = ars[0].rests.clone()
    ars[0].reset()
    assert float(ars[0].rests.abs().sum()) == 0.0
    ars[0].load_state_dict(sd)
    assert torch.equal(ars[0].rests, saved)


def test_apply_checks_size_and_accepts_numpy():
    import numpy as np
    env = cx.GaspiEnvironment(1 << 20, device="cpu")
    ar = cx.Comprex_BigRingAllreduce(env)
    ar.setup_connections(100, 1, 0.1, 3.0)
    with pytest.raises(cx.ComprexError, match="does not match allreduce size"):
        ar.apply(torch.zeros(99))
    v = np.arange(100, dtype=np.float32).reshape(10, 10)
    out = ar.apply(v)
    assert out is v and out.shape == (10, 10)      # single rank: own dense data is kept
    assert np.array_equal(v.reshape(-1), np.arange(100, dtype=np.float32))
    assert ar.getSize() == 100
    env.close()


def test_select_schedule_follows_the_measured_regimes():
    """The cost model ranks the three schedules the way the sweeps on 2, 4 and 8 B200 did: tiny and
    dense vectors go to the dense kernels, the compressed BigRing wins while (P-1) payloads are
    small, the compressed Ring for large vectors, high ratios and many peers."""
    from comprex_b200.allreduce import schedule_costs, select_schedule
    assert select_schedule(1 << 16, 0.01, 8) == "bigring"
    assert select_schedule(1 << 16, 0.001, 2) == "bigring"
    assert select_schedule(1 << 24, 1.0, 8) == "bigring"            # nothing to compress
    assert select_schedule(1 << 20, 0.01, 4) == "comprex_bigring"
    assert select_schedule(1 << 24, 0.01, 2) == "comprex_bigring"
    assert select_schedule(1 << 24, 0.01, 8) == "comprex_bigring"
    assert select_schedule(1 << 24, 0.1, 8) == "comprex_ring"
    assert select_schedule(1 << 28, 0.01, 8) == "comprex_ring"
    assert select_schedule(1 << 28, 0.1, 2) == "comprex_ring"
    assert select_schedule(1000, 0.01, 1) == "comprex_bigring"      # a single rank exchanges nothing
    # more peers cost the BigRing (P-1) payloads, the Ring 2 (P-1)/P of one
    c4, c8 = schedule_costs(1 << 26, 0.1, 4), schedule_costs(1 << 26, 0.1, 8)
    assert c8["comprex_bigring"] - c4["comprex_bigring"] > 4 * (c8["comprex_ring"] - c4["comprex_ring"])
    # a 16-bit vector halves the dense traffic, not the pairs
    assert schedule_costs(1 << 26, 0.01, 8, 2)["bigring"] < 0.6 * schedule_costs(1 << 26, 0.01, 8, 4)["bigring"]


@pytest.mark.parametrize("n,ratio,want", [(3000, 0.01, "bigring"), (1 << 20, 0.01, "comprex_bigring")])
def test_auto_allreduce_is_the_chosen_schedule(device, n, ratio, want):
    """AutoAllreduce sets up the schedule select_schedule names and gives its bits."""
    results = {}
    for kind in ("auto", "explicit"):
        w = cx.LoopbackWorld(3, device=device, timeout_ms=2000)
        ars = []
        for e in w.envs:
            if kind == "auto":
                a = cx.AutoAllreduce(e)
                a.setup_connections(n, 1, ratio, 3.0)
                assert a.choice == want and a.compressed == (want != "bigring")
                ars.append(a.impl)
            elif want == "bigring":
                a = cx.BigRingAllreduce(e)
                a.setup_connections(n, 1, ordered=True)
                ars.append(a)
            else:
                a = cx.Comprex_BigRingAllreduce(e)
                a.setup_connections(n, 1, ratio, 3.0, consistent=True)
                ars.append(a)
        out = []
        for step in range(3):
            torch.manual_seed(10 + step)
            xs = [torch.randn(n).to(device) for _ in range(3)]
            w.run(ars, "apply", [(x,) for x in xs])
            assert all(torch.equal(x, xs[0]) for x in xs[1:])       # replicas agree in both cases
            out.append(xs[0].cpu())
        results[kind] = out
        w.close()
    for a, b in zip(results["auto"], results["explicit"]):
        assert torch.equal(a, b)

