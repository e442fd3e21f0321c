"""Randomised properties of the native primitives (host back end; the CUDA kernels are tied to it
bit for bit by test_primitives.py): conservation through compression, residual and capacity
limits; decode of what was encoded; run-length round trips on arbitrary masks."""
import pytest
import torch
from hypothesis import HealthCheck, given, settings, strategies as st

import comprex_b200 as cx
from comprex_b200 import _lib
from comprex_b200.ops import primitives as P

from test_primitives import read_pairs

SETTINGS = dict(max_examples=40, deadline=None, suppress_health_check=[HealthCheck.function_scoped_fixture])


@pytest.fixture(scope="module")
def cpu_world():
    w = cx.LoopbackWorld(2, device="cpu", timeout_ms=200)
    yield w
    w.close()


@settings(**SETTINGS)
@given(n=st.integers(1, 5000), thr=st.sampled_from([0.0, 0.3, 1.0, 2.5, 50.0]), cap_frac=st.floats(0.01, 1.0),
       seed=st.integers(0, 2 ** 16), with_g=st.booleans())
def test_compress_conserves_and_respects_capacity(cpu_world, n, thr, cap_frac, seed, with_g):
    """sent + new residual == old residual + input, element by element and exactly; at most `cap`
    pairs, in index order inside every sub-tile; what does not fit stays in the residual."""
    e0, e1 = cpu_world.envs
    cap = max(1, int(n * cap_frac))
    gen = torch.Generator().manual_seed(seed)
    g = torch.randn(n, generator=gen) if with_g else None
    r0 = torch.randn(n, generator=gen) * 0.5
    r = r0.clone()
    mark = e0.heap_mark()
    slot = [P.SparseSlot.create(e, n, cap) for e in cpu_world.envs][1]
    comp = P.Compressor(e0, n)
    comp.set_threshold(thr)
    comp.compress(g, r, n, cap, 1, P.make_targets([slot.endpoint(e0, 1)]))
    hdr, idx, val, counts = read_pairs(e1, slot)
    total = r0 + (g if with_g else 0)
    sent = torch.zeros(n)
    sent[idx.long()] = val
    assert torch.equal(sent + r, total)
    assert hdr.nnz <= cap and hdr.nnz == idx.numel() and hdr.nnz_found >= hdr.nnz
    assert int((total.abs() > thr).sum()) == hdr.nnz_found
    assert bool((val.abs() > thr).all())
    if hdr.nnz_found <= cap:                       # everything above the threshold went out
        assert hdr.nnz == hdr.nnz_found and not bool((r.abs() > thr).any())
    assert int(counts.sum()) == hdr.nnz
    stats = comp.last_stats()
    assert stats["nnz"] == hdr.nnz and bool(stats["status"] & _lib.ST_OVERFLOW) == (hdr.nnz_found > cap)
    e0.heap_release(mark)


@settings(**SETTINGS)
@given(n=st.integers(1, 4000), nsrc=st.integers(1, 5), seed=st.integers(0, 2 ** 16),
       op=st.sampled_from(["add", "set", "sgd_wd"]))
def test_apply_equals_dense_restatement(cpu_world, n, nsrc, seed, op):
    """Decoding several payloads in source order equals adding their dense forms in that order."""
    e0, _ = cpu_world.envs
    gen = torch.Generator().manual_seed(seed)
    mark = e0.heap_mark()
    slots, dense = [], []
    for j in range(nsrc):
        x = torch.randn(n, generator=gen) * (torch.rand(n, generator=gen) < 0.3)
        slot = [P.SparseSlot.create(e, n, n) for e in cpu_world.envs][0]
        comp = P.Compressor(e0, n)
        comp.set_threshold(0.0)
        comp.compress(x, None, n, n, 1, P.make_targets([slot.endpoint(e0, 0)]))
        slots.append(slot)
        dense.append(x)
    src = P.make_sources([s.endpoint(e0, 0) for s in slots], [1] * nsrc)
    base = torch.randn(n, generator=gen)
    out = base.clone()
    status = e0.new_status("p")
    scale = 0.5
    if op == "add":
        P.apply_sparse(e0, src, n, P.args_add(out, scale), status)
        want = base.clone()
        for x in dense:
            want = want + scale * x
    elif op == "set":
        P.apply_sparse(e0, src, n, P.args_set(out, scale), status)
        acc = torch.zeros(n)
        for x in dense:
            acc = acc + x
        want = scale * acc
    else:
        P.apply_sparse(e0, src, n, P.args_update(_lib.OP_SGD, out, scale, wd=0.1), status)
        acc = torch.zeros(n)
        for x in dense:
            acc = acc + x
        want = (1 - 0.1) * base - scale * acc
    assert status.value == 0
    assert torch.equal(out, want)
    e0.heap_release(mark)


@settings(**SETTINGS)
@given(n=st.integers(0, 3000), thr=st.sampled_from([0.0, 0.5, 1.5]), seed=st.integers(0, 2 ** 16),
       density=st.floats(0.0, 1.0), add=st.booleans())
def test_rle_round_trip(n, thr, seed, density, add):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(n, generator=gen) * (torch.rand(n, generator=gen) < density)
    r = torch.zeros(n)
    payload = cx.CompressorRLE.encode(x, r, thr)
    keep = (x.abs() >= thr) & ~((thr == 0.0) & (x == 0))
    base = torch.randn(n, generator=gen)
    out = base.clone()
    cx.CompressorRLE.decode(payload, out, add=add)
    kept = torch.where(keep, x, torch.zeros(n))
    assert torch.equal(out, base + kept if add else kept)
    assert torch.equal(r, torch.where(keep, torch.zeros(n), x))
    nnz = int.from_bytes(payload[4:8], "little")
    assert nnz == int(keep.sum()) and len(payload) <= 16 + 8 * n
