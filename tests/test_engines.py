"""GaspiEx / Comprex / FastComprex on two (or three) virtual ranks of one device.

Scenarios follow the reference's own checks: test/comprex.cpp (3 x writeRemote +
flushRests, receiver accumulates with readRemote_add, result == 3 * values),
examples/comprEx.cpp, examples/gaspiEx.py.
"""
import numpy as np
import pytest
import torch

import comprex_b200 as cx

from helpers import alt_ramp


@pytest.fixture
def world(device):
    w = cx.LoopbackWorld(3, device=device, timeout_ms=300)
    yield w
    w.close()


def make(world, cls, *args, **kw):
    return [cls(e, *args, **kw) for e in world.envs]


def test_gaspiex_roundtrip_and_add(world):
    n, dev = 5003, world.device
    ex = make(world, cx.GaspiEx, n)
    ex[0].connectTx(1, 0)
    ex[1].connectRx(0, 0)
    for step in range(4):   # more messages than slots: parity reuse
        v = torch.randn(n, device=dev)
        ex[0].writeRemote(v)
        if step % 2 == 0:
            assert torch.equal(ex[1].readRemote(), v)
        else:
            acc = torch.ones(n, device=dev)
            ex[1].readRemote_add(acc)
            assert torch.equal(acc, v + 1)
    with pytest.raises(cx.ComprexError, match="too large"):
        ex[0].writeRemote(torch.zeros(n + 1, device=dev))
    with pytest.raises(cx.ComprexError, match="without connecting"):
        ex[2].writeRemote(torch.zeros(n, device=dev))


def test_gaspiex_numpy_vectors_and_short_messages(world):
    ex = make(world, cx.GaspiEx, 100)
    ex[0].connectTx(2, 5)
    ex[2].connectRx(0, 5)
    v = np.arange(60, dtype=np.float32)
    ex[0].writeRemote(v)
    out = np.zeros(60, dtype=np.float32)
    ex[2].readRemote_vec(out, 60)
    assert np.array_equal(out, v)


def test_gaspiex_broadcast_shared_buffer_and_forward(world):
    n, dev = 2000, world.device
    ex = make(world, cx.GaspiEx, n)
    v = torch.randn(n, device=dev)
    # chief 0 -> {1, 2} in one launch
    ex[0].writeRemote_multi(v, [1, 2])
    for r in (1, 2):
        ex[r].connectRx(0, 0)
        assert torch.equal(ex[r].readRemote(), v)
    # shared-buffer fan-out of the reference: second engine re-sends the first one's vector
    a, b = make(world, cx.GaspiEx, n), make(world, cx.GaspiEx, n)
    a[0].connectTx(1, 1)
    b[0].connectTx_sameBufferAs(2, 2, a[0])
    a[1].connectRx(0, 1)
    b[2].connectRx(0, 2)
    a[0].writeRemote(v)
    b[0].writeRemote(size=n)
    assert torch.equal(a[1].readRemote(), v) and torch.equal(b[2].readRemote(), v)
    # ring hop: 0 -> 1 -> 2 with forward_buffer / forward_add
    ring = make(world, cx.GaspiEx, n)
    ring[0].connectTx(1, 0)
    ring[1].connectTo(0, 2, 0)
    ring[2].connectRx(1, 0)
    ring[0].writeRemote(v)
    mid = torch.ones(n, device=dev)
    ring[1].readRemote_wait()
    ring[1].forward_buffer()
    ring[1].forward_add(mid)
    assert torch.equal(mid, v + 1)
    assert torch.equal(ring[2].readRemote(), v)


@pytest.mark.parametrize("n,topk", [(50, 0.1), (500000, 0.01)])
def test_comprex_write_flush_accumulate(world, n, topk):
    """test/comprex.cpp:73-120 and examples/comprEx.cpp: nothing is lost after flushRests."""
    dev = world.device
    cm = make(world, cx.Comprex, n, 3.0, True)
    for c in cm:
        c.setThreshold(cx.ThresholdTopK(topk))
        c.setCompressor(cx.CompressorIndexPairs())
    cm[0].connectTx(1, 1)
    cm[1].connectRx(0, 1)
    vals = alt_ramp(n, dev)
    acc = torch.zeros(n, device=dev)
    runs = 3
    for _ in range(runs):
        cm[0].writeRemote(vals)
        cm[1].readRemote_add(acc)
    assert not torch.equal(acc, runs * vals)            # something was held back ...
    held = cm[0].getRests()
    assert torch.equal(acc + held, runs * vals)          # ... and it sits in the residual
    cm[0].flushRests()
    cm[1].readRemote_add(acc)
    assert torch.equal(acc, runs * vals)
    assert float(cm[0].getRests().abs().sum()) == 0.0
    st = cm[0].stats()
    assert st["n"] == n and st["status"] == 0


def test_comprex_topk_fraction_and_threshold_readback(world):
    n, dev = 1 << 18, world.device
    cm = make(world, cx.Comprex, n, 1.0)
    thr = cx.ThresholdTopK(0.01)
    cm[0].setThreshold(thr)
    cm[0].connectTx(1, 0)
    cm[1].connectRx(0, 0)
    torch.manual_seed(0)
    v = torch.randn(n, device=dev)
    cm[0].writeRemote(v)
    out = cm[1].readRemote()
    frac = float((out != 0).float().mean())
    assert 0.002 <= frac <= 0.03   # the estimate uses the 10th largest of 1000 samples: about top-k
    t = cm[0].threshold.getThreshold()
    assert torch.equal(out, torch.where(v.abs() > t, v, torch.zeros_like(v)))
    assert cm[0].getSize() == n


def test_comprex_variants_and_rests_api(world):
    n, dev = 4000, world.device
    cm = make(world, cx.Comprex, n, 3.0)
    cm[0].setThreshold(cx.ThresholdConst(1.0))
    cm[0].connectTx(1, 0)
    cm[1].connectRx(0, 0)
    torch.manual_seed(1)
    v = torch.randn(n, device=dev)
    big = v.abs() > 1.0
    cm[0].writeRemote_NoResidual(v)                      # the remainder is dropped
    assert torch.equal(cm[1].readRemote(), torch.where(big, v, torch.zeros_like(v)))
    assert float(cm[0].getRests().abs().sum()) == 0.0
    cm[0].writeRemote_compressOnly(v)                    # everything non-zero travels
    assert torch.equal(cm[1].readRemote(), v)
    cm[0].writeRemote(v)
    cm[1].readRemote()
    rest = cm[0].getRests()
    assert torch.equal(rest, torch.where(big, torch.zeros_like(v), v))
    x = torch.ones(n, device=dev)
    cm[0].addRests(x)
    assert torch.equal(x, 1 + rest)
    sd = cm[0].state_dict()
    cm[0].resetRests()
    assert float(cm[0].getRests().abs().sum()) == 0.0
    cm[0].load_state_dict(sd)
    assert torch.equal(cm[0].getRests(), rest)
    cm[0].setRests(np.zeros(n, dtype=np.float32))
    assert float(cm[0].getRests().abs().sum()) == 0.0
    with pytest.raises(cx.ComprexError, match="without connecting"):
        cm[2].writeRemote(v)
    with pytest.raises(cx.ComprexError, match="without connecting"):
        cm[2].readRemote()


def test_comprex_forwarding_ring(world):
    """0 -> 1 -> 2: rank 1 passes the compressed bytes on unchanged (readRemote_forward, forward_add)."""
    n, dev = 30000, world.device
    cm = make(world, cx.Comprex, n, 3.0, True)
    for c in cm:
        c.setThreshold(cx.ThresholdTopK(0.05))
    cm[0].connectTx(1, 0)
    cm[1].connectTo(0, 2, 0)
    cm[2].connectRx(1, 0)
    v = torch.randn(n, device=dev)
    cm[0].writeRemote(v)
    mid = torch.empty(n, device=dev)
    cm[1].readRemote_forward(mid)
    end = cm[2].readRemote()
    assert torch.equal(mid, end) and 0 < int((end != 0).sum()) < n // 5
    cm[0].writeRemote(v)
    acc = torch.ones(n, device=dev)
    cm[1].readRemote_wait()
    cm[1].forward_buffer()
    cm[1].forward_add(acc)
    end2 = cm[2].readRemote()
    assert torch.equal(acc, 1 + end2)


@pytest.mark.parametrize("codec", ["none", "rle"])
def test_comprex_other_codecs(world, codec):
    n, dev = 3000, world.device
    cm = make(world, cx.Comprex, n, 3.0)
    for c in cm:
        c.setCompressor(cx.CompressorNone() if codec == "none" else cx.CompressorRLE())
        c.setThreshold(cx.ThresholdConst(0.8))
    cm[0].connectTx(1, 0)
    cm[1].connectRx(0, 0)
    torch.manual_seed(2)
    v = torch.randn(n, device=dev)
    cm[0].writeRemote(v)
    out = cm[1].readRemote()
    if codec == "none":
        assert torch.equal(out, v)                       # dense payload: data + rests, rests = 0
    else:
        assert torch.equal(out, torch.where(v.abs() >= 0.8, v, torch.zeros_like(v)))
    acc = torch.ones(n, device=dev)
    cm[0].writeRemote(v)
    cm[1].readRemote_add(acc)
    total = out.clone()
    cm[0].flushRests()
    cm[1].readRemote_add(acc)
    assert torch.allclose(acc, 1 + 2 * v - total, atol=1e-6)


def test_fastcomprex_is_one_step_stale_and_conserves(world):
    n, dev = 20000, world.device
    fc = make(world, cx.FastComprex, n, 3.0)
    for c in fc:
        c.setThreshold(cx.ThresholdTopK(0.05))
    fc[0].connectTx(1, 0)
    fc[1].connectRx(0, 0)
    vals = alt_ramp(n, dev)
    acc = torch.zeros(n, device=dev)
    fc[0].writeRemote(vals)
    first = fc[1].readRemote()
    assert float(first.abs().sum()) == 0.0               # the first message is empty
    runs = 4
    for _ in range(runs - 1):
        fc[0].writeRemote(vals)
        fc[1].readRemote_add(acc)
    fc[0].flushRests()                                   # pending payload + residual
    fc[1].readRemote_add(acc)
    assert torch.equal(acc, runs * vals)
    # writeRemote_sameAs: a second engine sends the bytes the first one compressed
    a, b = make(world, cx.FastComprex, n, 3.0), make(world, cx.FastComprex, n, 3.0)
    for c in a + b:
        c.setThreshold(cx.ThresholdTopK(0.05))
    a[0].connectTx(1, 0)
    b[0].connectTx_sameBufferAs(2, 1, a[0])
    a[1].connectRx(0, 0)
    b[2].connectRx(0, 1)
    for _ in range(3):
        a[0].writeRemote(vals)
        b[0].writeRemote_sameAs(a[0])
        ra, rb = a[1].readRemote(), b[2].readRemote()
        assert torch.equal(ra, rb)
    assert float(ra.abs().sum()) > 0
