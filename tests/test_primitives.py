"""Unit tests of the native primitives against plain PyTorch fp32 restatements.

Every test runs on the host implementation (CPU) and, marked ``gpu``, on the
CUDA kernels; the CUDA kernels are additionally compared bit for bit with the
host implementation of the same primitive.
"""
import ctypes as C

import pytest
import torch

import comprex_b200 as cx
from comprex_b200 import _lib
from comprex_b200.ops import primitives as P

from helpers import ref_compress, ref_threshold_topk

SIZES = [1, 31, 32, 33, 1023, 1024, 1025, 4095, 4096, 4097, 10007, 70001]


@pytest.fixture
def world(device):
    w = cx.LoopbackWorld(2, device=device, timeout_ms=200)
    yield w
    w.close()


def read_pairs(env, slot, rank=None):
    """Header, pairs in index order, and the per-sub-tile counts of a slot.

    Sub-tiles sit in the pair list in the order of their reservations; the table entry
    {start, count} of each sub-tile must address exactly its own pairs, each index once.
    """
    ep = slot.endpoint(env, rank)
    hdr = env.read_header(ep.hdr)
    raw = env.read_bytes(ep.pairs, 8 * slot.cap)    # the list may have gaps between its regions
    buf = torch.frombuffer(bytearray(raw), dtype=torch.int32).view(-1, 2)
    nsub = (hdr.n + _lib.SUBTILE - 1) // _lib.SUBTILE
    traw = env.read_bytes(ep.table, 8 * max(nsub, 1))[: 8 * nsub]
    table = torch.frombuffer(bytearray(traw), dtype=torch.int32).view(-1, 2).clone() if nsub else torch.zeros(0, 2, dtype=torch.int32)
    idx_parts, val_parts = [], []
    for s_ in range(nsub):
        start, count = int(table[s_, 0]), int(table[s_, 1])
        assert start + count <= slot.cap
        part = buf[start:start + count]
        i = part[:, 0]
        assert bool((i >= s_ * _lib.SUBTILE).all()) and bool((i < (s_ + 1) * _lib.SUBTILE).all())
        order = torch.argsort(i)                  # the order inside a sub-tile is not part of the format
        i = i[order]
        assert bool((i[1:] > i[:-1]).all())      # but every index occurs once
        idx_parts.append(i.clone())
        val_parts.append(part[:, 1][order].clone().view(torch.float32))
    idx = torch.cat(idx_parts) if idx_parts else torch.zeros(0, dtype=torch.int32)
    val = torch.cat(val_parts) if val_parts else torch.zeros(0)
    assert idx.numel() == hdr.nnz            # every stored pair belongs to exactly one sub-tile
    return hdr, idx, val, table[:, 1].clone()


@pytest.mark.parametrize("n", [1, 50, 999, 1000, 1001, 4096, 100003, 1 << 20])
@pytest.mark.parametrize("ratio", [0.1, 0.01, 0.001])
def test_threshold_matches_reference_rule(device, n, ratio):
    torch.manual_seed(n)
    env = cx.GaspiEnvironment(1 << 16, device=device)
    g = torch.randn(n).to(device)
    r = (0.5 * torch.randn(n)).to(device)
    comp = P.Compressor(env, n)
    comp.threshold_topk(g, r, n, ratio)
    got = comp.thr.item()
    want = ref_threshold_topk(r.cpu() + g.cpu(), ratio)
    assert got == want
    # sampling parameters of the ring variants
    comp.threshold_topk(g, None, n, ratio, 250, 4.0)
    assert comp.thr.item() == ref_threshold_topk(g.cpu(), ratio, 250, 4.0)
    env.close()


@pytest.mark.parametrize("n,ratio", [(999, 0.05), (30000, 0.01), (150001, 0.002)])
def test_exact_topk_threshold(device, n, ratio):
    """exact=True: the threshold is the ceil(n*ratio)-th largest magnitude of the whole vector
    (for n above the shared-memory key cache the kernel re-reads the vector in every pass)."""
    torch.manual_seed(n)
    env = cx.GaspiEnvironment(1 << 16, device=device)
    g, r = torch.randn(n).to(device), (0.3 * torch.randn(n)).to(device)
    thr = cx.ThresholdTopK(ratio, exact=True)
    thr.prepare_with(r, g)
    mags = (g + r).abs().cpu().sort(descending=True).values
    k = int(torch.ceil(torch.tensor(float(n) * ratio)).item())
    assert thr.getThreshold() == float(mags[k - 1])
    comp = P.Compressor(env, n)
    thr._launch(comp, g, r, n)
    assert comp.thr.item() == float(mags[k - 1])
    assert int(((g + r).abs() > comp.thr).sum()) == k - 1      # strict ">" of the pair codec
    env.close()


def test_threshold_reference_vector(device):
    """test/threshold.cpp:58-85: 100 ints, top 10 % -> threshold 90, 10 elements pass with >=."""
    from helpers import alt_ramp
    v = alt_ramp(100, device)
    thr = cx.ThresholdTopK(0.10)
    thr.prepare(v)
    assert thr.getThreshold() == 90.0
    kept = thr.apply(v)
    assert int((kept != 0).sum()) == 10
    const = cx.ThresholdConst(20)
    assert int((const.apply(v) != 0).sum()) == 80


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_compress_add_update(world, n, dtype):
    torch.manual_seed(n)
    e0, e1 = world.envs
    dev = world.device
    cap = n
    slot0 = P.SparseSlot.create(e0, n, cap)
    slot1 = P.SparseSlot.create(e1, n, cap)
    assert slot0.alloc == slot1.alloc
    g = torch.randn(n).to(dtype).to(dev)
    r0 = (0.3 * torch.randn(n)).to(dev)
    r = r0.clone()
    comp = P.Compressor(e0, n)
    comp.set_threshold(1.0)
    comp.compress(g, r, n, cap, 7, P.make_targets([slot1.endpoint(e0, 1), slot0.endpoint(e0, 0)]))
    e0.flush()
    idx_w, val_w, r_w = ref_compress(g.cpu(), r0.cpu(), 1.0)
    for env, slot in ((e1, slot1), (e0, slot0)):
        hdr, idx, val, prefix = read_pairs(env, slot)
        assert hdr.seq == 7 and hdr.n == n and hdr.kind == _lib.KIND_PAIRS
        assert hdr.nnz == idx_w.numel() == hdr.nnz_found
        assert torch.equal(idx, idx_w)           # the same set of survivors as the reference codec
        assert torch.equal(val, val_w)
        # counts[s] == number of survivors with index in [s*1024, (s+1)*1024)
        want = torch.bincount(idx_w.long() // _lib.SUBTILE, minlength=prefix.numel())
        assert torch.equal(prefix.long(), want)
    assert torch.equal(r.cpu(), r_w)
    # conservation: what was sent plus what stayed equals what came in
    dense = torch.zeros(n)
    dense[idx_w.long()] = val_w
    assert torch.equal(dense + r.cpu(), r0.cpu() + g.cpu().float())
    st = comp.last_stats()
    assert st["nnz"] == idx_w.numel() and st["status"] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1024, 4097, 70001, (1 << 20) + 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mode", ["add_update", "update", "plain"])
def test_compress_bulk_copy_kernel_matches_register_kernel(monkeypatch, n, dtype, mode):
    """The opt-in compress kernel whose sub-tiles arrive through bulk copies into shared memory
    (cp.async.bulk + mbarrier, a pipeline per warp) selects the same survivors, writes the same
    table counts and leaves the same residual as the default kernel, for all three modes, on
    sizes with a partial last sub-tile, and with a slot that overflows."""
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    results = []
    for bulk in ("0", "1"):
        monkeypatch.setenv("COMPREX_COMPRESS_BULK", bulk)
        world = cx.LoopbackWorld(2, device="cuda", timeout_ms=2000)
        e0, e1 = world.envs
        gen = torch.Generator().manual_seed(n)
        g = torch.randn(n, generator=gen).to(dtype).cuda()
        r = (0.3 * torch.randn(n, generator=gen)).cuda()
        out = []

        def run(cap, rr, seq, slot, comp):
            tg = P.make_targets([slot.endpoint(e0, 1)])
            if mode == "add_update":
                comp.compress(g, rr, n, cap, seq, tg)
            elif mode == "update":
                comp.compress(None, rr, n, cap, seq, tg)
            else:
                comp.compress(g, None, n, cap, seq, tg)
            e0.flush()
            hdr, idx, val, counts = read_pairs(e1, slot)
            return hdr, idx, val, counts, comp.last_stats()

        P.SparseSlot.create(e0, n, n)                 # allocations are symmetric across the ranks
        slot = P.SparseSlot.create(e1, n, n)
        comp = P.Compressor(e0, n)
        comp.set_threshold(1.0)
        for seq in (1, 2):
            hdr, idx, val, counts, st = run(n, r, seq, slot, comp)
            assert hdr.nnz == hdr.nnz_found and st["status"] == 0
            out.append((hdr.nnz, idx, val, counts, r.cpu().clone()))
            r.add_(0.5)                               # something to send in the second round
        # a slot that overflows: which sub-tiles find room is a matter of timing, the totals are not
        cap = max(n // 64, 8)
        P.SparseSlot.create(e0, n, cap)
        slot = P.SparseSlot.create(e1, n, cap)
        hdr, idx, val, counts, st = run(cap, r.clone(), 1, slot, comp)
        assert hdr.nnz < hdr.nnz_found and st["status"] & _lib.ST_OVERFLOW
        out.append((hdr.nnz, hdr.nnz_found))
        results.append(out)
        world.close()
    for a, b in zip(*results):
        assert len(a) == len(b)
        for x, y in zip(a, b):
            assert torch.equal(x, y) if isinstance(x, torch.Tensor) else x == y


def test_compress_capacity_overflow_keeps_residual(world):
    e0, e1 = world.envs
    dev, n, cap = world.device, 20000, 100
    slot = [P.SparseSlot.create(e, n, cap) for e in world.envs][1]
    g = torch.randn(n).to(dev)
    r = torch.zeros(n, device=dev)
    comp = P.Compressor(e0, n)
    comp.set_threshold(0.5)
    comp.compress(g, r, n, cap, 1, P.make_targets([slot.endpoint(e0, 1)]))
    hdr, idx, val, _ = read_pairs(e1, slot)
    assert hdr.nnz == cap and hdr.nnz_found == int((g.abs() > 0.5).sum())
    # which survivors made it depends on the order of the reservations; whatever was
    # emitted passed the threshold and left the residual, everything else stayed in it
    sent = torch.zeros(n)
    sent[idx.long()] = val
    assert bool((val.abs() > 0.5).all()) and idx.unique().numel() == cap
    assert torch.equal(sent + r.cpu(), g.cpu())
    assert float((r.cpu()[idx.long()]).abs().sum()) == 0.0
    assert comp.last_stats()["status"] & _lib.ST_OVERFLOW
    e0.check()  # overflow is soft: no exception


@pytest.mark.parametrize("mode", ["update", "plain"])
def test_compress_modes(world, mode):
    e0, e1 = world.envs
    dev, n = world.device, 5000
    slot = [P.SparseSlot.create(e, n, n) for e in world.envs][1]
    x = torch.randn(n).to(dev)
    x[::3] = 0
    comp = P.Compressor(e0, n)
    comp.set_threshold(0.0)
    if mode == "update":   # flushRests: everything non-zero leaves, the residual ends up zero
        r = x.clone()
        comp.compress(None, r, n, n, 1, P.make_targets([slot.endpoint(e0, 1)]))
        assert int(r.abs().sum().item()) == 0
    else:                  # compressOnly: the input is untouched
        comp.compress(x, None, n, n, 1, P.make_targets([slot.endpoint(e0, 1)]))
    hdr, idx, val, _ = read_pairs(e1, slot)
    nz = torch.nonzero(x.cpu()).flatten()
    assert torch.equal(idx.long(), nz) and torch.equal(val, x.cpu()[nz])


def _fill_slots(world, n, nsrc, seed=0):
    """Each virtual rank j < nsrc compresses its own vector into rank 0's slot j."""
    torch.manual_seed(seed)
    dev = world.device
    e0 = world.envs[0]
    slots = [[P.SparseSlot.create(e, n, n) for e in world.envs] for _ in range(nsrc)]
    dense = []
    for j in range(nsrc):
        x = torch.randn(n)
        x[torch.rand(n) > 0.2] = 0
        dense.append(x)
        comp = P.Compressor(e0, n)
        comp.set_threshold(0.0)
        comp.compress(x.to(dev), None, n, n, 3, P.make_targets([slots[j][0].endpoint(e0, 0)]))
    src = P.make_sources([slots[j][0].endpoint(e0, 0) for j in range(nsrc)], [3] * nsrc)
    return src, dense


@pytest.mark.parametrize("n", [1, 1000, 1024, 4097, 50001])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_apply_add_and_set(world, n, out_dtype):
    e0 = world.envs[0]
    dev = world.device
    src, dense = _fill_slots(world, n, 3)
    st = e0.new_status("t")
    base = torch.randn(n).to(out_dtype)
    out = base.clone().to(dev)
    P.apply_sparse(e0, src, n, P.args_add(out, 0.5), st)
    want = base.clone()
    for d in dense:   # same order, same rounding as the kernel: one source after the other
        want = (want.float() + 0.5 * d).to(out_dtype)
    assert torch.equal(out.cpu(), want)
    out2 = torch.full((n,), 7.0, dtype=out_dtype, device=dev)
    P.apply_sparse(e0, src, n, P.args_set(out2, 0.25), st)
    acc = torch.zeros(n)
    for d in dense:
        acc += d
    assert torch.equal(out2.cpu(), (0.25 * acc).to(out_dtype))
    e0.flush()
    assert st.value == 0


@pytest.mark.parametrize("op", ["sgd", "sgd_wd", "momentum", "adamw"])
@pytest.mark.parametrize("shadow", [False, True])
def test_apply_fused_updates(world, op, shadow):
    e0 = world.envs[0]
    dev, n = world.device, 30011
    src, dense = _fill_slots(world, n, 4, seed=5)
    g = torch.zeros(n)
    for d in dense:
        g += d
    g *= 0.25
    w0, m0, v0 = torch.randn(n), 0.1 * torch.randn(n), 0.01 * torch.rand(n) + 0.01
    w, m, v = w0.clone().to(dev), m0.clone().to(dev), v0.clone().to(dev)
    sh = w0.to(torch.bfloat16).to(dev) if shadow else None  # the shadow starts in sync, as in real use
    st = e0.new_status("t")
    lr, mu, wd, b1, b2, eps, step = 0.1, 0.9, 0.01, 0.9, 0.999, 1e-8, 3
    if op == "sgd":
        args = P.args_update(_lib.OP_SGD, w, 0.25, shadow=sh)
        want_w = w0 - g
    elif op == "sgd_wd":
        args = P.args_update(_lib.OP_SGD, w, 0.25, shadow=sh, wd=wd)
        want_w = (1 - wd) * w0 - g
    elif op == "momentum":
        args = P.args_update(_lib.OP_MOMENTUM, w, 0.25, shadow=sh, m=m, lr=lr, momentum=mu, wd=wd)
        want_m = mu * m0 + lr * g
        want_w = (1 - wd) * w0 - want_m
    else:
        args = P.args_update(_lib.OP_ADAMW, w, 0.25, shadow=sh, m=m, v=v, lr=lr, beta1=b1, beta2=b2, eps=eps,
                             wd=wd, step=step)
        want_m = b1 * m0 + (1 - b1) * g
        want_v = b2 * v0 + (1 - b2) * g * g
        want_w = w0 * (1 - lr * wd) - lr * (want_m / (1 - b1 ** step)) / ((want_v / (1 - b2 ** step)).sqrt() + eps)
    P.apply_sparse(e0, src, n, args, st)
    e0.flush()
    assert st.value == 0
    torch.testing.assert_close(w.cpu(), want_w, rtol=1e-5, atol=1e-6)
    if op in ("momentum", "adamw"):
        torch.testing.assert_close(m.cpu(), want_m, rtol=1e-5, atol=1e-7)
    if op == "adamw":
        torch.testing.assert_close(v.cpu(), want_v, rtol=1e-5, atol=1e-8)
    if shadow:
        assert torch.equal(sh.cpu(), w.cpu().to(torch.bfloat16))


@pytest.mark.gpu
@pytest.mark.parametrize("stages", ["1", "2"])
@pytest.mark.parametrize("op", ["sgd_wd", "momentum", "adamw"])
@pytest.mark.parametrize("n", [1024, 30011, (1 << 20) + 77])
def test_apply_bulk_copy_kernel_matches_register_kernel(monkeypatch, n, op, stages):
    """The opt-in dense update that stages w / m / v through shared memory with bulk copies
    (cp.async.bulk + mbarrier) gives the bits of the default kernel."""
    results = []
    for bulk in ("0", "1"):
        monkeypatch.setenv("COMPREX_APPLY_BULK", bulk)
        monkeypatch.setenv("COMPREX_APPLY_STAGES", stages)
        world = cx.LoopbackWorld(2, device="cuda", timeout_ms=2000)
        e0 = world.envs[0]
        src, _ = _fill_slots(world, n, 5, seed=9)
        g = torch.Generator().manual_seed(n)
        w = torch.randn(n, generator=g).cuda()
        m = (0.1 * torch.randn(n, generator=g)).cuda()
        v = (0.01 * torch.rand(n, generator=g) + 0.01).cuda()
        sh = w.to(torch.bfloat16)
        st = e0.new_status("t")
        code = {"sgd_wd": _lib.OP_SGD, "momentum": _lib.OP_MOMENTUM, "adamw": _lib.OP_ADAMW}[op]
        args = P.args_update(code, w, 0.2, shadow=sh, m=None if op == "sgd_wd" else m, v=v if op == "adamw" else None,
                             lr=0.05, momentum=0.9, wd=0.01, step=4)
        for _ in range(2):
            P.apply_sparse(e0, src, n, args, st)
        e0.flush()
        assert st.value == 0
        results.append((w.cpu(), m.cpu(), v.cpu(), sh.cpu()))
        world.close()
    for a, b in zip(*results):
        assert torch.equal(a, b)


@pytest.mark.parametrize("graph", [False, True])
def test_recorded_sequence_with_lanes_and_graph(world, graph):
    """Six independent threshold + compress pairs on side-stream lanes, joined by one apply:
    recorded once, replayed three times (as an op list, and on a GPU as a CUDA graph whose
    kernels take the sequence number from a device cell); equals the direct launches."""
    from comprex_b200.allreduce import _OpSeq
    e0, e1 = world.envs
    dev, nchunk, k = world.device, 3000, 6
    torch.manual_seed(11)
    g = torch.randn(k * nchunk).to(dev)
    slots = [[P.SparseSlot.create(e, nchunk, nchunk) for e in world.envs] for _ in range(k)]
    comps = [P.Compressor(e0, nchunk) for _ in range(k)]
    outs = [torch.zeros(nchunk, device=dev) for _ in range(k)]
    rests = [torch.zeros(k * nchunk, device=dev) for _ in range(2)]
    st = e1.new_status("t")

    def launches(r, seq):
        for c in range(k):
            view, rv = g[c * nchunk:(c + 1) * nchunk], r[c * nchunk:(c + 1) * nchunk]
            with P.lane(e0, c + 1):
                comps[c].threshold_topk(view, rv, nchunk, 0.05)
                comps[c].compress(view, rv, nchunk, nchunk, seq, P.make_targets([slots[c][1].endpoint(e0, 1)]))
        for c in range(k):
            with P.lane(e0, c + 1):
                P.apply_sparse(e0, P.make_sources([slots[c][1].endpoint(e0, 1)], [seq]), nchunk,
                               P.args_add(outs[c]), st)

    e0._rec = rec = []
    try:
        launches(rests[0], 0)
    finally:
        e0._rec = None
    assert len(rec) == 3 * k and {op.lane for op in rec} == set(range(1, k + 1))
    seq_obj = _OpSeq(e0, rec, graph=graph)
    assert (seq_obj.graph is not None) == (graph and e0.dev == _lib.DEV_CUDA)
    for step in (1, 2, 3):
        seq_obj.run(step)
    e0.flush()
    got = torch.cat(outs).cpu()
    for o in outs:
        o.zero_()
    for step in (4, 5, 6):                      # the same launches issued directly
        launches(rests[1], step)
    e0.flush()
    assert st.value == 0
    assert torch.equal(torch.cat(outs).cpu(), got)
    assert torch.equal(rests[0].cpu(), rests[1].cpu())
    assert float(got.abs().sum()) > 0


def test_apply_timeout_sets_status_and_leaves_output(world):
    """A notification that never arrives: the wait gives up, the output is untouched."""
    e0 = world.envs[0]
    n = 2048
    slot = [P.SparseSlot.create(e, n, n) for e in world.envs][0]
    out = torch.ones(n, device=world.device)
    st = e0.new_status("waiter")
    P.apply_sparse(e0, P.make_sources([slot.endpoint(e0)], [1]), n, P.args_add(out), st)
    with pytest.raises(cx.ComprexError, match="TIMEOUT"):
        e0.flush()
    assert torch.equal(out.cpu(), torch.ones(n))
    e0.flush()  # the status word was cleared, the context is still usable
    comp = P.Compressor(e0, n)
    comp.set_threshold(0.0)
    comp.compress(out, None, n, n, 1, P.make_targets([slot.endpoint(e0)]))
    P.apply_sparse(e0, P.make_sources([slot.endpoint(e0)], [1]), n, P.args_add(out), st)
    e0.flush()
    assert torch.equal(out.cpu(), 2 * torch.ones(n))


def test_pushing_reduce_timeout_leaves_counters_clean(world):
    """A pushing reduce whose source never arrives reports TIMEOUT, publishes nothing and leaves
    the completion counters at zero, so that the same launch works when the sender is there."""
    e0, e1 = world.envs
    n = 5000
    src_slot = [P.DenseSlot.create(e, 4 * n) for e in world.envs][0]
    dst_slot = [P.DenseSlot.create(e, 4 * n) for e in world.envs][0]
    own = torch.ones(n, device=world.device)
    out = torch.zeros(n, device=world.device)
    st = e0.new_status("reducer")
    counters = e0.scratch(int(e0.lib.cx_sizeof(4)))
    push = P.make_targets([dst_slot.endpoint(e0, 1)])

    def reduce(seq):
        P.dense_reduce(e0, out, own, n, P.make_sources([src_slot.endpoint(e0)], [seq]), st, push=push,
                       push_seq=seq, counters=counters)
    reduce(1)
    with pytest.raises(cx.ComprexError, match="TIMEOUT"):
        e0.flush()
    assert int(counters.view(torch.int32)[:64].abs().sum()) == 0          # done and the failure mark
    assert e1.read_header(dst_slot.endpoint(e1).hdr).seq == 0             # nothing was published
    sender_counters = e1.scratch(int(e1.lib.cx_sizeof(4)))
    P.dense_send(e1, 2 * torch.ones(n, device=world.device), None, n, 1,
                 P.make_targets([src_slot.endpoint(e1, 0)]), sender_counters)
    e1.flush()
    reduce(1)
    e0.flush()
    assert torch.equal(out.cpu(), 3 * torch.ones(n))
    assert e1.read_header(dst_slot.endpoint(e1).hdr).seq == 1
    assert int(counters.view(torch.int32)[:64].abs().sum()) == 0


def test_apply_rejects_corrupt_header_and_index(world):
    """Host-written garbage in a local slot is reported, never dereferenced."""
    e0 = world.envs[0]
    n = 3000
    slot = [P.SparseSlot.create(e, n, n) for e in world.envs][0]
    x = torch.zeros(n, device=world.device)
    x[5] = 1.0
    comp = P.Compressor(e0, n)
    comp.set_threshold(0.0)
    comp.compress(x, None, n, n, 1, P.make_targets([slot.endpoint(e0)]))
    e0.flush()
    ep = slot.endpoint(e0)
    bad_pair = (C.c_int32 * 2)(2_000_000, 0x3F800000)
    if world.device.type == "cuda":
        _lib.check(e0.lib.cx_cuda_memcpy(ep.pairs, bad_pair, 8, 1, None))
        torch.cuda.synchronize()
    else:
        C.memmove(ep.pairs, bad_pair, 8)
    out = torch.zeros(n, device=world.device)
    st = e0.new_status("decoder")
    P.apply_sparse(e0, P.make_sources([ep], [1]), n, P.args_add(out), st)
    with pytest.raises(cx.ComprexError, match="BAD_INDEX"):
        e0.flush()
    assert float(out.abs().sum()) == 0.0
    # wrong length in the header
    P.apply_sparse(e0, P.make_sources([ep], [1]), n + 1, P.args_add(torch.zeros(n + 1, device=world.device)), st)
    with pytest.raises(cx.ComprexError, match="BAD_HEADER"):
        e0.flush()


@pytest.mark.parametrize("n", [1, 5, 1000, 4099, 65537])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_dense_send_reduce(world, n, dtype):
    e0, e1 = world.envs
    dev = world.device
    es = torch.empty(0, dtype=dtype).element_size()
    slots = [[P.DenseSlot.create(e, n * es) for e in world.envs] for _ in range(2)]
    ctr = e0.scratch(64)
    a, b = torch.randn(n).to(dtype), torch.randn(n).to(dtype)
    own = torch.randn(n).to(dtype)
    P.dense_send(e0, a.to(dev), None, n, 1, P.make_targets([slots[0][1].endpoint(e0, 1)]), ctr)
    P.dense_send(e0, b.to(dev), None, n, 1, P.make_targets([slots[1][1].endpoint(e0, 1)]), ctr)
    st = e1.new_status("t")
    out = own.clone().to(dev)
    src = P.make_sources([slots[0][1].endpoint(e1), slots[1][1].endpoint(e1)], [1, 1])
    P.dense_reduce(e1, out, out, n, src, st, scale=0.5)
    want = ((own.float() + a.float() + b.float()) * 0.5).to(dtype)
    assert torch.equal(out.cpu(), want)
    cp = torch.empty(n, dtype=dtype, device=dev)
    P.dense_reduce(e1, cp, None, n, P.make_sources([slots[0][1].endpoint(e1)], [1]), st)
    assert torch.equal(cp.cpu(), a)
    e1.flush()


def test_dense_send_with_residual_is_compressor_none(world):
    e0, e1 = world.envs
    dev, n = world.device, 3001
    slot = [P.DenseSlot.create(e, 4 * n) for e in world.envs][1]
    g, r0 = torch.randn(n), torch.randn(n)
    r = r0.clone().to(dev)
    P.dense_send(e0, g.to(dev), r, n, 1, P.make_targets([slot.endpoint(e0, 1)]), e0.scratch(64))
    out = torch.empty(n, device=dev)
    P.dense_reduce(e1, out, None, n, P.make_sources([slot.endpoint(e1)], [1]), e1.new_status("t"))
    assert torch.equal(out.cpu(), g + r0)
    assert float(r.abs().sum()) == 0.0


def test_rle_roundtrip_and_residual():
    """Corrected RLE codec: round trip with a threshold above zero, plus error feedback."""
    torch.manual_seed(1)
    n = 1000
    g, r0 = torch.randn(n), 0.2 * torch.randn(n)
    r = r0.clone()
    payload = cx.CompressorRLE.encode(g, r, 1.0)
    v = g + r0
    keep = v.abs() >= 1.0
    out = torch.full((n,), 9.0)
    cx.CompressorRLE.decode(payload, out)
    assert torch.equal(out, torch.where(keep, v, torch.zeros(n)))
    assert torch.equal(r, torch.where(keep, torch.zeros(n), v))
    acc = torch.ones(n)
    cx.CompressorRLE.decode(payload, acc, add=True)
    assert torch.equal(acc, 1 + torch.where(keep, v, torch.zeros(n)))
    # the sparse test vector of test/compressor.cpp (75 % zeros, threshold 0)
    x = torch.arange(16).float() * (torch.arange(16) % 4 == 0)
    out = torch.empty(16)
    cx.CompressorRLE.decode(cx.CompressorRLE.encode(x, None, 0.0), out)
    assert torch.equal(out, x)


@pytest.mark.parametrize("n", [1, 7, 2047, 2048, 2049, 4096, 10007, 70001])
@pytest.mark.parametrize("thr,density", [(0.0, 0.25), (0.8, 1.0), (3.5, 1.0), (100.0, 1.0)])
def test_rle_fused_codec_matches_host_bytes(world, n, thr, density):
    """Fused RLE send/receive (kernels on a GPU, host twin on the CPU): the bytes that land in
    the receiver's slot equal the host codec's payload, the expansion equals the plain
    restatement, the residual keeps what was not sent, and `add` accumulates."""
    e0, e1 = world.envs
    codecs = [P.RleCodec(e, n) for e in world.envs]
    torch.manual_seed(n)
    g = torch.randn(n) * (torch.rand(n) < density)
    r0 = 0.3 * torch.randn(n) * (torch.rand(n) < density)
    cell = torch.full((1,), thr, dtype=torch.float32, device=e0.device)
    gd, r = g.to(e0.device), r0.clone().to(e0.device)
    codecs[0].send(gd, r, cell, 1, 1)
    status = e1.new_status("t")
    out = torch.full((n,), 9.0, device=e1.device)
    codecs[1].recv(out, 1, False, status)
    e1.flush()
    assert status.value == 0
    v = g + r0
    keep = (v.abs() >= thr) & ~((thr == 0.0) & (v == 0))
    assert torch.equal(out.cpu(), torch.where(keep, v, torch.zeros(n)))
    assert torch.equal(r.cpu(), torch.where(keep, torch.zeros(n), v))
    rh = r0.clone()
    expect = cx.CompressorRLE.encode(g, rh, thr)
    ep = codecs[1].slots[1].endpoint(e1)
    hdr = e1.read_header(ep.hdr)
    assert (hdr.kind, hdr.n, hdr.bytes, hdr.nnz) == (_lib.KIND_RLE, n, len(expect), int(keep.sum()))
    assert e1.read_bytes(ep.pairs, len(expect)) == expect
    # second payload (other parity) accumulated on top
    codecs[0].send(None, r, cell.zero_(), 2, 1)            # flush of the residual at threshold 0
    acc = torch.ones(n, device=e1.device)
    codecs[1].recv(acc, 2, True, status)
    e1.flush()
    assert status.value == 0
    assert torch.equal(acc.cpu(), 1 + torch.where(keep, torch.zeros(n), v))
    assert float(r.abs().sum()) == 0.0


def test_rle_fused_receive_rejects_corrupt_runs(world):
    """Host-side fault injection: run lengths that do not add up to n set BAD_HEADER and leave
    the output untouched; a payload that never arrives times out with a status."""
    e0, e1 = world.envs
    n = 5000
    codecs = [P.RleCodec(e, n) for e in world.envs]
    g = torch.randn(n, generator=torch.Generator().manual_seed(0))
    cell = torch.full((1,), 1.0, dtype=torch.float32, device=e0.device)
    codecs[0].send(g.to(e0.device), None, cell, 1, 1)
    e0.flush()
    ep = codecs[1].slots[1].endpoint(e1)
    hdr = e1.read_header(ep.hdr)
    raw = bytearray(e1.read_bytes(ep.pairs, hdr.bytes))
    runs_at = 16 + 4 * hdr.nnz
    first = int.from_bytes(raw[runs_at:runs_at + 4], "little")
    raw[runs_at:runs_at + 4] = (first + 1).to_bytes(4, "little")       # one element too many
    t = torch.frombuffer(raw, dtype=torch.uint8)
    if e1.dev == _lib.DEV_CUDA:
        _lib.check(e1.lib.cx_cuda_memcpy(ep.pairs, t.data_ptr(), len(raw), 1, None), "memcpy")
    else:
        C.memmove(ep.pairs, t.data_ptr(), len(raw))
    status = e1.new_status("t")
    out = torch.full((n,), 9.0, device=e1.device)
    codecs[1].recv(out, 1, False, status)
    with pytest.raises(cx.ComprexError, match="BAD_HEADER"):
        e1.flush()
    assert torch.equal(out.cpu(), torch.full((n,), 9.0))
    status2 = e1.new_status("t2")
    codecs[1].recv(out, 2, False, status2)                 # nobody sent payload 2
    with pytest.raises(cx.ComprexError, match="TIMEOUT"):
        e1.flush()
    assert torch.equal(out.cpu(), torch.full((n,), 9.0))


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1000, 4096, 100003, (1 << 22) + 5])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_cuda_kernels_match_host_bitwise(n, dtype):
    """threshold + compress + apply on the GPU produce the bits of the host implementation
    (the AdamW weights to within the hardware's approximate square root and reciprocal)."""
    torch.manual_seed(n)
    g = torch.randn(n).to(dtype)
    r0 = 0.7 * torch.randn(n)
    w0 = torch.randn(n)
    res = {}
    for dev in ("cpu", "cuda"):
        world = cx.LoopbackWorld(2, device=dev)
        e0, e1 = world.envs
        cap = n // 8
        slot = [P.SparseSlot.create(e, n, cap) for e in world.envs][1]
        comp = P.Compressor(e0, n)
        r = r0.clone().to(dev)
        comp.threshold_topk(g.to(dev), r, n, 0.02)
        comp.compress(g.to(dev), r, n, cap, 1, P.make_targets([slot.endpoint(e0, 1)]))
        hdr, idx, val, prefix = read_pairs(e1, slot)
        w = w0.clone().to(dev)
        m = torch.zeros(n, device=dev)
        v = torch.zeros(n, device=dev)
        sh = torch.zeros(n, dtype=torch.bfloat16, device=dev)
        st = e1.new_status("t")
        P.apply_sparse(e1, P.make_sources([slot.endpoint(e1)], [1]), n,
                       P.args_update(_lib.OP_ADAMW, w, 0.5, shadow=sh, m=m, v=v, lr=0.01, wd=0.1, step=2), st)
        e1.flush()
        res[dev] = (comp.thr.cpu().clone(), idx, val, prefix, r.cpu(), w.cpu(), m.cpu(), v.cpu(), sh.cpu())
        world.close()
    names = ["thr", "idx", "val", "prefix", "r", "w", "m", "v", "shadow"]
    for name, a, b in zip(names, res["cpu"], res["cuda"]):
        if name == "w":        # the kernel's AdamW step uses the approximate sqrt / reciprocal units
            torch.testing.assert_close(b, a, rtol=1e-6, atol=1e-6)
        elif name == "shadow":
            torch.testing.assert_close(b.float(), a.float(), rtol=1e-2, atol=1e-7)
        else:
            assert torch.equal(a, b), name
