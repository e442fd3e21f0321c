"""The allocation-free compress entry point against the regular one.

Some users of the native library cannot allocate device memory at the point
where they call it, for instance a plug-in that runs inside a runtime which
has claimed the whole GPU for its own pool.  ``cx_compress_noalloc`` serves
them: it keeps its scratch in a static device array.  This test calls it
through its exported C symbol, twice in a row on evolving state, and expects
exactly what ``cx_compress`` with a caller-provided scratch buffer produces.
It lives in a file that sorts last so that a run stopping at the first failure
has already run everything else.
"""
import ctypes as C

import pytest
import torch

import comprex_b200 as cx
from comprex_b200 import _lib
from comprex_b200.ops import primitives as P


def _canonical(env, slot):
    """Header plus the stored pairs sorted by index, and the per-sub-tile counts."""
    ep = slot.endpoint(env)
    hdr = env.read_header(ep.hdr)
    pairs = torch.frombuffer(bytearray(env.read_bytes(ep.pairs, 8 * slot.cap)), dtype=torch.int32).view(-1, 2)
    nsub = (hdr.n + _lib.SUBTILE - 1) // _lib.SUBTILE
    table = torch.frombuffer(bytearray(env.read_bytes(ep.table, 8 * nsub)), dtype=torch.int32).view(-1, 2)
    parts = [pairs[int(s):int(s) + int(c)] for s, c in table.tolist()]
    got = torch.cat(parts) if parts else torch.zeros(0, 2, dtype=torch.int32)
    got = got[torch.argsort(got[:, 0])]
    return hdr, got[:, 0].clone(), got[:, 1].clone().view(torch.float32), table[:, 1].clone()


@pytest.mark.gpu
@pytest.mark.parametrize("n,dtype", [(300_001, torch.float32), (1 << 20, torch.bfloat16)])
def test_noalloc_entry_matches_regular_entry_twice(n, dtype):
    lib = _lib.load()
    fn = lib.cx_compress_noalloc          # the exported C symbol itself
    fn.restype = C.c_int
    fn.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_uint32, C.c_uint64,
                   C.POINTER(_lib.Targets), C.c_void_p, C.c_uint32, C.c_void_p]
    torch.manual_seed(11)
    env = cx.GaspiEnvironment(32 << 20, device="cuda")
    # warm-up as the header asks: an empty call sets the static array up on this device
    none = _lib.Targets()
    assert fn(_lib.F32, None, None, 0, torch.zeros(1, device="cuda").data_ptr(), 0, 0, C.byref(none), None, 0,
              torch.cuda.current_stream().cuda_stream) == 0, _lib.last_error()
    cap = n // 4
    slot_a, slot_b = P.SparseSlot.create(env, n, cap), P.SparseSlot.create(env, n, cap)
    comp = P.Compressor(env, n)                       # regular entry: scratch from the caller
    thr = torch.tensor([1.5], device="cuda")
    r_a = (0.4 * torch.randn(n, device="cuda"))
    r_b = r_a.clone()
    stream = torch.cuda.current_stream().cuda_stream
    for call in (1, 2):                               # two calls in a row, the residual carries over
        g = torch.randn(n, device="cuda").to(dtype)
        comp.thr.copy_(thr)
        comp.compress(g, r_a, n, cap, call, P.make_targets([slot_a.endpoint(env)]))
        tg = P.make_targets([slot_b.endpoint(env)])
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(_lib.dtype_code(dtype), g.data_ptr(), r_b.data_ptr(), n, thr.data_ptr(), cap, call,
                C.byref(tg), None, 0, stream)
        assert rc == 0, _lib.last_error()
        torch.cuda.synchronize()
        if call == 2:      # the property in the name: once set up, a call takes no device memory
            assert torch.cuda.mem_get_info()[0] == free_before
        env.flush()
        ha, ia, va, ca = _canonical(env, slot_a)
        hb, ib, vb, cb = _canonical(env, slot_b)
        assert hb.seq == call and hb.n == n and hb.kind == _lib.KIND_PAIRS
        assert ha.nnz == hb.nnz > 0 and ha.nnz_found == hb.nnz_found
        assert torch.equal(ia, ib) and torch.equal(ca, cb)
        torch.testing.assert_close(va, vb, rtol=0, atol=0)
        torch.testing.assert_close(r_a, r_b, rtol=0, atol=0)
    # sizes the static scratch cannot serve are refused with a message, nothing is launched
    tg = P.make_targets([slot_b.endpoint(env)])
    rc = fn(_lib.F32, r_a.data_ptr(), r_b.data_ptr(), 1 << 31, thr.data_ptr(), cap, 3, C.byref(tg), None, 0, stream)
    assert rc != 0 and "2^31-1" in _lib.last_error()
    env.close()
