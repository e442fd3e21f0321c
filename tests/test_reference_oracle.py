"""The native primitives against the reference's own code.

When ``COMPREX_REFERENCE`` names the root of the reference's source tree, ``reference_oracle.cpp``
is compiled against its header-only ``src/threshold.hxx`` / ``src/compressor.hxx`` (unmodified) and
the host back end must reproduce, bit for bit, the threshold of ``ThresholdTopK::prepare_with``, the
(index, value) pairs of ``CompressorIndexPairs::compress_add_update``, the residual it leaves, and the
results of ``::add`` (scatter-add) and ``::decompress``.
(The CUDA kernels are tied to the host back end bit for bit by test_primitives.py.)  Without the
variable the tests are skipped."""
import os
import struct
import subprocess

import numpy as np
import pytest
import torch

import comprex_b200 as cx
from comprex_b200.ops import primitives as P

from test_primitives import read_pairs

REF = os.environ.get("COMPREX_REFERENCE")
pytestmark = pytest.mark.skipif(not REF or not os.path.exists(os.path.join(REF or "", "src", "compressor.hxx")),
                                reason="COMPREX_REFERENCE does not point at the reference's tree")


@pytest.fixture(scope="module")
def oracle(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("oracle") / "reference_oracle")
    src = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_oracle.cpp")
    subprocess.run([os.environ.get("CXX", "g++"), "-O2", "-std=c++14", "-fpermissive", "-w", "-ffp-contract=off",
                    "-I", os.path.join(REF, "src"), src, "-o", exe], check=True)
    return exe


@pytest.mark.parametrize("mode", [0, 1, 2], ids=["add_update", "update", "compress"])
@pytest.mark.parametrize("n", [50, 999, 1000, 4097, 100003, 1 << 20])
@pytest.mark.parametrize("ratio", [0.1, 0.01, 0.001])
def test_threshold_pairs_and_residual_match_the_reference(oracle, tmp_path, n, ratio, mode):
    torch.manual_seed(n)
    g, r0, base = torch.randn(n), 0.5 * torch.randn(n), torch.randn(n)
    fin, fout = str(tmp_path / "in.bin"), str(tmp_path / "out.bin")
    with open(fin, "wb") as f:
        f.write(struct.pack("<if", n, ratio))
        f.write(g.numpy().tobytes())
        f.write(r0.numpy().tobytes())
        f.write(base.numpy().tobytes())
    subprocess.run([oracle, fin, fout, str(mode)], check=True)
    raw = open(fout, "rb").read()
    ref_thr = np.frombuffer(raw, dtype=np.float32, count=1)[0]
    nbytes = struct.unpack_from("<i", raw, 4)[0]
    payload = raw[8:8 + nbytes]
    ref_n, ref_nnz = struct.unpack_from("<ii", payload, 0)
    pairs = np.frombuffer(payload, dtype=np.int32, offset=8).reshape(-1, 2)
    ref_idx = torch.from_numpy(pairs[:, 0].copy())
    ref_val = torch.from_numpy(pairs[:, 1].copy().view(np.float32))
    tail = torch.from_numpy(np.frombuffer(raw, dtype=np.float32, offset=8 + nbytes).copy())
    ref_r, ref_add, ref_dec = tail[:n], tail[n:2 * n], tail[2 * n:3 * n]
    assert ref_n == n and ref_nnz == ref_idx.numel()

    world = cx.LoopbackWorld(2, device="cpu", timeout_ms=200)
    e0, e1 = world.envs
    slot = [P.SparseSlot.create(e, n, n) for e in world.envs][1]
    comp = P.Compressor(e0, n)
    r = r0.clone()
    g_arg, r_arg = (g, r) if mode == 0 else ((None, r) if mode == 1 else (g, None))
    comp.threshold_topk(g_arg, r_arg, n, ratio)
    assert comp.thr.numpy().view(np.uint32)[0] == np.float32(ref_thr).view(np.uint32)      # same bits
    comp.compress(g_arg, r_arg, n, n, 1, P.make_targets([slot.endpoint(e0, 1)]))
    hdr, idx, val, _ = read_pairs(e1, slot)
    assert hdr.nnz == ref_nnz
    assert torch.equal(idx.to(torch.int32), ref_idx) and torch.equal(val, ref_val)
    assert torch.equal(r, ref_r)
    status = e1.new_status("oracle")
    src = P.make_sources([slot.endpoint(e1)], [1])
    acc = base.clone()
    P.apply_sparse(e1, src, n, P.args_add(acc), status)
    assert torch.equal(acc, ref_add)
    dec = torch.full((n,), 7.0)
    P.apply_sparse(e1, src, n, P.args_set(dec), status)
    assert torch.equal(dec, ref_dec) and status.value == 0
    world.close()


@pytest.mark.parametrize("n", [100, 4097, 100003])
@pytest.mark.parametrize("ratio", [0.1, 0.01])
def test_threshold_apply_and_split_match_the_reference(oracle, tmp_path, n, ratio):
    torch.manual_seed(n + 1)
    g = torch.randn(n)
    fin, fout = str(tmp_path / "in.bin"), str(tmp_path / "out.bin")
    with open(fin, "wb") as f:
        f.write(struct.pack("<if", n, ratio))
        f.write(g.numpy().tobytes() * 3)               # g, r, base slots of the file format
    subprocess.run([oracle, fin, fout, "3"], check=True)
    ref = torch.from_numpy(np.fromfile(fout, dtype=np.float32))
    ref_out, ref_hi, ref_lo = ref[:n], ref[n:2 * n], ref[2 * n:]
    thr = cx.ThresholdTopK(ratio)
    assert torch.equal(thr.apply(g), ref_out)
    hi, lo = cx.ThresholdTopK(ratio).apply_split(g)
    assert torch.equal(hi, ref_hi) and torch.equal(lo, ref_lo)
