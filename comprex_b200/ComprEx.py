"""Compressed point-to-point exchange with local error accumulation
(reference: include/comprEx.hxx:22-227, src/comprEx.tpp:32-514, Python face
ComprEx.py:100-199; thresholds src/threshold.hxx, codecs src/compressor.hxx).

``Comprex.writeRemote(v)`` is two launches on the caller's stream:

1. the threshold kernel estimates the magnitude cut of ``rests + v`` with the
   reference's sampling rule (bit-exact) and leaves it in device memory;
2. the compress kernel does ``rests += v``, selects ``|rests| > thr``, stores
   the (index, value) pairs, grouped by 1024-element sub-tile, directly into the
   destination rank's receive slot over NVLink, zeroes what it sent and
   publishes the sequence number.

``readRemote*`` is one launch that waits (bounded) and scatters.  The
residual ("rests") is an ordinary ``float32`` tensor owned by this object: it
can be read, set, and travels in ``state_dict()``.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from .common import AbstractExchange, Getable  # noqa: F401  (the reference defines Getable in this module too)
from ._lib import ComprexError
from .GaspiEx import to_device_vector, write_back
from .ops import primitives as P


# ---------------------------------------------------------------------------------
# Thresholds (src/threshold.hxx:16-242, ComprEx.py:158-178)
# ---------------------------------------------------------------------------------
class _Threshold:
    kind = "none"

    def __init__(self):
        self._threshold = 0.0

    def get(self):
        return self

    def clone(self):
        import copy
        return copy.copy(self)

    def getThreshold(self) -> float:
        return float(self._threshold)

    get_threshold = getThreshold

    def prepare(self, vec) -> None:
        """Compute the threshold for ``vec`` (no-op for fixed thresholds)."""

    def prepare_with(self, rests, add_vec) -> None:
        """Compute the threshold for ``rests + add_vec``."""

    def apply(self, vec: torch.Tensor) -> torch.Tensor:
        """Dense copy with everything below the threshold zeroed (``|x| >= thr`` stays).  Like the
        reference (src/threshold.hxx:19-27) the threshold is first prepared from ``vec`` itself."""
        self.prepare(vec)
        self._threshold = self.getThreshold()
        return torch.where(vec.abs() >= self._threshold, vec, torch.zeros_like(vec))

    def apply_split(self, vec: torch.Tensor):
        """(kept, rest): the part at or above the threshold and the remainder (prepared from ``vec``)."""
        self.prepare(vec)
        self._threshold = self.getThreshold()
        keep = vec.abs() >= self._threshold
        zero = torch.zeros_like(vec)
        return torch.where(keep, vec, zero), torch.where(keep, zero, vec)

    # used by the engines: leave the cut in the compressor's device cell
    def _launch(self, comp: P.Compressor, g, r, n: int) -> None:
        comp.set_threshold(self._threshold)


class ThresholdNone(_Threshold):
    """Everything passes (threshold 0); exact zeros are not transmitted."""
    kind = "none"


class ThresholdConst(_Threshold):
    kind = "const"

    def __init__(self, thresh: float):
        super().__init__()
        if thresh < 0:
            raise ComprexError("Threshold must be non-negative!")
        self._threshold = float(thresh)


class ThresholdTopK(_Threshold):
    """Adaptive threshold that lets about ``topK`` of the elements pass.

    The estimate uses the reference's strided sample: ``max(default_subsamples,
    subsample_factor / topK)`` elements, rank ``ceil(samples*topK)-1`` by
    magnitude, "send nothing" when that rank is <= 0 (src/threshold.hxx:182-205).
    """
    kind = "topk"

    EXACT = 2 ** 31 - 128      # "sample" larger than any vector: every element is looked at

    def __init__(self, topK: float, default_subsamples: int = 1000, subsample_factor: float = 10.0,
                 exact: bool = False):
        super().__init__()
        if topK > 1.0 or topK < 0.0:
            raise ComprexError("topK value must be between 0.0 and 1.0!")
        self.topK = float(topK)
        # exact=True: the threshold is the true ceil(n*topK)-th largest magnitude (a select over
        # the whole vector, several passes over it) instead of the reference's sampled estimate
        self.exact = bool(exact)
        if exact:
            default_subsamples = self.EXACT
        self.default_subsamples = int(default_subsamples)
        self.subsample_factor = float(subsample_factor)
        self._cell = None
        self._ws = None

    def getTopK(self) -> float:
        return self.topK

    def getThreshold(self) -> float:
        if self._cell is not None:
            self._threshold = float(self._cell.item())
        return float(self._threshold)

    get_threshold = getThreshold

    def _standalone(self, g, r) -> None:
        lib = _lib.load()
        ref = g if g is not None else r
        out = torch.zeros(1, dtype=torch.float32, device=ref.device)
        gd = _lib.dtype_code(g.dtype) if g is not None else _lib.F32
        ws_bytes = int(lib.cx_threshold_workspace_bytes()) if self.exact else 0
        if self.exact and (self._ws is None or self._ws.device != ref.device):
            self._ws = torch.zeros(ws_bytes, dtype=torch.uint8, device=ref.device)   # grid-wide exact selection
        _lib.check(lib.cx_threshold_select(_lib.dev_code(ref), gd, g.data_ptr() if g is not None else 0,
                                           r.data_ptr() if r is not None else 0, ref.numel(), self.topK,
                                           self.default_subsamples, self.subsample_factor, out.data_ptr(),
                                           self._ws.data_ptr() if self.exact else 0, ws_bytes,
                                           _lib.stream_ptr(ref.device)), "cx_threshold_select")
        self._cell = out

    def prepare(self, vec) -> None:
        self._standalone(vec.contiguous().view(-1), None)

    def prepare_with(self, rests, add_vec) -> None:
        if rests.numel() != add_vec.numel():
            raise ComprexError("vector sizes must be the same!")
        self._standalone(add_vec.contiguous().view(-1), rests.contiguous().view(-1))

    def _launch(self, comp: P.Compressor, g, r, n: int) -> None:
        comp.threshold_topk(g, r, n, self.topK, self.default_subsamples, self.subsample_factor)
        self._cell = comp.thr


# ---------------------------------------------------------------------------------
# Compressors (src/compressor.hxx:84-661, ComprEx.py:183-199)
# ---------------------------------------------------------------------------------
class _Compressor:
    kind = "pairs"

    def get(self):
        return self

    def clone(self):
        return type(self)()


class CompressorIndexPairs(_Compressor):
    """``int32 n | int32 nnz | nnz x (int32 index, value)``, ascending index, strict ``>``."""
    kind = "pairs"


class CompressorNone(_Compressor):
    """Dense payload: ``out = data + rests; rests = 0`` (src/compressor.hxx:93-105)."""
    kind = "none"


class CompressorRLE(_Compressor):
    """Run-length coded selection mask plus packed values.

    The byte layout follows the reference (``n | nnz | values | nRuns |
    firstIsYes | runs``) but values are stored at their packed position, which
    the reference's codec gets wrong for thresholds above zero.  Engines use the
    fused codec of ``csrc/rle.cu`` (count / scan / emit kernels that store the
    payload straight into the receiver's slot, bounded wait + run check + expand on
    the other side); ``encode`` / ``decode`` below are the host codec on byte strings,
    the oracle of the tests.
    """
    kind = "rle"

    @staticmethod
    def encode(vec: torch.Tensor, rests: torch.Tensor | None, thr: float) -> bytes:
        lib = _lib.load()
        g = vec.detach().to("cpu", torch.float32).contiguous() if vec is not None else None
        r = rests.detach().to("cpu", torch.float32).contiguous() if rests is not None else None
        n = (g if g is not None else r).numel()
        if n == 0:                                  # an empty tensor has no address to hand over
            return (0).to_bytes(4, "little") * 4    # n | nnz | nRuns | firstIsYes
        buf = (C.c_char * (16 + 8 * n + 16))()
        used = lib.cx_rle_compress_host(g.data_ptr() if g is not None else 0, r.data_ptr() if r is not None else 0,
                                        n, float(thr), buf, len(buf))
        if used < 0:
            raise ComprexError("RLE encode: " + _lib.last_error())
        if rests is not None:
            rests.copy_(r)
        return bytes(buf[:used])

    @staticmethod
    def decode(payload: bytes, out: torch.Tensor, add: bool = False) -> None:
        lib = _lib.load()
        o = out.detach().to("cpu", torch.float32).contiguous()
        _lib.check(lib.cx_rle_decode_host(payload, len(payload), o.data_ptr(), o.numel(), int(add)), "RLE decode")
        out.copy_(o)


# ---------------------------------------------------------------------------------
# ComprEx
# ---------------------------------------------------------------------------------
class Comprex(AbstractExchange):
    """Compressed exchange with residual; mirrors ``ComprEx<T>`` and its Python class.

    ``size_factor`` sizes the receive slot like the reference does
    (``size * sizeof(T) * size_factor`` bytes, src/comprEx.tpp:61); survivors
    that do not fit stay in the residual instead of overflowing the buffer.
    """

    def __init__(self, gaspi_env, size: int, size_factor: float = 1.0, send_sizeBytes: bool = False):
        self._env = env = gaspi_env.get()
        self.size = int(size)
        self.size_factor = float(size_factor)
        self.send_sizeBytes = bool(send_sizeBytes)
        self.cap = max(int(self.size * 4 * self.size_factor - 8) // 8, 1)
        self._slots = [P.SparseSlot.create(env, self.size, self.cap) for _ in range(self._nslots())]
        self._dense = None  # CompressorNone payloads, created on demand
        self._rle = None    # CompressorRLE slots and scratch, created on demand
        self._comp = P.Compressor(env, self.size)
        self._counters = env.scratch(64)
        self._status = env.new_status(type(self).__name__)
        self.threshold: _Threshold = ThresholdNone()
        self.compressor: _Compressor = CompressorIndexPairs()
        self.restsVect: torch.Tensor | None = None
        self._tx_seq: dict[int, int] = {}
        self._rx_seq: dict[int, int] = {}
        self._dest = None
        self._src = None
        self._rx_current = None
        self._held = None

    def _nslots(self) -> int:
        return 2

    # ---- strategy objects ---------------------------------------------------------------
    def setThreshold(self, threshold) -> None:
        self.threshold = threshold.get().clone()

    def setCompressor(self, compressor) -> None:
        comp = compressor.get().clone()
        if comp.kind == "none" and self._dense is None:
            from .GaspiEx import GaspiEx
            self._dense = GaspiEx(self._env, self.size)      # dense payloads travel through a dense slot
            if self._dest is not None:
                self._dense.connectTx(self._dest)
            if self._src is not None:
                self._dense.connectRx(self._src)
        if comp.kind == "rle" and self._rle is None:
            self._rle = P.RleCodec(self._env, self.size)     # worst-case sized slots (collective allocation)
        self.compressor = comp

    def getSize(self) -> int:
        return self.size

    # ---- residual -------------------------------------------------------------------------
    def _alloc_rests(self) -> None:
        self.restsVect = torch.zeros(self.size, dtype=torch.float32, device=self._env.device)

    def resetRests(self) -> None:
        if self.restsVect is not None:
            self.restsVect.zero_()

    def getRests(self) -> torch.Tensor:
        """Copy of the residual (zeros when there is no outgoing connection)."""
        if self.restsVect is None:
            return torch.zeros(self.size, dtype=torch.float32, device=self._env.device)
        return self.restsVect.clone()

    def getRests_p(self) -> torch.Tensor | None:
        return self.restsVect

    def setRests(self, values) -> None:
        """Restore the residual (checkpoint resume); not available in the reference."""
        t, _ = to_device_vector(self._env, values, torch.float32)
        if t.numel() != self.size:
            raise ComprexError(f"Vector of size {t.numel()} does not match Rests Vector of size {self.size}!")
        if self.restsVect is None:
            self._alloc_rests()
        self.restsVect.copy_(t)

    def addRests(self, vector) -> None:
        """vector += rests (src/comprEx.tpp:160-169)."""
        t, orig = to_device_vector(self._env, vector)
        if t.numel() != self.size:
            raise ComprexError(f"Vector of size {t.numel()} does not match Rests Vector of size {self.size}!")
        if self.restsVect is not None:
            P.axpy(self._env, t, self.restsVect, 1.0, self.size)
        write_back(t, orig)

    def state_dict(self) -> dict:
        return {"size": self.size, "rests": None if self.restsVect is None else self.restsVect.detach().cpu().clone(),
                "tx_seq": dict(self._tx_seq), "rx_seq": dict(self._rx_seq)}

    def load_state_dict(self, state: dict) -> None:
        if state["size"] != self.size:
            raise ComprexError("state_dict belongs to an engine of a different size")
        if state["rests"] is not None:
            self.setRests(state["rests"].to(self._env.device))

    # ---- connections --------------------------------------------------------------------------
    def connectTx(self, Rank: int, tag: int = 0) -> None:      # parameter name as in ComprEx.py:148
        self._check_rank(Rank)
        self._dest = int(Rank)
        self._alloc_rests()
        if self._dense is not None:
            self._dense.connectTx(Rank, tag)

    def connectRx(self, Rank: int, tag: int = 0) -> None:
        self._check_rank(Rank)
        self._src = int(Rank)
        if self._dense is not None:
            self._dense.connectRx(Rank, tag)

    def connectTo(self, srcRank: int, targRank: int, tag: int = 0) -> None:
        self.connectRx(srcRank, tag)
        self.connectTx(targRank, tag)

    def _check_rank(self, r: int) -> None:
        if not 0 <= int(r) < self._env.ranks:
            raise ComprexError(f"rank {r} outside 0..{self._env.ranks - 1}")

    def _require_tx(self) -> None:
        if self._dest is None:
            raise ComprexError("Send issued without connecting to Remote!")

    def _require_rx(self) -> None:
        if self._src is None:
            raise ComprexError("Receive issued without connecting to Remote!")

    # ---- send -----------------------------------------------------------------------------------
    def _next_tx(self, dest: int):
        seq = self._tx_seq.get(dest, 0) + 1
        self._tx_seq[dest] = seq
        return self._slots[seq & 1].endpoint(self._env, dest), seq

    def _vec(self, vector):
        t, _ = to_device_vector(self._env, vector)
        if t.numel() != self.size:
            raise ComprexError(f"vector of size {t.numel()} does not match the engine's size {self.size}")
        return t

    def _send_pairs(self, g, r, thr_obj, fixed_thr=None) -> None:
        ep, seq = self._next_tx(self._dest)
        if fixed_thr is not None:
            self._comp.set_threshold(fixed_thr)
        else:
            thr_obj._launch(self._comp, g, r, self.size)
        self._comp.compress(g, r, self.size, self.cap, seq, P.make_targets([ep]))
        self._env.maybe_check()

    def _send_other(self, g, r, thr_obj, fixed_thr=None) -> None:
        """CompressorNone / CompressorRLE payloads through the dense slot."""
        if self.compressor.kind == "none":
            src = g if g is not None else torch.zeros(self.size, dtype=torch.float32, device=self._env.device)
            tg, seq = self._dense._targets([self._dest])
            P.dense_send(self._env, src.to(torch.float32) if src.dtype != torch.float32 else src, r, self.size, seq, tg,
                         self._dense._counters)
            self._env.maybe_check()
            return
        if fixed_thr is not None:
            self._comp.set_threshold(fixed_thr)
        else:
            thr_obj._launch(self._comp, g, r, self.size)
        seq = self._tx_seq.get(self._dest, 0) + 1
        self._tx_seq[self._dest] = seq
        if g is not None and g.dtype not in (torch.float32, torch.bfloat16, torch.float16):
            g = g.to(torch.float32)
        self._rle.send(g, r, self._comp.thr, seq, self._dest)
        self._env.maybe_check()

    def _send(self, g, r, thr_obj, fixed_thr=None) -> None:
        if self.compressor.kind == "pairs":
            self._send_pairs(g, r, thr_obj, fixed_thr)
        else:
            self._send_other(g, r, thr_obj, fixed_thr)

    def writeRemote(self, vector) -> None:
        """threshold(rests + v); rests += v; send |rests| > thr; zero what was sent."""
        self._require_tx()
        self._send(self._vec(vector), self.restsVect, self.threshold)

    def writeRemote_compressOnly(self, vector) -> None:
        """Send every non-zero of ``vector``; the residual is not involved."""
        self._require_tx()
        self._send(self._vec(vector), None, None, fixed_thr=0.0)

    def writeRemote_NoResidual(self, vector) -> None:
        """Threshold from the vector alone; what is not sent is dropped."""
        self._require_tx()
        self._send(self._vec(vector), None, self.threshold)

    def flushRests(self) -> None:
        """Send the whole residual (threshold 0) and zero it."""
        self._require_tx()
        self._send(None, self.restsVect, None, fixed_thr=0.0)

    # ---- receive --------------------------------------------------------------------------------
    def _next_rx(self):
        self._require_rx()
        seq = self._rx_seq.get(self._src, 0) + 1
        self._rx_seq[self._src] = seq
        return self._slots[seq & 1].endpoint(self._env), seq

    def _take_rx(self):
        if self._rx_current is not None:
            cur, self._rx_current = self._rx_current, None
            return cur
        return self._next_rx()

    def _recv_other(self, t: torch.Tensor, add: bool) -> None:
        if self.compressor.kind == "none":
            if add:
                self._dense.readRemote_add(t, self.size)
            else:
                self._dense.readRemote_vec(t, self.size)
            return
        seq = self._rx_seq.get(self._src, 0) + 1
        self._rx_seq[self._src] = seq
        if t.dtype == torch.float32:
            self._rle.recv(t, seq, add, self._status)
        else:
            tmp = t.to(torch.float32)
            self._rle.recv(tmp, seq, add, self._status)
            t.copy_(tmp)
        self._env.maybe_check()

    def readRemote(self, vector=None):
        """Wait and decompress (overwrite).  Returns a new tensor without ``vector``."""
        self._require_rx()
        ret = vector is None
        if ret:
            vector = torch.empty(self.size, dtype=torch.float32, device=self._env.device)
        t, orig = to_device_vector(self._env, vector)
        if self.compressor.kind != "pairs":
            self._recv_other(t, add=False)
        else:
            ep, seq = self._take_rx()
            P.apply_sparse(self._env, P.make_sources([ep], [seq]), self.size, P.args_set(t), self._status)
            self._env.maybe_check()
        write_back(t, orig)
        return vector if ret else None

    def readRemote_add(self, vector) -> None:
        """Wait and scatter-add into ``vector``."""
        self._require_rx()
        t, orig = to_device_vector(self._env, vector)
        if self.compressor.kind != "pairs":
            self._recv_other(t, add=True)
        else:
            ep, seq = self._take_rx()
            P.apply_sparse(self._env, P.make_sources([ep], [seq]), self.size, P.args_add(t), self._status)
            self._env.maybe_check()
        write_back(t, orig)

    def readRemote_wait(self) -> None:
        self._rx_current = self._next_rx()

    # ---- forwarding (src/comprEx.tpp:248-301) -----------------------------------------------------
    def _require_pairs(self, what: str) -> None:
        if self.compressor.kind != "pairs":
            raise ComprexError(f"{what} needs the IndexPairs compressor")

    def readRemote_forward(self, vector) -> None:
        """Wait, pass the payload on unchanged, decompress it into ``vector``."""
        self._require_pairs("readRemote_forward")
        self._require_tx()
        t, orig = to_device_vector(self._env, vector)
        ep, seq = self._take_rx()
        tep, tseq = self._next_tx(self._dest)
        P.forward(self._env, ep, seq, P.make_targets([tep]), tseq, self.cap, self._counters, self._status)
        P.apply_sparse(self._env, P.make_sources([ep], [seq]), self.size, P.args_set(t), self._status)
        self._env.maybe_check()
        write_back(t, orig)

    def readRemote_forwardCopy(self, vector=None) -> None:
        """Wait and stage the payload for a later ``forward_add``."""
        self.forward_buffer()

    def forward_buffer(self) -> None:
        self._require_pairs("forward_buffer")
        self._held = self._take_rx()

    def forward_add(self, vector) -> None:
        """Send the staged payload on and scatter-add it into ``vector``."""
        self._require_pairs("forward_add")
        self._require_tx()
        if self._held is None:
            raise ComprexError("forward_add without a preceding forward_buffer")
        ep, seq = self._held
        self._held = None
        t, orig = to_device_vector(self._env, vector)
        tep, tseq = self._next_tx(self._dest)
        P.forward(self._env, ep, seq, P.make_targets([tep]), tseq, self.cap, self._counters, self._status)
        P.apply_sparse(self._env, P.make_sources([ep], [seq]), self.size, P.args_add(t), self._status)
        self._env.maybe_check()
        write_back(t, orig)

    def stats(self) -> dict:
        """nnz, threshold and status of the last compression (synchronises)."""
        return self._comp.last_stats()


class FastComprex(Comprex):
    """One-step-stale variant (src/comprEx.tpp:371-514).

    ``writeRemote`` first sends what the previous call compressed and then
    compresses the current input into a local staging slot; the receiver sees
    every update one call late.  On NVLink the overlap this buys in the
    reference is not needed, the class exists so that code written against
    ``FastComprEx`` keeps its semantics (including ``flushRests`` folding the
    pending payload back into the residual and ``writeRemote_sameAs``).
    """

    def __init__(self, gaspi_env, size: int, size_factor: float = 1.0):
        super().__init__(gaspi_env, size, size_factor)
        self._stage = [P.SparseSlot.create(self._env, self.size, self.cap) for _ in range(2)]
        self._stage_seq = 0
        self.is_first = True

    def resetRests(self) -> None:
        super().resetRests()
        self.is_first = True

    def _stage_ep(self, seq: int):
        return self._stage[seq & 1].endpoint(self._env)

    def _send_pending(self) -> None:
        """Forward the payload staged by the previous call (empty on the first call)."""
        ep, seq = self._next_tx(self._dest)
        if self.is_first:
            self._comp.set_threshold(self.threshold.getThreshold() if not isinstance(self.threshold, ThresholdTopK) else 0.0)
            # rests are all zero at this point: an empty payload
            self._comp.compress(None, self.restsVect, self.size, self.cap, seq, P.make_targets([ep]))
            self.is_first = False
        else:
            P.forward(self._env, self._stage_ep(self._stage_seq), self._stage_seq, P.make_targets([ep]), seq,
                      self.cap, self._counters, self._status)

    def _stage_new(self, g, r, thr_obj, fixed_thr=None) -> None:
        self._stage_seq += 1
        if fixed_thr is not None:
            self._comp.set_threshold(fixed_thr)
        else:
            thr_obj._launch(self._comp, g, r, self.size)
        self._comp.compress(g, r, self.size, self.cap, self._stage_seq,
                            P.make_targets([self._stage_ep(self._stage_seq)]))

    def writeRemote(self, vector) -> None:
        self._require_tx()
        self._require_pairs("FastComprex")
        t = self._vec(vector)
        self._send_pending()
        self._stage_new(t, self.restsVect, self.threshold)
        self._env.maybe_check()

    def writeRemote_compressOnly(self, vector) -> None:
        self._require_tx()
        self._require_pairs("FastComprex")
        t = self._vec(vector)
        self._send_pending()
        self._stage_new(t, None, None, fixed_thr=0.0)
        self._env.maybe_check()

    def writeRemote_sameAs(self, other: "FastComprex") -> None:
        """Send my pending payload, then take over what ``other`` just staged."""
        self._require_tx()
        self._send_pending()
        if not other.is_first:
            self._stage_seq += 1
            P.forward(self._env, other._stage_ep(other._stage_seq), other._stage_seq,
                      P.make_targets([self._stage_ep(self._stage_seq)]), self._stage_seq, self.cap,
                      self._counters, self._status)
        else:
            self.is_first = True
        self._env.maybe_check()

    def connectTx_sameBufferAs(self, targRank: int, tag: int, other: "FastComprex") -> None:
        if other._dest is None:
            raise ComprexError("Cannot connected with buffer of unconnected communicator!")
        self.connectTx(targRank, tag)

    def flushRests(self) -> None:
        """Fold the pending payload back into the residual, then send everything."""
        self._require_tx()
        if not self.is_first:
            ep = self._stage_ep(self._stage_seq)
            P.apply_sparse(self._env, P.make_sources([ep], [self._stage_seq]), self.size,
                           P.args_add(self.restsVect), self._status)
        ep, seq = self._next_tx(self._dest)
        self._comp.set_threshold(0.0)
        self._comp.compress(None, self.restsVect, self.size, self.cap, seq, P.make_targets([ep]))
        self.is_first = True
        self._env.maybe_check()
