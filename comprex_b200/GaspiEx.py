"""Dense point-to-point vector exchange (reference: include/gaspiEx.hxx:15-89,
src/gaspiEx.tpp:32-192, Python face GaspiEx.py:44-96).

A ``GaspiEx`` of ``size`` elements owns a double-buffered receive slot in the
symmetric heap.  ``writeRemote`` launches one kernel that reads the user's
vector and stores it straight into the destination rank's slot over NVLink
(no staging copy, no library call) and then publishes a sequence number;
``readRemote*`` launches a kernel that waits for that number with a time
budget and copies or adds the slot into the user's vector.  Construction is
collective (every rank creates its engines in the same order); the connect
calls only record the peer, the tag is kept for interface parity.

Vectors may be ``torch`` tensors on the environment's device or NumPy arrays
(copied to the device and, for in-place calls, back).

Flow control: the receive slot is double-buffered by the parity of the message
number and nothing is acknowledged, so a sender may be at most two writes ahead
of its receiver's reads; a third write overwrites a slot that may not have been
read yet.  Exchanges in which both sides send and receive every step (the
allreduce schedules) keep within that by construction; a one-directional stream
of writes has to be paced by the caller (a barrier, or a message back), as in the
reference, whose transport has no flow control either (src/gaspiEx.tpp:70-88).
"""
from __future__ import annotations

import numpy as np
import torch

from .common import AbstractExchange, Getable  # noqa: F401  (the reference defines Getable in this module too)
from ._lib import ComprexError
from .ops import primitives as P


def to_device_vector(env, vector, dtype=None):
    """Returns (flat tensor on env.device, original NumPy array or None)."""
    if isinstance(vector, np.ndarray):
        t = torch.from_numpy(np.ascontiguousarray(vector).reshape(-1))
        if dtype is not None and t.dtype != dtype:
            t = t.to(dtype)
        return t.to(env.device), vector
    if not isinstance(vector, torch.Tensor):
        raise ComprexError("vector must be a torch.Tensor or a numpy.ndarray")
    if vector.device != env.device:
        raise ComprexError(f"vector lives on {vector.device}, the environment on {env.device}")
    if not vector.is_contiguous():
        raise ComprexError("vector must be contiguous")
    return vector.view(-1), None


def write_back(t: torch.Tensor, original) -> None:
    if original is not None:
        np.copyto(original.reshape(-1), t.detach().cpu().numpy().astype(original.dtype, copy=False))


class GaspiEx(AbstractExchange):
    def __init__(self, gaspi_env, size: int, dtype: torch.dtype = torch.float32):
        self._env = env = gaspi_env.get()
        self.size = int(size)
        self.dtype = dtype
        self._es = torch.empty(0, dtype=dtype).element_size()
        self._slots = [P.DenseSlot.create(env, self.size * self._es) for _ in range(2)]
        self._counters = env.scratch(64)
        self._status = env.new_status("GaspiEx")
        self._tx_seq: dict[int, int] = {}
        self._rx_seq: dict[int, int] = {}
        self._dest = None
        self._src = None
        self._alias_of = None
        self._last_sent = None
        self._held = None       # (tensor, n) copied by forward_buffer
        self._rx_current = None  # endpoint + seq picked by readRemote_wait

    # ---- connections (src/gaspiEx.tpp:121-192) -----------------------------------
    def connectTx(self, destRank: int, tag: int = 0) -> None:
        self._check_rank(destRank)
        self._dest = int(destRank)

    def connectRx(self, srcRank: int, tag: int = 0) -> None:
        self._check_rank(srcRank)
        self._src = int(srcRank)

    def connectTo(self, srcRank: int, destRank: int, tag: int = 0) -> None:
        self.connectRx(srcRank, tag)
        self.connectTx(destRank, tag)

    def connectTx_sameBufferAs(self, destRank: int, tag: int, other: "GaspiEx") -> None:
        """This engine re-sends what ``other`` sent last (zero-copy fan-out)."""
        if other._dest is None:
            raise ComprexError("Cannot connect with buffer of unconnected communicator!")
        self.connectTx(destRank, tag)
        self._alias_of = other

    def _check_rank(self, r: int) -> None:
        if not 0 <= int(r) < self._env.ranks:
            raise ComprexError(f"rank {r} outside 0..{self._env.ranks - 1}")

    def getSize(self) -> int:
        return self.size

    # ---- send ------------------------------------------------------------------------
    def _targets(self, dests):
        eps, seqs = [], []
        for d in dests:
            seq = self._tx_seq.get(d, 0) + 1
            self._tx_seq[d] = seq
            eps.append(self._slots[seq & 1].endpoint(self._env, d))
            seqs.append(seq)
        if len(set(seqs)) != 1:
            raise ComprexError("destinations of one multi-target write must have seen the same number of writes")
        # Several destinations share one payload: where the heap is bound to a multicast object the
        # vector crosses the sender's link once (connectTx_sameBufferAs, src/gaspiEx.tpp:142-153).
        # A multicast store also lands in the sender's own copy of the slot, so it is only used by
        # an engine that does not receive (a broadcasting chief).
        mc = self._slots[seqs[0] & 1].mc_endpoint(self._env) if self._src is None else None
        return P.make_targets(eps, mc=mc), seqs[0]

    def writeRemote(self, vector=None, size: int | None = None) -> None:
        """Send ``vector`` to the connected rank.  Without a vector, re-send the
        aliased engine's last vector (``writeRemote(size)`` of the reference)."""
        if self._dest is None:
            raise ComprexError("Send issued without connecting to Remote!")
        if vector is None or isinstance(vector, int):
            src = self._alias_of if self._alias_of is not None else self
            if src._last_sent is None:
                raise ComprexError("nothing was sent yet through the shared buffer")
            t = src._last_sent
        else:
            t, _ = to_device_vector(self._env, vector, self.dtype)
        n = t.numel() if size is None else int(size)
        if n > self.size:
            raise ComprexError("Vector is too large to be send with this GaspiEx instance!")
        if t.dtype != self.dtype:
            raise ComprexError(f"vector dtype {t.dtype} does not match the engine's {self.dtype}")
        tg, seq = self._targets([self._dest])
        P.dense_send(self._env, t, None, n, seq, tg, self._counters)
        self._last_sent = t
        self._env.maybe_check()

    def writeRemote_multi(self, vector, dests) -> None:
        """One launch that stores ``vector`` into the slots of all ``dests``."""
        t, _ = to_device_vector(self._env, vector, self.dtype)
        if t.numel() > self.size:
            raise ComprexError("Vector is too large to be send with this GaspiEx instance!")
        tg, seq = self._targets([int(d) for d in dests])
        P.dense_send(self._env, t, None, t.numel(), seq, tg, self._counters)
        self._last_sent = t
        self._env.maybe_check()

    # ---- receive ---------------------------------------------------------------------
    def _next_rx(self):
        if self._src is None:
            raise ComprexError("Receive issued without connecting to Remote!")
        seq = self._rx_seq.get(self._src, 0) + 1
        self._rx_seq[self._src] = seq
        return self._slots[seq & 1].endpoint(self._env), seq

    def _take_rx(self):
        if self._rx_current is not None:
            cur, self._rx_current = self._rx_current, None
            return cur
        return self._next_rx()

    def readRemote(self) -> torch.Tensor:
        out = torch.empty(self.size, dtype=self.dtype, device=self._env.device)
        self.readRemote_vec(out, self.size)
        return out

    def readRemote_vec(self, vector, size: int | None = None) -> None:
        t, orig = to_device_vector(self._env, vector, self.dtype)
        n = t.numel() if size is None else int(size)
        if n > self.size:
            raise ComprexError("Too much data to be read with this GaspiEx instance!")
        ep, seq = self._take_rx()
        P.dense_reduce(self._env, t, None, n, P.make_sources([ep], [seq]), self._status)
        self._env.maybe_check()
        write_back(t, orig)

    def readRemote_add(self, vector, size: int | None = None) -> None:
        t, orig = to_device_vector(self._env, vector, self.dtype)
        n = t.numel() if size is None else int(size)
        if n > self.size:
            raise ComprexError("Too much data to be read with this GaspiEx instance!")
        ep, seq = self._take_rx()
        P.dense_reduce(self._env, t, t, n, P.make_sources([ep], [seq]), self._status)
        self._env.maybe_check()
        write_back(t, orig)

    def readRemote_wait(self) -> None:
        """Select the next incoming message; later calls in the stream wait for it."""
        self._rx_current = self._next_rx()

    # ---- forwarding (src/gaspiEx.tpp:105-119) ---------------------------------------------
    def forward_buffer(self, size: int | None = None) -> None:
        """Copy the received message into this engine's send side."""
        n = self.size if size is None else int(size)
        ep, seq = self._take_rx()
        held = torch.empty(self.size, dtype=self.dtype, device=self._env.device)
        P.dense_reduce(self._env, held, None, n, P.make_sources([ep], [seq]), self._status)
        self._held = (held, n)

    def forward_add(self, vector, size: int | None = None) -> None:
        """Send the held message on and add it to ``vector``."""
        if self._held is None:
            raise ComprexError("forward_add without a preceding forward_buffer")
        held, n = self._held
        t, orig = to_device_vector(self._env, vector, self.dtype)
        tg, seq = self._targets([self._dest])
        P.dense_send(self._env, held, None, n, seq, tg, self._counters)
        P.axpy(self._env, t, held, 1.0, n)
        self._last_sent = held
        self._env.maybe_check()
        write_back(t, orig)
