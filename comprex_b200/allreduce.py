"""Allreduce collectives: AllToOne, Ring, BigRing, dense and compressed
(reference: include/allreduce.hxx:15-211, src/allreduce.tpp:20-721, Python
face allreduce.py:143-355).

The reference moves data hop by hop through GaspiEx/ComprEx pairs because its
transport is point-to-point RDMA.  Behind an NVSwitch every peer is one hop
away at full bandwidth, so each schedule is re-expressed as direct stores:

* **BigRing** ("everyone gets everyone's whole vector"): one compression whose
  pairs are stored into all P-1 peers' slots by the same kernel, then one
  kernel that scatter-adds all received payloads in the order the ring would
  have delivered them.  Dense: one-shot push + reduce.
* **Ring** (reduce-scatter + allgather over P chunks; rank r ends up owning
  chunk (r+1) mod P like the reference): every rank compresses each foreign
  chunk, with that chunk's residual, straight into the owner's slot; the owner
  adds them to its dense chunk, re-selects the top-k of the reduced chunk and
  stores it to all peers; everyone decodes.  Dense: two-shot.
* **AllToOne**: workers store into the chief's slots, the chief reduces,
  compresses once and stores to all workers (``writeRemote_sameAs`` of the
  reference is "one compression, P-1 store streams" here).

All classes keep the reference's surface: ``setup_connections``, ``apply``
(in place, returns the vector), and for the compressed ones ``flush``,
``reset``, ``set_compression_ratio``, ``getSize``.  Additions: ``dtype`` for
bf16/fp16 vectors, ``consistent=True`` (every rank, the sender included,
applies only what was transmitted, so replicas stay bit-identical),
``state_dict``/``load_state_dict`` for the residuals, ``stats``.

``apply`` is split into phases (``_plan_apply``) so that a
:class:`~comprex_b200.parallel.env.LoopbackWorld` can run P virtual ranks on
one device.  Between real ranks the launches of a call are recorded once per
parity of the step and replayed with one native call, from six launches on as
a CUDA graph; independent launches (the per-chunk work of the compressed Ring)
run on side-stream lanes.
"""
from __future__ import annotations

import ctypes as C
import logging
import math
import os

import torch

from . import _lib
from ._lib import ComprexError
from .GaspiEx import to_device_vector, write_back
from .ops import primitives as P


_log = logging.getLogger("comprex.allreduce")


def _chunks(size: int, nranks: int, align: int = 1):
    """Chunk sizes and starts of the ring (src/allreduce.tpp:279-295).  With ``align`` > 1 every
    chunk but the last is a multiple of ``align`` elements, so that every chunk starts on an
    address the kernels can use 16-byte accesses on (the last chunk takes the remainder)."""
    if align > 1:
        base = (size // nranks) // align * align
        sizes = [base] * (nranks - 1) + [size - base * (nranks - 1)]
    else:
        base, rem = divmod(size, nranks)
        sizes = [base + (1 if i < rem else 0) for i in range(nranks)]
    starts = [0] * nranks
    for i in range(1, nranks):
        starts[i] = starts[i - 1] + sizes[i - 1]
    return sizes, starts


def _cap_for(n: int, size_factor: float) -> int:
    """Pair capacity of a buffer of n*4*size_factor bytes (src/comprEx.tpp:61)."""
    return max(int(n * 4 * size_factor - 8) // 8, 1)


def _use_switch(env, nbytes: int) -> bool:
    """Dense vectors go through the NVSwitch's in-switch reduction when the heap is bound to a
    multicast object, from ``COMPREX_MM_MIN_RANKS`` ranks (default 4: with two ranks the switch
    saves no traffic over plain peer stores) and ``COMPREX_MM_MIN_BYTES`` bytes (default 256 KiB:
    below that the two-launch peer-store schedule has the lower latency)."""
    if env.ranks < int(os.environ.get("COMPREX_MM_MIN_RANKS", 4)):
        return False
    if nbytes < int(os.environ.get("COMPREX_MM_MIN_BYTES", 256 << 10)):
        return False
    return env.nvls


class _OpSeq:
    """A launch sequence built once (an array of CxOp) and run with one native call per step.

    With ``graph=True`` on a CUDA device the sequence is also captured as a CUDA graph whose
    kernels read the sequence number from a device cell: a step is then one 8-byte copy plus one
    graph launch, whatever the number of kernels (``COMPREX_GRAPHS=0`` keeps the plain list)."""

    def __init__(self, env, ops, graph: bool = False):
        self.env = env
        self.arr = (_lib.Op * len(ops))(*ops)
        self.count = len(ops)
        self.graph = None
        if graph:
            self.enable_graph()

    def enable_graph(self) -> None:
        """Capture the sequence (once).  A graph pays off from about half a dozen launches
        (measured: 3-launch sequences lose ~7 us to the cell copy and the graph's own launch, the
        24-launch compressed ring gains 25 %)."""
        env = self.env
        if (self.graph is not None or getattr(self, "_no_graph", False) or env.dev != _lib.DEV_CUDA
                or self.count < 6 or os.environ.get("COMPREX_GRAPHS", "1") == "0"):
            return
        handle = C.c_void_p()
        if env.lib.cx_graph_build(self.arr, self.count, C.byref(handle)) == 0:
            self.graph = handle
        else:
            _log.warning("launch sequence not captured as a graph (%s); using the op list", _lib.last_error())
            self._no_graph = True            # not retried

    def run(self, seq: int) -> None:
        env = self.env
        if self.graph is not None:
            _lib.check(env.lib.cx_graph_launch(self.graph, seq, _lib.stream_ptr(env.device)), "cx_graph_launch")
            return
        _lib.check(env.lib.cx_run_ops(self.arr, self.count, seq, _lib.stream_ptr(env.device)), "cx_run_ops")

    def __del__(self):
        try:
            if self.graph is not None:
                self.env.lib.cx_graph_free(self.graph)
                self.graph = None
        except Exception:
            pass


class _AllreduceBase:
    compressed = False

    def __init__(self, gaspi_env):
        self._env = gaspi_env.get()
        self.gaspi_env = gaspi_env
        self.size = None
        self._step = 0
        # dense variants: factor applied to the sum inside the reducing kernel (1/P gives the mean
        # without an extra pass); set it before the first apply
        self.result_scale = 1.0

    def get(self):
        return self

    def getSize(self):
        return self.size

    @property
    def first_phase_waits(self) -> bool:
        """True when already the first phase of ``_plan_apply`` waits for the peers (the
        single-kernel allreduce through the switch); otherwise the first phase only sends."""
        return getattr(self, "_mm", None) is not None

    def _setup_common(self, size: int, dtype: torch.dtype) -> None:
        if self.size is not None:
            raise ComprexError("connections are already set up")
        self.size = int(size)
        self.dtype = dtype
        self._check_agreement()
        self._status = self._env.new_status(type(self).__name__)
        self._counters = self._env.scratch(64)

    def _check_agreement(self) -> None:
        """Collective: every rank must set up the same kind of allreduce for the same size (slot
        layouts are derived from it; a mismatch would otherwise show up as BAD_HEADER later)."""
        env = self._env
        if env._world is not None or env.ranks == 1 or env.group is None:
            return
        mine = (type(self).__name__, self.size, str(self.dtype))
        theirs = env._exchange(mine)
        if any(t != mine for t in theirs):
            raise ComprexError("allreduce set-up differs between ranks: " +
                               ", ".join(f"rank {r}: {t}" for r, t in enumerate(theirs)))

    # Target / source descriptors depend only on the parity of the step: they are built
    # once and reused, a call then only refreshes the sequence numbers.
    def _cached_targets(self, key, build):
        cache = self.__dict__.setdefault("_desc_cache", {})
        tg = cache.get(key)
        if tg is None:
            tg = cache[key] = P.make_targets(build())
        return tg

    def _cached_sources(self, key, build, seq):
        cache = self.__dict__.setdefault("_desc_cache", {})
        src = cache.get(key)
        if src is None:
            eps = build()
            src = cache[key] = P.make_sources(eps, [seq] * len(eps))
        for i in range(src.count):
            src.seq[i] = seq
        return src

    def _prep(self, vector):
        if self.size is None:
            raise ComprexError("setup_connections was not called")
        n = vector.size if hasattr(vector, "size") and not callable(vector.size) else vector.numel()
        if n != self.size:
            raise ComprexError("Allreduce input vector of size %d does not match allreduce size %d!" % (n, self.size))
        t, orig = to_device_vector(self._env, vector)
        return t, orig

    def _run(self, plan, t, orig, vector):
        for phase in plan:
            phase()
        self._env.maybe_check()
        write_back(t, orig)
        return vector

    def apply(self, vector):
        """In-place allreduce of ``vector``; returns it (allreduce.py:159-166).

        Between real ranks the launches of a call depend only on the vector's address and
        the parity of the step, so they are recorded once as an array of CxOp and replayed
        with one native call per step.  Virtual ranks (``LoopbackWorld``) run phase by phase."""
        t, orig = self._prep(vector)
        env = self._env
        if env._world is not None or not self._replay:
            return self._run(self._plan_apply(t), t, orig, vector)
        cache = self.__dict__.setdefault("_replay_cache", {})
        key = (t.data_ptr(), t.dtype, (self._step + 1) & 1)
        ops = cache.get(key)
        if ops is None:
            if len(cache) >= 64:
                cache.clear()
            env._rec = rec = []
            try:
                for phase in self._plan_apply(t):     # advances the step itself
                    phase()
            finally:
                env._rec = None
            ops = cache[key] = _OpSeq(env, rec) if rec else False
        else:
            self._step += 1
            if ops and ops.graph is None:
                # the same vector came back: worth capturing (a caller that hands over a new
                # tensor every time never pays for a capture)
                ops.enable_graph()
        if ops:
            ops.run(self._step)
        env.maybe_check()
        write_back(t, orig)
        return vector

    __call__ = apply
    _replay = True


# =====================================================================================
# dense variants
# =====================================================================================
class AllToOneAllreduce(_AllreduceBase):
    """Workers -> chief -> workers (src/allreduce.tpp:29-118)."""

    def setup_connections(self, size, tag=0, chiefRank=0, dtype=torch.float32):
        self._setup_common(size, dtype)
        env, nb = self._env, size * torch.empty(0, dtype=dtype).element_size()
        self.chiefRank = int(chiefRank)
        self._rs = [[P.DenseSlot.create(env, nb) for _ in range(2)] for _ in range(env.ranks)]
        self._bc = [P.DenseSlot.create(env, nb) for _ in range(2)]

    def _plan_apply(self, t):
        env, me, chief = self._env, self._env.rank, self.chiefRank
        self._step += 1
        seq, par = self._step, self._step & 1
        workers = [r for r in range(env.ranks) if r != chief]

        def send():
            if me != chief:
                P.dense_send(env, t, None, self.size, seq, P.make_targets([self._rs[me][par].endpoint(env, chief)]),
                             self._counters)

        def reduce():
            if me == chief:
                src = P.make_sources([self._rs[w][par].endpoint(env) for w in workers], [seq] * len(workers))
                push = P.make_targets([self._bc[par].endpoint(env, w) for w in workers],
                                      mc=self._bc[par].mc_endpoint(env))
                P.dense_reduce(env, t, t, self.size, src, self._status, scale=self.result_scale, push=push,
                               push_seq=seq, counters=self._counters)

        def recv():
            if me != chief:
                P.dense_reduce(env, t, None, self.size, P.make_sources([self._bc[par].endpoint(env)], [seq]),
                               self._status)
        return [send, reduce, recv]


class RingAllreduce(_AllreduceBase):
    """Reduce-scatter + allgather over P chunks (src/allreduce.tpp:273-351), two-shot.

    Where the heap is bound to an NVSwitch multicast object (``env.nvls``) both shots happen in
    the switch: every rank pulls the sum of its chunk with ``multimem.ld_reduce`` and broadcasts
    it with ``multimem.st``, one kernel per call; ``COMPREX_NVLS=0`` keeps the peer-store kernels."""

    def setup_connections(self, size, tag=0, dtype=torch.float32):
        self._setup_common(size, dtype)
        env = self._env
        self.segment_sizes, self.segment_starts = _chunks(size, env.ranks)
        self._mm = None
        if _use_switch(env, size * torch.empty(0, dtype=dtype).element_size()):
            # the switch reduces and broadcasts: one kernel per rank (csrc/nvls.cu)
            self._mm = P.MultimemAllreduce(env, size, dtype)
            return
        nb = max(self.segment_sizes) * torch.empty(0, dtype=dtype).element_size()
        self._rs = [[P.DenseSlot.create(env, nb) for _ in range(2)] for _ in range(env.ranks)]
        self._ag = [[P.DenseSlot.create(env, nb) for _ in range(2)] for _ in range(env.ranks)]

    def _owner(self, chunk: int) -> int:
        return (chunk - 1) % self._env.ranks

    def _plan_apply(self, t):
        env, me, nr = self._env, self._env.rank, self._env.ranks
        self._step += 1
        seq, par = self._step, self._step & 1
        if self._mm is not None:
            return [lambda: self._mm.run(t, seq, self.result_scale, self._status)]
        mine = (me + 1) % nr
        others = [c for c in range(nr) if c != mine]
        peers = [r for r in range(nr) if r != me]
        my_view = t[self.segment_starts[mine]: self.segment_starts[mine] + self.segment_sizes[mine]]

        def scatter():
            if nr == 1:
                return
            tg = P.make_targets([self._rs[me][par].endpoint(env, self._owner(c)) for c in others])
            P.dense_send(env, t, None, self.size, seq, tg, self._counters,
                         ranges=[(self.segment_starts[c], self.segment_sizes[c]) for c in others])

        def reduce():
            if nr == 1:
                return
            src = P.make_sources([self._rs[j][par].endpoint(env) for j in peers], [seq] * len(peers))
            push = P.make_targets([self._ag[me][par].endpoint(env, j) for j in peers])
            P.dense_reduce(env, my_view, my_view, self.segment_sizes[mine], src, self._status,
                           scale=self.result_scale, push=push, push_seq=seq, counters=self._counters)

        def gather():
            if nr == 1:
                return
            src = P.make_sources([self._ag[j][par].endpoint(env) for j in peers], [seq] * len(peers))
            rg = [(self.segment_starts[(j + 1) % nr], self.segment_sizes[(j + 1) % nr]) for j in peers]
            P.dense_reduce(env, t, None, self.size, src, self._status, ranges=rg)
        return [scatter, reduce, gather]


class BigRingAllreduce(_AllreduceBase):
    """Every rank receives every other rank's whole vector (src/allreduce.tpp:542-601), one-shot.

    One-shot moves (P-1) n elements out of every GPU.  Through a switch that gives every
    pair full bandwidth this is the lowest-latency schedule for small vectors and the
    wrong one for large vectors, so above ``two_shot_bytes`` (default 1 MiB, environment
    variable ``COMPREX_TWO_SHOT_BYTES``; never with two ranks, where both schedules move
    the same bytes) the call runs the reduce-scatter + allgather schedule of
    ``RingAllreduce``: 2 (P-1)/P n elements, every rank ends with the same bits."""

    def setup_connections(self, size, tag=0, dtype=torch.float32, two_shot_bytes=None, ordered=False):
        """``ordered=True``: the one-shot form adds the vectors in rank order on every rank (the
        reference adds them in the order the ring delivers them, which differs from rank to rank
        in the last bits): all ranks then hold identical bits, like with the other schedules."""
        self._setup_common(size, dtype)
        self.ordered = bool(ordered)
        env, nb = self._env, size * torch.empty(0, dtype=dtype).element_size()
        if two_shot_bytes is None:
            two_shot_bytes = int(os.environ.get("COMPREX_TWO_SHOT_BYTES", 1 << 20))
        self._two_shot = None
        self._mm = None
        if _use_switch(env, nb):
            # through the switch: one-shot for small vectors, reduce-scatter + broadcast above
            self._mm = P.MultimemAllreduce(env, size, dtype)
            return
        if env.ranks > 2 and nb > two_shot_bytes:
            self._two_shot = RingAllreduce(self.gaspi_env)
            self._two_shot.setup_connections(size, tag, dtype)
            return
        self._slots = [[P.DenseSlot.create(env, nb) for _ in range(2)] for _ in range(env.ranks)]

    def _plan_apply(self, t):
        if self._mm is not None:
            self._step += 1
            seq = self._step
            return [lambda: self._mm.run(t, seq, self.result_scale, self._status)]
        if self._two_shot is not None:
            self._two_shot._step = self._step          # one step counter: sequence numbers and parity agree
            self._two_shot.result_scale = self.result_scale
            self._step += 1
            return self._two_shot._plan_apply(t)
        env, me, nr = self._env, self._env.rank, self._env.ranks
        self._step += 1
        seq, par = self._step, self._step & 1
        arrival = [(me - k) % nr for k in range(1, nr)]  # the order the ring delivers in
        if self.ordered:
            arrival = [r for r in range(nr) if r != me]   # rank order, the own vector at position `me`

        def send():
            if nr > 1:
                tg = self._cached_targets(("tg", par), lambda: [self._slots[me][par].endpoint(env, r)
                                                                 for r in range(nr) if r != me])
                P.dense_send(env, t, None, self.size, seq, tg, self._counters)

        def reduce():
            if nr > 1:
                src = self._cached_sources(("src", par), lambda: [self._slots[j][par].endpoint(env) for j in arrival],
                                           seq)
                src.pad = me if self.ordered else 0
                P.dense_reduce(env, t, t, self.size, src, self._status, scale=self.result_scale)
        return [send, reduce]


# =====================================================================================
# compressed variants
# =====================================================================================
class _ComprexAllreduceBase(_AllreduceBase):
    compressed = True

    def _setup_compressed(self, size, compression_ratio, size_factor, consistent):
        self._setup_common(size, torch.float32)
        self.compression_ratio = float(compression_ratio)
        self.size_factor = float(size_factor)
        self.consistent = bool(consistent)
        # sampling of the reduce-side threshold (src/allreduce.tpp:401-403, 625-627)
        self._subsamples = 1000 // self._env.ranks
        self._sample_factor = 4.0

    def set_compression_ratio(self, compression_ratio):
        """Change top-k for later calls.  The ring-specific sampling parameters are
        kept (the reference silently falls back to the defaults here)."""
        self.compression_ratio = float(compression_ratio)
        self.__dict__.pop("_replay_cache", None)      # the ratio is part of the recorded launches
        self.__dict__.pop("_fast_cache", None)

    def set_exact_topk(self, exact: bool = True) -> None:
        """Threshold from a select over the whole vector (exactly top-k) instead of the sampled
        estimate of the reference; costs a few extra passes over the vector per call."""
        if exact:
            self._sampling = getattr(self, "_sampling", (self._subsamples, self._sample_factor))
            self._subsamples = 2 ** 31 - 128
        elif hasattr(self, "_sampling"):
            self._subsamples, self._sample_factor = self._sampling
        self.__dict__.pop("_replay_cache", None)
        self.__dict__.pop("_seq_cache", None)
        self.__dict__.pop("_fast_cache", None)

    def reset(self):
        for r in self._residuals():
            r.zero_()

    def flush(self, vector):
        """Drain all residuals into ``vector`` (see each class) and reset them."""
        t, orig = self._prep(vector)
        return self._run(self._plan_flush(t), t, orig, vector)

    def state_dict(self):
        return {"size": self.size, "ratio": self.compression_ratio, "step": self._step,
                "world_size": self._env.ranks, "rank": self._env.rank, "kind": type(self).__name__,
                "residuals": [r.detach().cpu().clone() for r in self._residuals()]}

    def load_state_dict(self, state):
        if state["size"] != self.size or state["kind"] != type(self).__name__:
            raise ComprexError("state_dict belongs to a different allreduce")
        self.compression_ratio = state["ratio"]
        for dst, src in zip(self._residuals(), state["residuals"]):
            dst.copy_(src.to(dst.device))

    def stats(self):
        """nnz / threshold / overflow of this rank's last compression (synchronises)."""
        return self._comp.last_stats()

    def _flush_rounds(self, n, cap):
        """Compress calls that drain a fully dense residual of ``n`` elements through a slot of
        ``cap`` pairs.  The compress kernel cuts the pair list into R regions and sub-tile s may
        only use region s mod R, so the bound is the busiest region's, not n / cap."""
        regions, region_size = P.compress_regions(n, cap)
        nsub = (n + _lib.SUBTILE - 1) // _lib.SUBTILE
        per_region = math.ceil(nsub / regions) * _lib.SUBTILE
        return max(1, math.ceil(per_region / max(region_size, 1)))


class Comprex_BigRingAllreduce(_ComprexAllreduceBase):
    """Top-k of (vector + residual) from every rank to every rank
    (src/allreduce.tpp:616-721).

    Reference semantics (default): rank r ends with its own dense vector plus
    the sparse contributions of all peers, added in ring arrival order.
    ``consistent=True``: every rank ends with exactly the sum of all sparse
    contributions (its own included), identical bits everywhere.
    """

    def setup_connections(self, size, tag=0, compression_ratio=0.01, size_factor=1.0, consistent=False):
        self._setup_compressed(size, compression_ratio, size_factor, consistent)
        env = self._env
        self.cap = _cap_for(size, size_factor)
        self._slots = [[P.SparseSlot.create(env, size, self.cap) for _ in range(2)] for _ in range(env.ranks)]
        self._comp = P.Compressor(env, size)
        self.rests = torch.zeros(size, dtype=torch.float32, device=env.device)

    def _residuals(self):
        return [self.rests]

    def _order(self):
        me, nr = self._env.rank, self._env.ranks
        return list(range(nr)) if self.consistent else [(me - k) % nr for k in range(1, nr)]

    def _send_targets(self, par):
        env, me = self._env, self._env.rank
        dests = [r for r in range(env.ranks) if r != me or self.consistent]
        cache = self.__dict__.setdefault("_desc_cache", {})
        tg = cache.get(("tg", par))
        if tg is None:      # one multicast store reaches all peers' slots where the switch offers it
            tg = cache[("tg", par)] = P.make_targets([self._slots[me][par].endpoint(env, r) for r in dests],
                                                     mc=self._slots[me][par].mc_endpoint(env))
        return tg

    def _plan_common(self, t, g, fixed_thr, rounds=1, recv_args=None):
        env = self._env
        phases = []
        for _ in range(rounds):
            self._step += 1
            seq, par = self._step, self._step & 1

            def send(seq=seq, par=par):
                if env.ranks == 1 and not self.consistent:
                    return
                if fixed_thr is None:
                    self._comp.threshold_topk(g, self.rests, self.size, self.compression_ratio, self._subsamples,
                                              self._sample_factor)
                else:
                    self._comp.set_threshold(fixed_thr)
                self._comp.compress(g, self.rests, self.size, self.cap, seq, self._send_targets(par))

            def recv(seq=seq, par=par, first=(_ == 0)):
                order = self._order()
                if not order:
                    return
                src = self._cached_sources(("src", par), lambda: [self._slots[j][par].endpoint(env) for j in order],
                                           seq)
                if recv_args is not None:
                    # fused averaging + parameter update instead of a dense result; ``True``
                    # means "whatever the owner sets in _recv_args_now before this phase runs"
                    args = self._recv_args_now if recv_args is True else recv_args
                else:
                    args = P.args_set(t) if (self.consistent and first) else P.args_add(t)
                P.apply_sparse(env, src, self.size, args, self._status)
            phases += [send, recv]
        return phases

    def _plan_apply(self, t, recv_args=None):
        return self._plan_common(t, t, None, recv_args=recv_args)

    # ---- pre-built launch sequences: one native call for the send half, one for the receive half
    def _seqs(self, par):
        cache = self.__dict__.setdefault("_seq_cache", {})
        got = cache.get(par)
        if got is None:
            env, comp = self._env, self._comp
            thr, cmp_, app = _lib.Op(), _lib.Op(), _lib.Op()
            thr.kind, cmp_.kind, app.kind = _lib.OPK_THRESHOLD, _lib.OPK_COMPRESS, _lib.OPK_APPLY
            for op in (thr, cmp_, app):
                op.dev, op.n = env.dev, self.size
            thr.r = cmp_.r = self.rests.data_ptr()
            thr.thr = cmp_.thr = comp.thr.data_ptr()
            thr.default_subsamples, thr.subsample_factor = self._subsamples, self._sample_factor
            thr.workspace, thr.ws_bytes = comp.thr_ws.data_ptr(), comp.thr_ws_bytes
            cmp_.cap, cmp_.src_rank = self.cap, env.rank
            cmp_.workspace, cmp_.ws_bytes, cmp_.stats = comp.workspace.data_ptr(), comp.ws_bytes, comp.stats.dev_ptr
            cmp_.tg = self._send_targets(par)
            order = self._order()
            app.src = P.make_sources([self._slots[j][par].endpoint(env) for j in order], [0] * len(order))
            app.status, app.timeout_ns = self._status.dev_ptr, env.timeout_ns
            got = cache[par] = (_OpSeq(env, [thr, cmp_]), _OpSeq(env, [app]))
        return got

    def send_fast(self, g: torch.Tensor):
        """Threshold + compress of ``g`` with one native call; returns (seq, parity) for recv_fast."""
        self._step += 1
        seq, par = self._step, self._step & 1
        if self._env.ranks == 1 and not self.consistent:
            return seq, par
        send, _ = self._seqs(par)
        code, ptr = _lib.dtype_code(g.dtype), g.data_ptr()
        thr, cmp_ = send.arr[0], send.arr[1]
        thr.g = cmp_.g = ptr
        thr.dtype = cmp_.dtype = code
        thr.ratio = self.compression_ratio
        send.run(seq)
        return seq, par

    def recv_fast(self, seq: int, par: int, args) -> None:
        """Wait for all payloads of step ``seq`` and apply them with ``args`` (one native call)."""
        _, recv = self._seqs(par)
        if recv.arr[0].src.count == 0:
            return
        recv.arr[0].apply = args
        recv.run(seq)

    def apply(self, vector):
        if self._env._world is not None:      # virtual ranks are driven phase by phase
            return super().apply(vector)
        t, orig = self._prep(vector)
        seq, par = self.send_fast(t)
        self.recv_fast(seq, par, P.args_set(t) if self.consistent else P.args_add(t))
        self._env.maybe_check()
        write_back(t, orig)
        return vector

    __call__ = apply

    def _plan_flush(self, t):
        """Every rank sends its whole residual; ``vector`` gains the peers' (and, when
        consistent, is replaced by everyone's) residuals; residuals end up zero."""
        return self._plan_common(t, None, 0.0, rounds=self._flush_rounds(self.size, self.cap))


class Comprex_RingAllreduce(_ComprexAllreduceBase):
    """Compressed reduce-scatter to the chunk owners, compressed allgather back
    (src/allreduce.tpp:366-528).

    Rank r owns chunk (r+1) mod P and keeps it dense.  Each rank holds one
    residual per chunk it sends (kept as one full-length tensor).  The
    allgather sends top-k of the reduced chunk; with ``owner_residual=False``
    (reference behaviour, ``writeRemote_NoResidual``) the remainder is dropped,
    with ``True`` the owner accumulates it for the next call.
    """

    def setup_connections(self, size, tag=0, compression_ratio=0.01, size_factor=1.0, consistent=False,
                          owner_residual=False, schedule="direct", chunk_align=1):
        if schedule not in ("direct", "hops"):
            raise ComprexError("schedule must be 'direct' or 'hops'")
        if consistent and schedule != "direct":
            raise ComprexError("consistent=True needs the direct schedule")
        self._setup_compressed(size, compression_ratio, size_factor, consistent)
        env = self._env
        self.schedule = schedule
        # consistent: the owner, too, applies only what it broadcast, and keeps the rest of its
        # reduced chunk in a residual of its own (otherwise that rest would be lost for everyone)
        self.owner_residual = bool(owner_residual) or self.consistent
        owner_residual = self.owner_residual
        self.segment_sizes, self.segment_starts = _chunks(size, env.ranks, chunk_align)
        nmax = max(max(self.segment_sizes), 1)
        self.cap = _cap_for(nmax, size_factor)
        self._rs = [[P.SparseSlot.create(env, nmax, self.cap) for _ in range(2)] for _ in range(env.ranks)]
        self._ag = [[P.SparseSlot.create(env, nmax, self.cap) for _ in range(2)] for _ in range(env.ranks)]
        self._comp = P.Compressor(env, nmax)
        # one compressor (scratch, threshold cell) per chunk: the per-chunk compressions of the
        # reduce-scatter are independent and run concurrently when the call is replayed
        self._chunk_comps = [P.Compressor(env, nmax) for _ in range(env.ranks)]
        self.rests = torch.zeros(size, dtype=torch.float32, device=env.device)
        self.owner_rests = torch.zeros(nmax, dtype=torch.float32, device=env.device) if owner_residual else None
        if schedule == "hops":
            # the reference's neighbour-to-neighbour ring: one slot per hop and parity in each phase
            hops = max(env.ranks - 1, 1)
            self._hop_rs = [[P.SparseSlot.create(env, nmax, self.cap) for _ in range(2)] for _ in range(hops)]
            self._hop_ag = [[P.SparseSlot.create(env, nmax, self.cap) for _ in range(2)] for _ in range(hops)]
            self._replay = False     # the forwarding launches are not part of recorded sequences

    def _residuals(self):
        return [self.rests] + ([self.owner_rests] if self.owner_rests is not None else [])

    def _plan_hops(self, t):
        """The reference's schedule hop by hop (src/allreduce.tpp:420-457): P-1 reduce steps in
        which every rank sends top-k of (chunk + that chunk's residual) to its right neighbour and
        adds what arrives from the left, so partial sums are compressed again at every hop; then
        the owner's top-k of the reduced chunk travels P-1 hops, forwarded unchanged.  On an
        NVSwitch this costs 2(P-1) dependent exchanges where ``direct`` needs two; it is kept for
        studies that need the reference's exact error behaviour."""
        env, me, nr = self._env, self._env.rank, self._env.ranks
        self._step += 1
        seq, par = self._step, self._step & 1
        if nr == 1:
            return []
        right = (me + 1) % nr
        phases = []
        for it in range(nr - 1):
            sc, rc = (me - it) % nr, (me - it - 1) % nr

            def send(it=it, sc=sc):
                g, r, n = self._view(t, sc), self._view(self.rests, sc), self.segment_sizes[sc]
                self._comp.threshold_topk(g, r, n, self.compression_ratio, self._subsamples, self._sample_factor)
                self._comp.compress(g, r, n, self.cap, seq,
                                    P.make_targets([self._hop_rs[it][par].endpoint(env, right)]))

            def recv(it=it, rc=rc):
                src = P.make_sources([self._hop_rs[it][par].endpoint(env)], [seq])
                P.apply_sparse(env, src, self.segment_sizes[rc], P.args_add(self._view(t, rc)), self._status)
            phases += [send, recv]

        def gather_send():
            c = (me + 1) % nr
            n, mv = self.segment_sizes[c], self._view(t, c)
            r = self.owner_rests[:n] if self.owner_rests is not None else None
            self._comp.threshold_topk(mv, r, n, self.compression_ratio)
            self._comp.compress(mv, r, n, self.cap, seq, P.make_targets([self._hop_ag[0][par].endpoint(env, right)]))
        phases.append(gather_send)
        for it in range(nr - 2):
            def fwd(it=it, rc=(me - it) % nr):
                ep = self._hop_ag[it][par].endpoint(env)
                P.forward(env, ep, seq, P.make_targets([self._hop_ag[it + 1][par].endpoint(env, right)]), seq,
                          self.cap, self._counters, self._status)
                P.apply_sparse(env, P.make_sources([ep], [seq]), self.segment_sizes[rc],
                               P.args_set(self._view(t, rc)), self._status)
            phases.append(fwd)

        def last(rc=(me + 2) % nr):
            src = P.make_sources([self._hop_ag[nr - 2][par].endpoint(env)], [seq])
            P.apply_sparse(env, src, self.segment_sizes[rc], P.args_set(self._view(t, rc)), self._status)
        phases.append(last)
        return phases

    def _owner(self, chunk):
        return (chunk - 1) % self._env.ranks

    def _view(self, t, c):
        return t[self.segment_starts[c]: self.segment_starts[c] + self.segment_sizes[c]]

    def _plan_ring(self, t, flush, rounds=1, final_args=None, fixed=None):
        """Phases of one call.  ``final_args(chunk)`` replaces the plain decode of the allgather
        (``SET`` into the chunk's part of ``t``) by another receive operation, e.g. a fused
        parameter update; ``fixed=(seq, parity)`` plans for that step instead of the next one."""
        env, me, nr = self._env, self._env.rank, self._env.ranks
        mine = (me + 1) % nr
        # chunk order starts behind this rank's own chunk: at any moment every rank addresses a
        # different owner instead of all ranks storing into the same receiver
        others = [(mine + k) % nr for k in range(1, nr)]
        peers = [r for r in range(nr) if r != me]
        everyone = list(range(nr))
        phases = []
        for rnd in range(rounds):
            if fixed is None:
                self._step += 1
                seq, par = self._step, self._step & 1
            else:
                seq, par = fixed

            def scatter(seq=seq, par=par):
                for k, c in enumerate(others):
                    n = self.segment_sizes[c]
                    g, r = (None if flush else self._view(t, c)), self._view(self.rests, c)
                    comp = self._chunk_comps[c]
                    with P.lane(env, k + 1):
                        if flush:
                            comp.set_threshold(0.0)
                        else:
                            comp.threshold_topk(g, r, n, self.compression_ratio, self._subsamples, self._sample_factor)
                        comp.compress(g, r, n, self.cap, seq,
                                      P.make_targets([self._rs[me][par].endpoint(env, self._owner(c))]))

            def reduce(seq=seq, par=par, last=(rnd == rounds - 1)):
                if nr == 1 and not self.consistent:
                    return
                n = self.segment_sizes[mine]
                mv = self._view(t, mine)
                if peers:
                    src = P.make_sources([self._rs[j][par].endpoint(env) for j in peers], [seq] * len(peers))
                    P.apply_sparse(env, src, n, P.args_add(mv), self._status)
                if flush and not last:
                    return  # more residual rounds follow; broadcast once at the end
                r = self.owner_rests[:n] if self.owner_rests is not None else None
                if flush:
                    self._comp.set_threshold(0.0)      # the owner's own residual is drained too
                else:
                    self._comp.threshold_topk(mv, r, n, self.compression_ratio)
                dests = everyone if self.consistent else peers
                self._comp.compress(mv, r, n, self.cap, seq,
                                    P.make_targets([self._ag[me][par].endpoint(env, j) for j in dests],
                                                   mc=self._ag[me][par].mc_endpoint(env)))

            def gather(seq=seq, par=par, last=(rnd == rounds - 1)):
                if flush and not last:
                    return
                for k, j in enumerate(everyone if self.consistent else peers):
                    c = (j + 1) % nr
                    src = P.make_sources([self._ag[j][par].endpoint(env)], [seq])
                    args = final_args(c) if final_args is not None else P.args_set(self._view(t, c))
                    with P.lane(env, k + 1):     # the chunks are disjoint: decode them side by side
                        P.apply_sparse(env, src, self.segment_sizes[c], args, self._status)
            phases += [scatter, reduce, gather]
        return phases

    # ---- pre-built launch sequences for the optimizer: a send half and a receive half ---------
    def _fast_seqs(self, t, par):
        cache = self.__dict__.setdefault("_fast_cache", {})
        key = (t.data_ptr(), par)
        got = cache.get(key)
        if got is None:
            env = self._env
            if len(cache) >= 16:
                cache.clear()
            patch = []                      # (index into the receive list, chunk) of the final decodes

            def placeholder(c):
                patch.append((len(env._rec), c))
                return P.args_set(self._view(t, c))
            plan = self._plan_ring(t, False, final_args=placeholder, fixed=(0, par))
            env._rec = send_rec = []
            try:
                plan[0]()
                env._rec = recv_rec = []
                plan[1]()
                plan[2]()
            finally:
                env._rec = None
            got = cache[key] = (_OpSeq(env, send_rec) if send_rec else None,
                                _OpSeq(env, recv_rec) if recv_rec else None, patch)
        return got

    def send_fast(self, t: torch.Tensor):
        """First half of a call on ``t`` (float32, this allreduce's size; it is used as work space):
        every foreign chunk is compressed into its owner's slot.  One native call; returns
        (seq, parity) for :meth:`recv_fast`."""
        self._step += 1
        seq, par = self._step, self._step & 1
        send, _, _ = self._fast_seqs(t, par)
        if send is not None:
            send.run(seq)
        return seq, par

    def recv_fast(self, t: torch.Tensor, seq: int, par: int, args_of_chunk=None) -> None:
        """Second half: reduce the own chunk, broadcast its top-k, decode every chunk.
        ``args_of_chunk(chunk, start, size)`` returns the receive operation for a chunk (a fused
        parameter update, say); the default writes the chunk into ``t``."""
        _, recv, patch = self._fast_seqs(t, par)
        if recv is None:
            return
        if args_of_chunk is not None:
            for i, c in patch:
                recv.arr[i].apply = args_of_chunk(c, self.segment_starts[c], self.segment_sizes[c])
        recv.run(seq)

    def _plan_apply(self, t):
        if self.schedule == "hops":
            return self._plan_hops(t)
        return self._plan_ring(t, flush=False)

    def _plan_flush(self, t):
        """Owners receive all residuals of their chunk uncompressed-by-threshold and
        everyone ends with the owners' exact chunks (src/allreduce.tpp:459-508).  When the
        slots are smaller than a full chunk, the last allgather carries the top ``cap``
        entries by index only; size the slots with ``size_factor > 2`` for an exact flush."""
        plan = self._plan_ring(t, flush=True, rounds=self._flush_rounds(max(self.segment_sizes), self.cap))
        return plan + [self.reset]


class Comprex_AllToOneAllreduce(_ComprexAllreduceBase):
    """Compressed gather to a chief and compressed broadcast back
    (src/allreduce.tpp:133-258).

    The chief accumulates densely; the broadcast has its own residual so that
    what the chief's sum loses to the threshold is sent later.  Workers'
    vectors are overwritten with the sparse broadcast.  The reference sends
    both legs one call late (FastComprEx double buffering, src/comprEx.tpp:428-448);
    here both legs are fresh by default and ``stale=True`` reproduces the
    reference: every call first forwards the payload compressed during the
    previous call (an empty one the first time) and then compresses the current
    input into a local staging slot.
    ``flush`` drains the workers' residuals (and their staged payloads) into the
    chief and does not broadcast, like the reference.
    """

    def setup_connections(self, size, tag=0, chiefRank=0, compression_ratio=0.01, size_factor=1.0, stale=False):
        self._setup_compressed(size, compression_ratio, size_factor, False)
        env = self._env
        self.chiefRank = int(chiefRank)
        self.stale = bool(stale)
        self._subsamples, self._sample_factor = 1000, 10.0  # default sampling (src/allreduce.tpp:142)
        self.cap = _cap_for(size, size_factor)
        self._rs = [[P.SparseSlot.create(env, size, self.cap) for _ in range(2)] for _ in range(env.ranks)]
        self._bc = [P.SparseSlot.create(env, size, self.cap) for _ in range(2)]
        self._comp = P.Compressor(env, size)
        self.rests = torch.zeros(size, dtype=torch.float32, device=env.device)
        if self.stale:
            self._stage = [P.SparseSlot.create(env, size, self.cap) for _ in range(2)]   # local staging
            self._stage_seq, self._first = 0, True
            self._replay = False        # forwarding is not part of recorded sequences

    def _residuals(self):
        return [self.rests]

    def reset(self):
        super().reset()
        if self.stale:
            self._first = True

    # ---- one-call-late mode -------------------------------------------------------------------
    def _send_pending(self, targets, seq) -> None:
        """Forward what the previous call staged; an empty payload on the first call."""
        env = self._env
        if self._first:
            self._comp.set_threshold(3.0e38)                 # nothing passes, the residual is untouched
            self._comp.compress(None, self.rests, self.size, self.cap, seq, targets)
            self._first = False
        else:
            ep = self._stage[self._stage_seq & 1].endpoint(env)
            P.forward(env, ep, self._stage_seq, targets, seq, self.cap, self._counters, self._status)

    def _stage_new(self, t) -> None:
        env = self._env
        self._stage_seq += 1
        self._comp.threshold_topk(t, self.rests, self.size, self.compression_ratio, self._subsamples,
                                  self._sample_factor)
        self._comp.compress(t, self.rests, self.size, self.cap, self._stage_seq,
                            P.make_targets([self._stage[self._stage_seq & 1].endpoint(env)]))

    def _plan_stale(self, t):
        env, me, chief = self._env, self._env.rank, self.chiefRank
        workers = [r for r in range(env.ranks) if r != chief]
        self._step += 1
        seq, par = self._step, self._step & 1

        def send():
            if me != chief:
                self._send_pending(P.make_targets([self._rs[me][par].endpoint(env, chief)]), seq)
                self._stage_new(t)

        def reduce():
            if me != chief or not workers:
                return
            src = P.make_sources([self._rs[w][par].endpoint(env) for w in workers], [seq] * len(workers))
            P.apply_sparse(env, src, self.size, P.args_add(t), self._status)
            self._send_pending(P.make_targets([self._bc[par].endpoint(env, w) for w in workers]), seq)
            self._stage_new(t)

        def recv():
            if me != chief:
                P.apply_sparse(env, P.make_sources([self._bc[par].endpoint(env)], [seq]), self.size,
                               P.args_set(t), self._status)
        return [send, reduce, recv]

    def _fold_pending(self):
        """Before a flush: a worker's staged payload goes back into its residual; the chief's
        staged broadcast is dropped with its residual (the reference resets it)."""
        env = self._env
        if self.stale and not self._first and env.rank != self.chiefRank:
            ep = self._stage[self._stage_seq & 1].endpoint(env)
            P.apply_sparse(env, P.make_sources([ep], [self._stage_seq]), self.size, P.args_add(self.rests),
                           self._status)
        if self.stale:
            self._first = True

    def _plan_common(self, t, flush, rounds=1):
        env, me, chief = self._env, self._env.rank, self.chiefRank
        workers = [r for r in range(env.ranks) if r != chief]
        phases = []
        for _ in range(rounds):
            self._step += 1
            seq, par = self._step, self._step & 1

            def send(seq=seq, par=par):
                if me == chief:
                    return
                if flush:
                    self._comp.set_threshold(0.0)
                else:
                    self._comp.threshold_topk(t, self.rests, self.size, self.compression_ratio,
                                              self._subsamples, self._sample_factor)
                self._comp.compress(None if flush else t, self.rests, self.size, self.cap, seq,
                                    P.make_targets([self._rs[me][par].endpoint(env, chief)]))

            def reduce(seq=seq, par=par):
                if me != chief or not workers:
                    return
                src = P.make_sources([self._rs[w][par].endpoint(env) for w in workers], [seq] * len(workers))
                P.apply_sparse(env, src, self.size, P.args_add(t), self._status)
                if flush:
                    return
                self._comp.threshold_topk(t, self.rests, self.size, self.compression_ratio,
                                          self._subsamples, self._sample_factor)
                self._comp.compress(t, self.rests, self.size, self.cap, seq,
                                    P.make_targets([self._bc[par].endpoint(env, w) for w in workers],
                                                   mc=self._bc[par].mc_endpoint(env)))

            def recv(seq=seq, par=par):
                if me == chief or flush:
                    return
                P.apply_sparse(env, P.make_sources([self._bc[par].endpoint(env)], [seq]), self.size,
                               P.args_set(t), self._status)
            phases += [send, reduce, recv]
        return phases

    def _plan_apply(self, t):
        if self.stale:
            return self._plan_stale(t)
        return self._plan_common(t, flush=False)

    def _plan_flush(self, t):
        return ([self._fold_pending] + self._plan_common(t, True, rounds=self._flush_rounds(self.size, self.cap))
                + [self.reset])


# =====================================================================================
# choice of schedule by size, ratio and number of ranks
# =====================================================================================
# Cost model behind ``select_schedule``: time = launch floor + bytes through HBM / HBM rate + bytes
# into this GPU's port / link rate + pairs decoded x time per pair, with the rates this package's
# kernels reach on 2-8 B200 behind an NVSwitch (bench/allreduce_sweep.py; microseconds, bytes per
# microsecond).  The model ranks the schedules; its absolute times run ~15 % high for large vectors
# because the phases overlap.
_COST = {
    "floor_dense_us": 30.0,      # dense one-shot: two launches
    "floor_two_shot_us": 50.0,   # dense reduce-scatter + allgather / through the switch
    "floor_bigring_us": 40.0,    # threshold + compress + decode
    "floor_ring_us": 44.0,       # 3 P launches on side streams (one graph), two dependent exchanges,
    "floor_ring_per_rank_us": 4.5,   # ... plus this per rank (55-85 us measured on 2 / 4 / 8 GPUs)
    "ring_stream": 0.9,          # the Ring's chunk kernels overlap on side streams and its decode writes
                                 # only the other ranks' chunks: less streaming time than the BigRing's passes
    "hbm_bpus": 6.0e6,           # streaming kernels
    "link_bpus": 5.5e5,          # into one GPU's port: peer stores and multicast stores alike
    "dense_link_bpus": 7.5e5,    # dense allreduce of a vector outside the heap (staging copies included)
    "pair_us": 4.0e-6,           # decode of one (index, value) pair
}


def schedule_costs(n: int, ratio: float, ranks: int, elem_bytes: int = 4) -> dict:
    """Modelled microseconds of the three schedules ``select_schedule`` chooses from."""
    c, p = _COST, max(int(ranks), 1)
    nb = n * elem_bytes
    pairs = ratio * n                                         # pairs of one rank's payload
    wire = 8.0 * pairs + 8.0 * n / 1024                       # its bytes: pairs + table
    one_shot = nb <= (1 << 20) or p <= 2
    dense = ((c["floor_dense_us"] + (p - 1) * nb / c["link_bpus"]) if one_shot else
             (c["floor_two_shot_us"] + 2.0 * (p - 1) / p * nb / c["dense_link_bpus"])) + 3.0 * nb / c["hbm_bpus"]
    bigring = (c["floor_bigring_us"] + (8.0 + elem_bytes) * n / c["hbm_bpus"] + (p - 1) * wire / c["link_bpus"]
               + p * pairs * c["pair_us"] + nb / c["hbm_bpus"])
    ring = (c["floor_ring_us"] + c["floor_ring_per_rank_us"] * p
            + c["ring_stream"] * ((8.0 + elem_bytes) * n + nb) / c["hbm_bpus"]
            + 2.0 * (p - 1) / p * wire / c["link_bpus"] + (2.0 * p - 1) / p * pairs * c["pair_us"])
    return {"bigring": dense, "comprex_bigring": bigring, "comprex_ring": ring}


def select_schedule(n: int, ratio: float, ranks: int, elem_bytes: int = 4) -> str:
    """``"bigring"`` (dense P2P kernels), ``"comprex_bigring"`` or ``"comprex_ring"``: the schedule
    with the lowest modelled time for a vector of ``n`` elements at top-k ``ratio`` on ``ranks``
    GPUs.  Tiny vectors are latency bound and go dense; a compressed BigRing pays (P-1) copies of
    the payload and wins while the payload is small; the compressed Ring moves 2 (P-1)/P payloads
    through two dependent exchanges and wins for large vectors and high ratios."""
    if ranks <= 1:
        return "comprex_bigring"
    if ratio >= 1.0:
        return "bigring"
    costs = schedule_costs(n, ratio, ranks, elem_bytes)
    return min(costs, key=costs.get)


class AutoAllreduce(_AllreduceBase):
    """The allreduce that ``select_schedule`` picks for (size, ratio, ranks), behind the common
    surface (``apply``, ``flush``, ``reset``, ``set_compression_ratio``, ``stats``,
    ``state_dict``).  ``choice`` names the schedule that was set up.  The compressed schedules are
    set up replica-consistent (``consistent=True``) unless told otherwise."""

    def setup_connections(self, size, tag=0, compression_ratio=0.01, size_factor=1.0, consistent=True,
                          dtype=torch.float32):
        env = self._env
        es = torch.empty(0, dtype=dtype).element_size()
        self.choice = select_schedule(int(size), float(compression_ratio), env.ranks, es)
        self.size, self.dtype = int(size), dtype
        if self.choice == "bigring":
            self.impl = BigRingAllreduce(self.gaspi_env)
            self.impl.setup_connections(size, tag, dtype=dtype, ordered=consistent)
        elif self.choice == "comprex_bigring":
            self.impl = Comprex_BigRingAllreduce(self.gaspi_env)
            self.impl.setup_connections(size, tag, compression_ratio, size_factor, consistent=consistent)
        else:
            self.impl = Comprex_RingAllreduce(self.gaspi_env)
            self.impl.setup_connections(size, tag, compression_ratio, size_factor, consistent=consistent,
                                        chunk_align=4)
        self.compressed = self.impl.compressed

    def apply(self, vector):
        return self.impl.apply(vector)

    __call__ = apply

    def flush(self, vector):
        return self.impl.flush(vector) if self.impl.compressed else vector

    def reset(self):
        if self.impl.compressed:
            self.impl.reset()

    def set_compression_ratio(self, compression_ratio):
        """Changes top-k of the schedule that was chosen at set-up (the choice itself is kept:
        slots and residuals belong to it)."""
        if self.impl.compressed:
            self.impl.set_compression_ratio(compression_ratio)

    def stats(self):
        return self.impl.stats() if self.impl.compressed else {}

    def state_dict(self):
        return {"choice": self.choice, "impl": self.impl.state_dict() if self.impl.compressed else None}

    def load_state_dict(self, state):
        if state["choice"] != self.choice:
            raise ComprexError("state_dict belongs to another schedule")
        if state["impl"] is not None:
            self.impl.load_state_dict(state["impl"])
