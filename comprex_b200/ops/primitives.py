"""Python face of the native primitives: slots, thresholds, compress, apply, dense.

Each function is a thin, allocation-free launch wrapper: it packs tensor
addresses into the C structs of csrc/cx_common.h and calls the exported
function on the current stream of the tensor's device (or synchronously for
host tensors).  Which reference routine each primitive replaces is stated in
the corresponding ``.cu`` file.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import torch

from .. import _lib
from .._lib import ApplyArgs, ComprexError, Endpoint, Sources, Targets
from ..parallel.env import GaspiEnvironment, SymmAlloc

HEADER_BYTES = 64


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass(frozen=True)
class SparseSlot:
    """Receive slot for an IndexPairs payload of a vector of up to ``n`` elements."""
    alloc: SymmAlloc
    n: int
    cap: int

    @staticmethod
    def nbytes(n: int, cap: int) -> int:
        nsub = (n + _lib.SUBTILE - 1) // _lib.SUBTILE
        return HEADER_BYTES + _round_up(8 * max(nsub, 1), 16) + 8 * max(cap, 1)

    @staticmethod
    def create(env: GaspiEnvironment, n: int, cap: int) -> "SparseSlot":
        return SparseSlot(env.alloc(SparseSlot.nbytes(n, cap)), n, cap)

    def endpoint(self, env: GaspiEnvironment, rank: int | None = None) -> Endpoint:
        base = env.ptr(self.alloc, rank)
        nsub = (self.n + _lib.SUBTILE - 1) // _lib.SUBTILE
        ep = Endpoint(base, base + HEADER_BYTES, base + HEADER_BYTES + _round_up(8 * max(nsub, 1), 16))
        ep.cap = self.cap   # travels to make_sources: receivers never read beyond their slot
        return ep

    def mc_endpoint(self, env: GaspiEnvironment):
        """The slot through the multicast mapping (a store there lands in every rank's copy of the
        slot), or None where the heap has none."""
        base = env.mc_ptr(self.alloc)
        if not base:
            return None
        nsub = (self.n + _lib.SUBTILE - 1) // _lib.SUBTILE
        return Endpoint(base, base + HEADER_BYTES, base + HEADER_BYTES + _round_up(8 * max(nsub, 1), 16))


@dataclass(frozen=True)
class DenseSlot:
    """Receive slot for a dense payload of up to ``nbytes_data`` bytes."""
    alloc: SymmAlloc
    nbytes_data: int

    @staticmethod
    def create(env: GaspiEnvironment, nbytes_data: int) -> "DenseSlot":
        return DenseSlot(env.alloc(HEADER_BYTES + _round_up(max(nbytes_data, 16), 16)), nbytes_data)

    def endpoint(self, env: GaspiEnvironment, rank: int | None = None) -> Endpoint:
        base = env.ptr(self.alloc, rank)
        return Endpoint(base, 0, base + HEADER_BYTES)

    def mc_endpoint(self, env: GaspiEnvironment):
        base = env.mc_ptr(self.alloc)
        return Endpoint(base, 0, base + HEADER_BYTES) if base else None


def make_targets(eps, mc=None) -> Targets:
    """Target descriptor.  ``mc`` is the multicast endpoint of the targets' slot (the same block on
    every rank): payload data then goes out once through the switch instead of once per target.
    It is only used for two or more targets (with one target a plain store moves the same bytes)."""
    eps = list(eps)
    if len(eps) > _lib.MAX_PEERS:
        raise ComprexError("too many targets")
    t = Targets()
    t.count = len(eps)
    for i, e in enumerate(eps):
        t.ep[i] = e
    if mc is not None and 2 <= len(eps) < _lib.MAX_PEERS:
        t.pad = _lib.TG_MULTICAST
        t.ep[len(eps)] = mc
    return t


def make_sources(eps, seqs, own_pos: int = 0) -> Sources:
    """Source descriptor.  ``own_pos``: dense reduce only, where the own vector enters the sum
    (0 = first; with the sources in rank order and ``own_pos`` = this rank all ranks add alike)."""
    eps = list(eps)
    if len(eps) > _lib.MAX_PEERS:
        raise ComprexError("too many sources")
    s = Sources()
    s.count = len(eps)
    s.pad = int(own_pos)
    for i, (e, q) in enumerate(zip(eps, seqs)):
        s.ep[i] = e
        s.seq[i] = q
        s.cap[i] = getattr(e, "cap", 0)
    return s


def _ptr(t: torch.Tensor | None) -> int:
    return 0 if t is None else t.data_ptr()


def _recording(env) -> bool:
    """True while a launch sequence is being recorded instead of launched (see
    ``allreduce._AllreduceBase.apply``): the wrappers below then append a CxOp to
    ``env._rec`` and launch nothing."""
    return getattr(env, "_rec", None) is not None


def _new_op(env, kind: int, dtype: int, n: int):
    op = _lib.Op()
    op.kind, op.dev, op.dtype, op.n = kind, env.dev, dtype, n
    op.lane = getattr(env, "_lane", 0)      # side stream of the recorded sequence (see ``lane``)
    return op


class lane:
    """``with lane(env, k):`` - launches recorded inside run on side stream ``k`` of the replayed
    sequence (concurrently with the other lanes, joined before the next lane-0 launch).  Outside a
    recording the launches simply go to the current stream."""

    def __init__(self, env, k: int):
        self.env, self.k = env, int(k)

    def __enter__(self):
        self.prev = getattr(self.env, "_lane", 0)
        self.env._lane = self.k
        return self

    def __exit__(self, *exc):
        self.env._lane = self.prev


def _set_ranges(op, ranges) -> None:
    if ranges is None:
        return
    if len(ranges) > _lib.MAX_PEERS:
        raise ComprexError("too many ranges")
    op.has_ranges = 1
    for i, (a, k) in enumerate(ranges):
        op.starts[i], op.lens[i] = a, k


def _flat(t: torch.Tensor, what: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise ComprexError(f"{what} must be contiguous")
    return t


def compress_regions(n: int, cap: int):
    """(regions, pairs per region) the compress kernel uses for a vector of ``n`` elements and a
    slot of ``cap`` pairs (the rule of ``cx_compress``: at least 8 sub-tiles and 256 pairs per
    region, at most 32 regions, a power of two)."""
    nsub = (n + _lib.SUBTILE - 1) // _lib.SUBTILE
    regions = 1
    while regions < 32 and nsub // (2 * regions) >= 8 and cap // (2 * regions) >= 256:
        regions *= 2
    return regions, cap // regions


class Compressor:
    """Scratch, threshold cell and statistics of one sparse sender.

    The scratch (a 64-byte block of counters that the kernel resets itself)
    is rank-local device memory; the threshold lives in a one-element device
    tensor that the threshold kernel writes and the compress kernel reads.
    """

    def __init__(self, env: GaspiEnvironment, n: int):
        self.env, self.n = env, n
        self.ws_bytes = int(env.lib.cx_workspace_bytes(n))
        self.workspace = env.scratch(self.ws_bytes)
        self.thr = torch.zeros(1, dtype=torch.float32, device=env.device)
        self.thr_ws_bytes = int(env.lib.cx_threshold_workspace_bytes())    # exact selection: grid-wide histograms
        self.thr_ws = env.scratch(self.thr_ws_bytes)
        self.stats = env.new_stats()

    def set_threshold(self, value: float) -> None:
        if _recording(self.env):
            raise ComprexError("a constant threshold cannot be part of a recorded launch sequence")
        self.thr.fill_(float(value))

    def threshold_topk(self, g, r, n: int, ratio: float, default_subsamples: int = 1000,
                       subsample_factor: float = 10.0) -> None:
        env = self.env
        gd = _lib.dtype_code(g.dtype) if g is not None else _lib.F32
        if _recording(env):
            op = _new_op(env, _lib.OPK_THRESHOLD, gd, n)
            op.g, op.r, op.thr, op.ratio = _ptr(g), _ptr(r), self.thr.data_ptr(), ratio
            op.default_subsamples, op.subsample_factor = int(default_subsamples), float(subsample_factor)
            op.workspace, op.ws_bytes = self.thr_ws.data_ptr(), self.thr_ws_bytes
            env._rec.append(op)
            return
        _lib.check(env.lib.cx_threshold_select(env.dev, gd, _ptr(g), _ptr(r), n, ratio, int(default_subsamples),
                                               float(subsample_factor), self.thr.data_ptr(), self.thr_ws.data_ptr(),
                                               self.thr_ws_bytes, _lib.stream_ptr(env.device)), "cx_threshold_select")

    def compress(self, g, r, n: int, cap: int, seq: int, targets: Targets) -> None:
        """r += g; emit |r| > thr into every target; zero what was emitted."""
        env = self.env
        if n > self.n:
            raise ComprexError(f"vector of {n} elements exceeds the compressor's size {self.n}")
        gd = _lib.dtype_code(g.dtype) if g is not None else _lib.F32
        if r is not None and r.dtype != torch.float32:
            raise ComprexError("the residual must be float32")
        if _recording(env):
            op = _new_op(env, _lib.OPK_COMPRESS, gd, n)
            op.g, op.r, op.thr, op.cap, op.src_rank = _ptr(g), _ptr(r), self.thr.data_ptr(), cap, env.rank
            op.workspace, op.ws_bytes, op.stats, op.tg = self.workspace.data_ptr(), self.ws_bytes, self.stats.dev_ptr, targets
            env._rec.append(op)
            return
        _lib.check(env.lib.cx_compress(env.dev, gd, _ptr(g), _ptr(r), n, self.thr.data_ptr(), cap, seq,
                                       C.byref(targets), self.workspace.data_ptr(), self.ws_bytes,
                                       self.stats.dev_ptr, env.rank, _lib.stream_ptr(env.device)),
                   "cx_compress")

    def last_stats(self) -> dict:
        """Statistics of the most recent compress call (synchronises)."""
        self.env.flush()
        return self.stats.read()


class RleCodec:
    """Slots and scratch of one run-length coded connection (csrc/rle.cu): two receive slots
    sized for the worst case (collective allocation) plus one workspace per direction."""

    def __init__(self, env: GaspiEnvironment, n: int):
        self.env, self.n = env, n
        self.slot_bytes = int(env.lib.cx_rle_slot_bytes(n))
        self.ws_bytes = int(env.lib.cx_rle_workspace_bytes(n))
        self.slots = [DenseSlot.create(env, self.slot_bytes) for _ in range(2)]
        self.tx_ws = env.scratch(self.ws_bytes)
        self.rx_ws = env.scratch(self.ws_bytes)

    def send(self, g, r, thr_cell: torch.Tensor, seq: int, dest: int) -> None:
        """Encode ``r + g`` at the threshold in ``thr_cell`` into rank ``dest``'s slot."""
        env = self.env
        gd = _lib.dtype_code(g.dtype) if g is not None else _lib.F32
        tg = make_targets([self.slots[seq & 1].endpoint(env, dest)])
        _lib.check(env.lib.cx_rle_send(env.dev, gd, _ptr(g), _ptr(r), self.n, thr_cell.data_ptr(), self.slot_bytes,
                                       seq, C.byref(tg), self.tx_ws.data_ptr(), self.ws_bytes, env.rank,
                                       _lib.stream_ptr(env.device)), "cx_rle_send")

    def recv(self, out: torch.Tensor, seq: int, add: bool, status) -> None:
        """Wait for payload ``seq`` in the local slot and expand it into the float32 ``out``."""
        env = self.env
        if out.dtype != torch.float32 or out.numel() != self.n:
            raise ComprexError("RLE decode needs a float32 vector of the connection's size")
        ep = self.slots[seq & 1].endpoint(env)
        _lib.check(env.lib.cx_rle_recv(env.dev, C.byref(ep), seq, out.data_ptr(), self.n, int(add), self.slot_bytes,
                                       self.rx_ws.data_ptr(), self.ws_bytes, status.dev_ptr, env.timeout_ns,
                                       _lib.stream_ptr(env.device)), "cx_rle_recv")


def apply_sparse(env: GaspiEnvironment, sources: Sources, n: int, args: ApplyArgs, status) -> None:
    if _recording(env):
        op = _new_op(env, _lib.OPK_APPLY, _lib.F32, n)
        op.src, op.apply, op.status, op.timeout_ns = sources, args, status.dev_ptr, env.timeout_ns
        env._rec.append(op)
        return
    _lib.check(env.lib.cx_apply(env.dev, C.byref(sources), n, C.byref(args), status.dev_ptr,
                                env.timeout_ns, _lib.stream_ptr(env.device)), "cx_apply")


def args_add(out: torch.Tensor, scale: float = 1.0) -> ApplyArgs:
    a = ApplyArgs()
    a.op, a.out, a.out_dtype, a.scale = _lib.OP_ADD, out.data_ptr(), _lib.dtype_code(out.dtype), scale
    return a


def args_set(out: torch.Tensor, scale: float = 1.0) -> ApplyArgs:
    a = ApplyArgs()
    a.op, a.out, a.out_dtype, a.scale = _lib.OP_SET, out.data_ptr(), _lib.dtype_code(out.dtype), scale
    return a


def args_update(op: int, w: torch.Tensor, scale: float, *, shadow=None, m=None, v=None, lr=0.0,
                momentum=0.0, beta1=0.9, beta2=0.999, eps=1e-8, wd=0.0, step=1) -> ApplyArgs:
    if w.dtype != torch.float32:
        raise ComprexError("master weights must be float32")
    a = ApplyArgs()
    a.op, a.out, a.out_dtype, a.scale = op, w.data_ptr(), _lib.F32, scale
    if shadow is not None:
        a.shadow, a.shadow_dtype = shadow.data_ptr(), _lib.dtype_code(shadow.dtype)
    a.m, a.v = _ptr(m), _ptr(v)
    a.lr, a.momentum, a.beta1, a.beta2, a.eps, a.wd = lr, momentum, beta1, beta2, eps, wd
    a.bc1 = 1.0 - beta1 ** step
    a.bc2 = 1.0 - beta2 ** step
    return a


def update_dense(env: GaspiEnvironment, g: torch.Tensor, n: int, args: ApplyArgs) -> None:
    """Parameter update from a dense averaged gradient ``g`` (float32): what follows a dense
    allreduce, and the whole step of a single rank (keras/comprex_optimizer.py:150-163)."""
    if g.dtype != torch.float32:
        raise ComprexError("the dense update reads a float32 vector")
    if _recording(env):
        op = _new_op(env, _lib.OPK_UPDATE, _lib.F32, n)
        op.g, op.apply = g.data_ptr(), args
        env._rec.append(op)
        return
    _lib.check(env.lib.cx_update_dense(env.dev, g.data_ptr(), n, C.byref(args), _lib.stream_ptr(env.device)),
               "cx_update_dense")


def forward(env: GaspiEnvironment, src: Endpoint, expect_seq: int, targets: Targets, seq: int, cap: int,
            counters: torch.Tensor, status) -> None:
    _lib.check(env.lib.cx_forward(env.dev, C.byref(src), expect_seq, C.byref(targets), seq, cap,
                                  counters.data_ptr(), status.dev_ptr, env.timeout_ns,
                                  _lib.stream_ptr(env.device)), "cx_forward")


def _ranges(ranges):
    if ranges is None:
        return None, None
    k = len(ranges)
    starts = (C.c_int64 * k)(*[r[0] for r in ranges])
    lens = (C.c_int64 * k)(*[r[1] for r in ranges])
    return starts, lens


def dense_send(env: GaspiEnvironment, g: torch.Tensor, r, n: int, seq: int, targets: Targets,
               counters: torch.Tensor, ranges=None) -> None:
    if _recording(env):
        op = _new_op(env, _lib.OPK_DENSE_SEND, _lib.dtype_code(g.dtype), n)
        op.g, op.r, op.tg, op.workspace, op.src_rank = g.data_ptr(), _ptr(r), targets, counters.data_ptr(), env.rank
        _set_ranges(op, ranges)
        env._rec.append(op)
        return
    starts, lens = _ranges(ranges)
    _lib.check(env.lib.cx_dense_send(env.dev, _lib.dtype_code(g.dtype), g.data_ptr(), _ptr(r), n, seq,
                                     C.byref(targets), starts, lens, counters.data_ptr(), env.rank,
                                     _lib.stream_ptr(env.device)), "cx_dense_send")


def dense_reduce(env: GaspiEnvironment, out: torch.Tensor, own, n: int, sources: Sources, status,
                 scale: float = 1.0, push: Targets | None = None, push_seq: int = 0,
                 counters: torch.Tensor | None = None, ranges=None) -> None:
    if _recording(env):
        op = _new_op(env, _lib.OPK_DENSE_REDUCE, _lib.dtype_code(out.dtype), n)
        op.out, op.own, op.src, op.scale = out.data_ptr(), _ptr(own), sources, scale
        op.workspace, op.src_rank, op.status, op.timeout_ns = _ptr(counters), env.rank, status.dev_ptr, env.timeout_ns
        if push is not None:
            op.has_push, op.tg = 1, push
        _set_ranges(op, ranges)
        env._rec.append(op)
        return
    starts, lens = _ranges(ranges)
    _lib.check(env.lib.cx_dense_reduce(env.dev, _lib.dtype_code(out.dtype), out.data_ptr(), _ptr(own), n,
                                       C.byref(sources), scale, C.byref(push) if push is not None else None,
                                       push_seq, starts, lens, _ptr(counters), env.rank, status.dev_ptr,
                                       env.timeout_ns, _lib.stream_ptr(env.device)), "cx_dense_reduce")


def axpy(env: GaspiEnvironment, y: torch.Tensor, x: torch.Tensor, a: float, n: int) -> None:
    _lib.check(env.lib.cx_axpy(env.dev, _lib.dtype_code(y.dtype), y.data_ptr(), _lib.dtype_code(x.dtype),
                               x.data_ptr(), a, n, _lib.stream_ptr(env.device)), "cx_axpy")


class MultimemAllreduce:
    """Staging block, flags and counters of one dense allreduce through the switch
    (csrc/nvls.cu: ``multimem.ld_reduce`` + ``multimem.st``, one kernel per rank and call).

    Construction is collective (symmetric allocations).  ``one_shot_bytes``: vectors up to that
    size are reduced by every rank itself in one exchange (double-buffered staging); larger ones
    use reduce-scatter + broadcast inside the switch, pipelined in slabs of ``slab_bytes``.  A
    vector that lives in the symmetric heap (``env.empty``) and is a multiple of 16 bytes is
    reduced in place, without the staging copies."""

    def __init__(self, env: GaspiEnvironment, size: int, dtype: torch.dtype, one_shot_bytes=None, slab_bytes=None):
        import os
        if not env.nvls:
            raise ComprexError("the heap has no multicast mapping")
        self.env, self.size, self.dtype = env, int(size), dtype
        es = torch.empty(0, dtype=dtype).element_size()
        nbytes = _round_up(max(self.size, 1) * es, 16)
        if one_shot_bytes is None:
            one_shot_bytes = int(os.environ.get("COMPREX_MM_ONE_SHOT_BYTES", 512 << 10))
        if slab_bytes is None:
            # a quarter of the vector, between 2 and 16 MiB: the pipeline of the staged form fills and
            # drains with one slab's copies, and every slab costs each group one arrival (measured on
            # 4 GPUs, fp32: 2^24 elements 218 us with 16 MiB slabs, 294 us with 32 MiB; 2^28 elements
            # 2702 / 2959 us; 8 MiB slabs 220 / 2952 us, 4 MiB slabs 249 / 3648 us)
            auto = min(16 << 20, max(2 << 20, (nbytes // 4) & ~((1 << 20) - 1)))
            slab_bytes = int(os.environ.get("COMPREX_MM_SLAB_BYTES", auto))
        self.one_shot = nbytes <= one_shot_bytes
        self.slab_bytes = int(slab_bytes)
        self.stride = _round_up(nbytes, 256)
        self.stage = env.alloc(self.stride * (2 if self.one_shot else 1), 256)
        self.flags = env.alloc(int(env.lib.cx_mm_flag_bytes()), 256)
        self.counters = env.scratch(int(env.lib.cx_mm_counter_bytes()))
        self._flag_list = [env.ptr(self.flags, r) for r in range(env.ranks)]
        self.flag_ptrs = (C.c_void_p * _lib.MAX_PEERS)(*(self._flag_list + [None] * (_lib.MAX_PEERS - env.ranks)))

    def run(self, t: torch.Tensor, seq: int, scale: float, status) -> None:
        """In-place allreduce of ``t`` (``scale`` times the sum, the same bits on every rank)."""
        env = self.env
        if t.dtype != self.dtype or t.numel() != self.size:
            raise ComprexError("vector does not match the allreduce")
        es = t.element_size()
        blk = env.heap_block(t)
        if blk is not None and not self.one_shot and (self.size * es) % 16 == 0 and env.mc_ptr(blk):
            out, src, stage, stage_mc, slab = 0, 0, env.ptr(blk), env.mc_ptr(blk), 0     # in place
        else:
            out, src, stage, stage_mc, slab = t.data_ptr(), t.data_ptr(), env.ptr(self.stage), env.mc_ptr(self.stage), self.slab_bytes
        if _recording(env):
            op = _new_op(env, _lib.OPK_MM_ALLREDUCE, _lib.dtype_code(t.dtype), self.size)
            op.out, op.own, op.g, op.r = out, src, stage, stage_mc
            op.starts[0], op.starts[1], op.starts[2] = self.stride, int(self.one_shot), slab
            for r, ptr in enumerate(self._flag_list):
                op.lens[r] = ptr
            op.src_rank, op.cap, op.workspace, op.scale = env.rank, env.ranks, self.counters.data_ptr(), scale
            op.status, op.timeout_ns = status.dev_ptr, env.timeout_ns
            env._rec.append(op)
            return
        _lib.check(env.lib.cx_mm_allreduce(_lib.dtype_code(t.dtype), out, src, stage, stage_mc, self.stride, self.size,
                                           env.rank, env.ranks, scale, int(self.one_shot), slab, seq, self.flag_ptrs,
                                           self.counters.data_ptr(), status.dev_ptr, env.timeout_ns,
                                           _lib.stream_ptr(env.device)), "cx_mm_allreduce")
