"""Runtime handle and symmetric heap.

``GaspiEnvironment`` plays the role of the reference's class of the same name
(include/gaspiEnvironment.hxx:9-28, src/gaspiEnvironment.tpp:15-43, gpi.py:147-174):
it knows rank and size, owns the communication segment, and offers ``barrier``
and ``flush``.  The segment here is a *symmetric heap*: every rank allocates
the same sequence of blocks, so a block is named by (segment, offset) and its
address on any peer is that peer's segment base plus the offset.  Peers' bases
come from

* CUDA IPC handles exchanged once per segment (one process per GPU; NVLink /
  NVSwitch peer access, the kernels then use plain loads and stores),
* POSIX shared memory for host ranks (CPU tensors, ``gloo``), or
* plain local allocations of a :class:`LoopbackWorld`, in which P virtual
  ranks live in one process on one device and phases of a collective are run
  rank after rank, so that no kernel ever waits for a kernel launched later.

Nothing on a hot path goes through this module: it hands out addresses at
set-up time, after that kernels talk to each other through the slots.
"""
from __future__ import annotations

import ctypes as C
import os
import socket
import uuid
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .. import _lib
from .._lib import ComprexError

_ALIGN = 256
_DEFAULT_SEGMENT = 64 << 20


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass(frozen=True)
class SymmAlloc:
    """A block that exists at the same (segment, offset) on every rank."""
    seg: int
    offset: int
    nbytes: int


class _RawCuda:
    """CUDA array interface over raw device memory, so that torch can wrap a heap block."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.owner = owner
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _tensor_at(ptr: int, n: int, dtype, device, owner) -> torch.Tensor:
    es = torch.empty(0, dtype=dtype).element_size()
    if device.type == "cuda":
        raw = torch.as_tensor(_RawCuda(ptr, max(n, 1) * es, owner), device=device)
    else:
        raw = torch.frombuffer((C.c_char * (max(n, 1) * es)).from_address(ptr), dtype=torch.uint8)
    return raw.view(dtype)[:n]


class _PinnedBlock:
    """Status words and statistics: host memory that kernels can write."""

    def __init__(self, lib, cuda: bool, nbytes: int = 1 << 16):
        self.lib, self.cuda, self.nbytes = lib, cuda, nbytes
        if cuda:
            dptr = C.c_void_p()
            self.host = lib.cx_pinned_alloc(nbytes, C.byref(dptr))
            if not self.host:
                raise ComprexError("pinned allocation failed: " + _lib.last_error())
            self.dev = dptr.value
        else:
            self.host = lib.cx_host_alloc(nbytes)
            self.dev = self.host
        self.used = 0

    def take(self, nbytes: int):
        nbytes = _round_up(nbytes, 32)
        if self.used + nbytes > self.nbytes:
            return None
        off = self.used
        self.used += nbytes
        return self.host + off, self.dev + off

    def close(self):
        if self.host:
            (self.lib.cx_pinned_free if self.cuda else self.lib.cx_host_free)(self.host)
            self.host = None


class StatusWord:
    """One uint32 a kernel ORs error bits into; read on the host after a sync."""

    def __init__(self, host_ptr: int, dev_ptr: int):
        self.dev_ptr = dev_ptr
        self._view = C.cast(host_ptr, C.POINTER(C.c_uint32))

    @property
    def value(self) -> int:
        return int(self._view[0])

    def clear(self) -> None:
        self._view[0] = 0


class StatsBlock:
    """CxStats of the last compress call of one compressor.

    The block lives in the memory of the device that runs the kernel (a write to mapped host
    memory would put a PCIe round trip on the tail of every compress launch); ``read`` copies
    it to the host."""

    def __init__(self, device):
        self._t = torch.zeros(C.sizeof(_lib.Stats), dtype=torch.uint8, device=device)
        self.dev_ptr = self._t.data_ptr()

    def read(self) -> dict:
        s = _lib.Stats.from_buffer_copy(bytes(self._t.cpu().numpy().tobytes()))
        return {"n": int(s.n), "nnz": int(s.nnz), "nnz_found": int(s.nnz_found),
                "status": int(s.status), "threshold": float(s.threshold)}


class GaspiEnvironment:
    """Rank, size, barrier, flush and the symmetric heap of one rank.

    Parameters
    ----------
    size : bytes of the first heap segment (the reference's ``segment_size``;
        more segments are added when needed).
    device : ``"cuda"``/``"cpu"``/``torch.device``; default CUDA when present.
    group : ``torch.distributed`` process group (default: the world group when
        ``torch.distributed`` is initialised, otherwise a single rank).
    timeout_ms : time budget of every device- or host-side wait.
    """

    def __init__(self, size: int = _DEFAULT_SEGMENT, device=None, group=None, timeout_ms=None,
                 _world=None, _rank=None):
        self.lib = _lib.load()
        self._world = _world
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:
            if _world is None and "LOCAL_RANK" in os.environ and dist.is_initialized():
                device = torch.device("cuda", int(os.environ["LOCAL_RANK"]) % torch.cuda.device_count())
            else:
                device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.dev = _lib.DEV_CUDA if device.type == "cuda" else _lib.DEV_HOST
        if self.dev == _lib.DEV_CUDA:
            torch.cuda.set_device(device)
        if _world is not None:
            self.rank, self.ranks, self.group = _rank, _world.size, None
        elif dist.is_available() and dist.is_initialized():
            self.group = group if group is not None else dist.group.WORLD
            self.rank, self.ranks = dist.get_rank(self.group), dist.get_world_size(self.group)
        else:
            self.group, self.rank, self.ranks = None, 0, 1
        if self.ranks > _lib.MAX_PEERS:
            raise ComprexError(f"at most {_lib.MAX_PEERS} ranks are supported, got {self.ranks}")
        if timeout_ms is None:
            timeout_ms = float(os.environ.get("COMPREX_TIMEOUT_MS", "20000"))
        self.timeout_ns = int(timeout_ms * 1e6)
        self.segment_size = max(int(size), 1 << 16)
        self._segments: list[dict] = []   # {"bases": [ptr per rank], "size", "used", "keep"}
        self._pinned: list[_PinnedBlock] = []
        self._status_words: list[tuple[StatusWord, str]] = []
        self._uid = None
        self._closed = False
        self._heap_tensors: dict[int, SymmAlloc] = {}
        self._bar = None
        self.sync_check = self.dev == _lib.DEV_HOST or os.environ.get("COMPREX_SYNC_CHECK", "0") == "1"
        # NVSwitch multicast (multimem stores / in-switch reduction): used where the heap can be
        # bound to a multicast object; COMPREX_NVLS=0 keeps every transfer on plain peer stores
        self.want_nvls = (self.dev == _lib.DEV_CUDA and _world is None and self.ranks > 1
                          and os.environ.get("COMPREX_NVLS", "1") != "0")

    # ---- reference surface (gpi.py:147-174) ---------------------------------
    def get_rank(self) -> int:
        return self.rank

    def get_ranks(self) -> int:
        return self.ranks

    def get(self):
        return self

    def get_segment(self):
        return self

    def barrier(self) -> None:
        """All ranks' earlier work is complete; raises pending kernel errors.

        Between real ranks this is the library's own barrier over the symmetric heap (one small
        kernel, or the host twin for CPU ranks: every rank stores the barrier's number into its
        cell on every peer and waits, bounded, for all of its own cells; csrc/nvls.cu); no
        ``torch.distributed`` collective is involved once the heap exists."""
        self.flush()
        if self._world is not None or self.group is None or self.ranks == 1:
            return
        if os.environ.get("COMPREX_DIST_BARRIER", "0") == "1":
            dist.barrier(group=self.group)
            return
        self._ensure_barrier()
        self._bar["seq"] += 1
        _lib.check(self.lib.cx_barrier(self.dev, self.rank, self.ranks, self._bar["ptrs"], self._bar["seq"],
                                       self._bar["status"].dev_ptr, self.timeout_ns, _lib.stream_ptr(self.device)),
                   "cx_barrier")
        self.flush()

    def _ensure_barrier(self) -> None:
        """Collective: the first barrier (or heap mark) allocates the barrier's flag block."""
        if self._bar is not None or self._world is not None or self.group is None or self.ranks == 1:
            return
        blk = self.alloc(8 * _lib.MAX_PEERS, 256)
        self._bar = {"ptrs": (C.c_void_p * _lib.MAX_PEERS)(*[self.ptr(blk, r) if r < self.ranks else None
                                                           for r in range(_lib.MAX_PEERS)]),
                     "seq": 0, "status": self.new_status("barrier")}
        dist.barrier(group=self.group)          # every rank's cells exist (and are zero) before the first store

    def flush(self) -> None:
        """Wait for this rank's queued work (src/gaspiEnvironment.tpp:37-39)."""
        if self.dev == _lib.DEV_CUDA:
            torch.cuda.current_stream(self.device).synchronize()
        self.check()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close(collective=False)
        except Exception:
            pass

    # ---- status ----------------------------------------------------------------
    def _pinned_take(self, nbytes: int):
        for blk in self._pinned:
            got = blk.take(nbytes)
            if got:
                return got
        blk = _PinnedBlock(self.lib, self.dev == _lib.DEV_CUDA)
        self._pinned.append(blk)
        return blk.take(nbytes)

    def new_status(self, owner: str = "") -> StatusWord:
        host, dev = self._pinned_take(32)
        word = StatusWord(host, dev)
        self._status_words.append((word, owner))
        return word

    def new_stats(self) -> StatsBlock:
        return StatsBlock(self.device)

    def check(self) -> None:
        """Turn status bits that kernels left behind into an exception."""
        bad = []
        for word, owner in self._status_words:
            v = word.value
            if v & ~_lib.ST_OVERFLOW:
                bad.append(f"{owner or 'op'}: {_lib.decode_status(v)}")
                word.clear()
        if bad:
            raise ComprexError(f"rank {self.rank}: " + "; ".join(bad))

    def maybe_check(self) -> None:
        if self.sync_check:
            if self.dev == _lib.DEV_CUDA:
                torch.cuda.current_stream(self.device).synchronize()
            self.check()

    # ---- heap ------------------------------------------------------------------
    def _exchange(self, obj):
        out = [None] * self.ranks
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def _new_segment(self, nbytes: int) -> None:
        nbytes = _round_up(max(nbytes, self.segment_size), 1 << 16)
        idx = len(self._segments)
        if self._world is not None:
            self._segments.append({"bases": self._world._segment_bases(idx, nbytes), "size": nbytes,
                                   "used": 0, "keep": None})
            return
        if self.ranks == 1:
            base = self.lib.cx_cuda_malloc(nbytes) if self.dev == _lib.DEV_CUDA else self.lib.cx_host_alloc(nbytes)
            if not base:
                raise ComprexError("segment allocation failed: " + _lib.last_error())
            self._segments.append({"bases": [base], "size": nbytes, "used": 0,
                                   "keep": ("local", base)})
            return
        if self.dev == _lib.DEV_CUDA:
            self._segments.append(self._new_cuda_segment(idx, nbytes))
        else:
            self._segments.append(self._new_shm_segment(idx, nbytes))

    def _new_cuda_segment(self, idx: int, nbytes: int) -> dict:
        hosts = self._exchange(socket.gethostname())
        if len(set(hosts)) != 1:
            raise ComprexError("all ranks of an environment must share one NVLink domain (one host)")
        mode = os.environ.get("COMPREX_HEAP", "symm" if self.want_nvls else "ipc")
        err = None
        if mode == "symm":
            seg = self._new_symm_segment(nbytes)
            if seg is not None:
                return seg
            mode = "ipc"
        if mode == "ipc":
            base = self.lib.cx_cuda_malloc(nbytes)
            handle = (C.c_char * 64)()
            ok = bool(base) and self.lib.cx_cuda_ipc_get(base, handle) == 0
            handles = self._exchange(bytes(handle) if ok else None)
            if all(h is not None for h in handles):
                bases, opened = [], []
                for r, h in enumerate(handles):
                    if r == self.rank:
                        bases.append(base)
                        continue
                    p = self.lib.cx_cuda_ipc_open(C.c_char_p(h))
                    if not p:
                        err = _lib.last_error()
                        break
                    bases.append(p)
                    opened.append(p)
                all_ok = all(self._exchange(err is None))
                if all_ok:
                    return {"bases": bases, "size": nbytes, "used": 0, "keep": ("ipc", base, opened)}
                for p in opened:
                    self.lib.cx_cuda_ipc_close(p)
            if base:
                self.lib.cx_cuda_free(base)
        # symmetric memory of torch.distributed as the second way to map peers
        seg = self._new_symm_segment(nbytes)
        if seg is None:
            raise ComprexError(f"cannot map peer memory (CUDA IPC: {err}; symmetric memory: {self._symm_error})")
        return seg

    def _new_symm_segment(self, nbytes: int):
        """A segment from torch's symmetric memory: peers are mapped like with CUDA IPC, and where
        the NVSwitch supports it the block is also bound to a multicast object, whose address
        (``mc``) lets one ``multimem`` instruction reach the same offset on every rank.  Returns
        None (on every rank alike) when any rank fails."""
        seg, self._symm_error = None, None
        try:
            import torch.distributed._symmetric_memory as symm
            t = symm.empty(nbytes, dtype=torch.uint8, device=self.device)
            t.zero_()
            hdl = symm.rendezvous(t, self.group.group_name if self.group is not None else dist.group.WORLD.group_name)
            bases = [int(p) for p in hdl.buffer_ptrs]
            mc = int(hdl.multicast_ptr) if (self.want_nvls and getattr(hdl, "has_multicast_support", False)) else 0
            torch.cuda.synchronize(self.device)
            seg = {"bases": bases, "size": nbytes, "used": 0, "keep": ("symm", t, hdl), "mc": mc}
        except Exception as exc:           # noqa: BLE001 - any failure means "use the other mapping"
            self._symm_error = exc
        oks = self._exchange((seg is not None, bool(seg and seg["mc"])))
        if not all(ok for ok, _ in oks):
            return None
        if not all(m for _, m in oks):
            seg["mc"] = 0
        return seg

    def _new_shm_segment(self, idx: int, nbytes: int) -> dict:
        if self._uid is None:
            uid = [uuid.uuid4().hex[:12] if self.rank == 0 else None]
            dist.broadcast_object_list(uid, src=dist.get_global_rank(self.group, 0), group=self.group)
            self._uid = uid[0]
        names = [f"/cx_{self._uid}_{idx}_{r}" for r in range(self.ranks)]
        mine = self.lib.cx_shm_create(names[self.rank].encode(), nbytes)
        if not mine:
            raise ComprexError("shared-memory segment: " + _lib.last_error())
        C.memset(mine, 0, nbytes)
        dist.barrier(group=self.group)
        bases = []
        for r in range(self.ranks):
            if r == self.rank:
                bases.append(mine)
                continue
            p = self.lib.cx_shm_open(names[r].encode(), nbytes)
            if not p:
                raise ComprexError("shared-memory segment: " + _lib.last_error())
            bases.append(p)
        dist.barrier(group=self.group)
        self.lib.cx_shm_unlink(names[self.rank].encode())  # mappings stay valid
        return {"bases": bases, "size": nbytes, "used": 0, "keep": ("shm", nbytes)}

    def alloc(self, nbytes: int, align: int = _ALIGN) -> SymmAlloc:
        """Collective: every rank must allocate the same sizes in the same order."""
        nbytes = max(int(nbytes), 1)
        for idx in range(len(self._segments) - 1, -1, -1):
            seg = self._segments[idx]
            off = _round_up(seg["used"], align)
            if off + nbytes <= seg["size"]:
                seg["used"] = off + nbytes
                return SymmAlloc(idx, off, nbytes)
            break  # only the newest segment is open, which keeps the order symmetric
        self._new_segment(nbytes + align)
        seg = self._segments[-1]
        seg["used"] = nbytes
        return SymmAlloc(len(self._segments) - 1, 0, nbytes)

    def ptr(self, a: SymmAlloc, rank: int | None = None, offset: int = 0) -> int:
        r = self.rank if rank is None else rank
        return self._segments[a.seg]["bases"][r] + a.offset + offset

    def mc_ptr(self, a: SymmAlloc, offset: int = 0) -> int:
        """Multicast address of the block (a store there lands in every rank's copy), 0 if none."""
        base = self._segments[a.seg].get("mc", 0)
        return base + a.offset + offset if base else 0

    @property
    def nvls(self) -> bool:
        """True when blocks of the heap have a multicast address (allocates the first segment)."""
        if not self.want_nvls:
            return False
        if not self._segments:
            self._new_segment(self.segment_size)
        return bool(self._segments[-1].get("mc", 0))

    def empty(self, n: int, dtype=torch.float32):
        """A vector of ``n`` elements inside the symmetric heap (collective: every rank allocates
        the same sizes in the same order).  Collectives that find their argument in the heap work
        on it in place, without staging copies; the reference requires the same of its buffers
        (they live in the registered GASPI segment, src/gaspiEx.tpp:127-135)."""
        es = torch.empty(0, dtype=dtype).element_size()
        a = self.alloc(max(n, 1) * es, 256)
        t = _tensor_at(self.ptr(a), n, dtype, self.device, self)
        self._heap_tensors[t.data_ptr()] = a
        return t

    def heap_block(self, t: torch.Tensor):
        """The SymmAlloc a tensor made by :meth:`empty` lives in (None for any other tensor)."""
        return self._heap_tensors.get(t.data_ptr()) if t is not None else None

    def heap_mark(self):
        """Snapshot of the allocator; pass to :meth:`heap_release` (collective)."""
        self._ensure_barrier()          # the barrier's own block must not be part of what is released
        return (len(self._segments), self._segments[-1]["used"] if self._segments else 0)

    def heap_release(self, mark) -> None:
        """Give back everything allocated since ``mark`` (stack discipline, collective).

        All ranks first finish their queued work: a peer may still be storing into the
        blocks that are about to be zeroed and handed out again."""
        nseg, used = mark
        self.barrier()
        self._heap_tensors = {k: a for k, a in self._heap_tensors.items()
                              if a.seg < nseg - 1 or (a.seg == nseg - 1 and a.offset + a.nbytes <= used)}
        while len(self._segments) > max(nseg, 1):
            self._free_segment(self._segments.pop(), collective=True)
        if self._segments and nseg >= 1:
            seg = self._segments[nseg - 1]
            lo, hi = used, seg["used"]
            if hi > lo:
                self.lib.cx_fill_zero(self.dev, seg["bases"][self.rank] + lo, hi - lo, _lib.stream_ptr(self.device))
            seg["used"] = used
        elif self._segments:
            seg = self._segments[0]
            self.lib.cx_fill_zero(self.dev, seg["bases"][self.rank], seg["used"], _lib.stream_ptr(self.device))
            seg["used"] = 0
        self.barrier()

    def _free_segment(self, seg: dict, collective: bool = False) -> None:
        keep = seg["keep"]
        if keep is None:
            return
        kind = keep[0]
        if kind == "local":
            (self.lib.cx_cuda_free if self.dev == _lib.DEV_CUDA else self.lib.cx_host_free)(keep[1])
        elif kind == "ipc":
            for p in keep[2]:
                self.lib.cx_cuda_ipc_close(p)
            if collective and self.group is not None:
                dist.barrier(group=self.group)   # every importer has unmapped before the owner frees
            self.lib.cx_cuda_free(keep[1])
        elif kind == "shm":
            for p in seg["bases"]:
                self.lib.cx_shm_close(p, keep[1])
        seg["keep"] = None            # "symm": torch frees the block when the last reference goes

    def close(self, collective: bool = True) -> None:
        """Free the heap.  With multicast-bound segments an explicit close first waits for all
        ranks: no rank unbinds its memory while a peer's kernel may still address it."""
        if self._closed:
            return
        self._closed = True
        try:
            if self.dev == _lib.DEV_CUDA and torch.cuda.is_available():
                torch.cuda.synchronize(self.device)
            if (collective and self.group is not None and dist.is_initialized()
                    and any(seg.get("mc", 0) for seg in self._segments)):
                dist.barrier(group=self.group)
        except Exception:
            pass
        self._heap_tensors = {}
        for seg in self._segments:
            self._free_segment(seg)
        self._segments = []
        for blk in self._pinned:
            blk.close()
        self._pinned = []

    # ---- helpers for the layers above -----------------------------------------------
    def scratch(self, nbytes: int) -> torch.Tensor:
        """Zeroed rank-local device memory (compressor workspaces, counters)."""
        return torch.zeros(max(int(nbytes), 64), dtype=torch.uint8, device=self.device)

    def read_bytes(self, ptr: int, nbytes: int) -> bytes:
        """Debug/test helper: copy raw heap bytes to the host."""
        buf = (C.c_char * nbytes)()
        if self.dev == _lib.DEV_CUDA:
            torch.cuda.synchronize(self.device)
            _lib.check(self.lib.cx_cuda_memcpy(buf, ptr, nbytes, 2, None), "memcpy")
            _lib.check(self.lib.cx_cuda_stream_sync(None), "sync")
        else:
            C.memmove(buf, ptr, nbytes)
        return bytes(buf)

    def read_header(self, ptr: int) -> _lib.Header:
        return _lib.Header.from_buffer_copy(self.read_bytes(ptr, 64))


class LoopbackWorld:
    """P virtual ranks in one process on one device.

    Used by single-GPU (and CPU) tests and benchmarks of the multi-rank
    schedules: a collective is run phase by phase, every phase for all ranks
    before the next one starts, so a consumer kernel is always launched after
    its producers and never has to wait.
    """

    def __init__(self, size: int, device=None, segment_size: int = _DEFAULT_SEGMENT, timeout_ms=None):
        self.size = size
        self.lib = _lib.load()
        self._segs: dict[int, tuple[list[int], int]] = {}
        self.envs = [GaspiEnvironment(segment_size, device=device, timeout_ms=timeout_ms, _world=self, _rank=r)
                     for r in range(size)]
        self.device = self.envs[0].device
        self._cuda = self.device.type == "cuda"

    def _segment_bases(self, idx: int, nbytes: int) -> list[int]:
        if idx not in self._segs:
            bases = []
            for _ in range(self.size):
                p = self.lib.cx_cuda_malloc(nbytes) if self._cuda else self.lib.cx_host_alloc(nbytes)
                if not p:
                    raise ComprexError("segment allocation failed: " + _lib.last_error())
                bases.append(p)
            self._segs[idx] = (bases, nbytes)
        bases, size = self._segs[idx]
        if size != nbytes:
            raise ComprexError("virtual ranks allocated different segment sizes: allocation order differs")
        return bases

    def run(self, objs, method: str, args_per_rank=None):
        """Run ``method`` of every rank's object phase by phase; returns the results."""
        args_per_rank = args_per_rank or [()] * self.size
        plans = [getattr(o, "_plan_" + method)(*a) for o, a in zip(objs, args_per_rank)]
        nph = {len(p) for p in plans}
        if len(nph) != 1:
            raise ComprexError("ranks disagree on the number of phases")
        for k in range(nph.pop()):
            for p in plans:
                p[k]()
        for o in objs:
            o._env.maybe_check()
        return [a[0] if a else None for a in args_per_rank]

    def close(self) -> None:
        for e in self.envs:
            e.close()
        if self._cuda and torch.cuda.is_available():
            torch.cuda.synchronize(self.device)
        for bases, _ in self._segs.values():
            for p in bases:
                (self.lib.cx_cuda_free if self._cuda else self.lib.cx_host_free)(p)
        self._segs = {}
