"""The native collectives (csrc/collectives.cpp) from Python.

The six allreduce classes also exist as C++ objects behind a flat C ABI, for callers without
Python (reference: src/allreduce_C.cpp:12-122).  ``NativeAllreduce`` drives one of them on the
heap of a :class:`~comprex_b200.parallel.env.GaspiEnvironment`: the environment's peer mappings
(and its multicast address, where there is one) are handed to ``cx_comm_create``, the schedule
itself runs in C++.  One native communicator per environment is shared by all objects; it takes
the heap from its current fill level on, so create native objects after (or instead of) Python-side
ones in the same order on every rank.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import ComprexError
from .GaspiEx import to_device_vector, write_back

KINDS = {"alltoone": 0, "comprex_alltoone": 1, "ring": 2, "comprex_ring": 3, "bigring": 4, "comprex_bigring": 5}
CONSISTENT, OWNER_RESIDUAL, ALIGNED_CHUNKS = 1, 2, 4


def _declare(lib) -> None:
    if getattr(lib, "_cx_native_declared", False):
        return
    vp, i32, i64, u64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_float
    sig = {
        "cx_comm_create": (vp, [i32, i32, i32, i32, C.POINTER(vp), vp, i64, u64]),
        "cx_comm_destroy": (None, [vp]),
        "cx_comm_check": (C.c_uint32, [vp]),
        "cx_comm_sync": (i32, [vp, vp]),
        "cx_allreduce_create": (vp, [vp, i32, i64, i32, f32, f32, i32, i32]),
        "cx_allreduce_apply": (i32, [vp, vp, vp]),
        "cx_allreduce_flush": (i32, [vp, vp, vp]),
        "cx_allreduce_reset": (i32, [vp]),
        "cx_allreduce_set_ratio": (i32, [vp, f32]),
        "cx_allreduce_set_scale": (None, [vp, f32]),
        "cx_allreduce_size": (i64, [vp]),
        "cx_allreduce_state": (i32, [vp, vp, i64, C.POINTER(u64)]),
        "cx_allreduce_load_state": (i32, [vp, vp, i64, u64]),
        "cx_allreduce_stats": (i32, [vp, C.POINTER(_lib.Stats)]),
        "cx_allreduce_destroy": (None, [vp]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    lib._cx_native_declared = True


def native_comm(env):
    """The native communicator of an environment (created on first use: a fresh segment of the
    environment's size, so that native and Python-side objects never share heap blocks)."""
    comm = getattr(env, "_native_comm", None)
    if comm is None:
        _declare(env.lib)
        env._new_segment(env.segment_size)
        seg = env._segments[-1]
        seg["used"] = seg["size"]                     # the native side owns this segment entirely
        bases = (C.c_void_p * _lib.MAX_PEERS)(*[seg["bases"][r] if r < env.ranks else None for r in range(_lib.MAX_PEERS)])
        comm = env.lib.cx_comm_create(env.dev, env.device.index or 0, env.rank, env.ranks, bases,
                                      seg.get("mc", 0) or None, seg["size"], env.timeout_ns)
        if not comm:
            raise ComprexError("cx_comm_create: " + _lib.last_error())
        env._native_comm = comm
    return comm


class NativeAllreduce:
    """One native allreduce object; same methods as the Python classes of ``allreduce.py``."""

    def __init__(self, gaspi_env, kind: str, size: int, compression_ratio: float = 0.01, size_factor: float = 1.0,
                 chiefRank: int = 0, dtype: torch.dtype = torch.float32, consistent: bool = False,
                 owner_residual: bool = False, chunk_align: int = 1):
        self._env = env = gaspi_env.get()
        if env._world is not None:
            raise ComprexError("native collectives need real ranks (their calls wait for the peers)")
        self.kind, self.size, self.dtype = kind, int(size), dtype
        self.compressed = kind.startswith("comprex")
        flags = (CONSISTENT if consistent else 0) | (OWNER_RESIDUAL if owner_residual else 0) | \
                (ALIGNED_CHUNKS if chunk_align > 1 else 0)
        self._comm = native_comm(env)
        self._h = env.lib.cx_allreduce_create(self._comm, KINDS[kind], self.size, _lib.dtype_code(dtype),
                                              compression_ratio, size_factor, chiefRank, flags)
        if not self._h:
            raise ComprexError("cx_allreduce_create: " + _lib.last_error())

    def getSize(self):
        return self.size

    def _call(self, fn, vector):
        env = self._env
        n = vector.size if hasattr(vector, "size") and not callable(vector.size) else vector.numel()
        if n != self.size:
            raise ComprexError("Allreduce input vector of size %d does not match allreduce size %d!" % (n, self.size))
        t, orig = to_device_vector(env, vector)
        _lib.check(fn(self._h, t.data_ptr(), _lib.stream_ptr(env.device)), "native allreduce")
        if env.sync_check or orig is not None:
            self.check()
        write_back(t, orig)
        return vector

    def apply(self, vector):
        return self._call(self._env.lib.cx_allreduce_apply, vector)

    __call__ = apply

    def flush(self, vector):
        return self._call(self._env.lib.cx_allreduce_flush, vector)

    def reset(self):
        _lib.check(self._env.lib.cx_allreduce_reset(self._h), "cx_allreduce_reset")

    def set_compression_ratio(self, compression_ratio):
        self._env.lib.cx_allreduce_set_ratio(self._h, float(compression_ratio))

    def check(self) -> None:
        """Wait for this rank's queued work and raise what kernels reported."""
        env = self._env
        _lib.check(env.lib.cx_comm_sync(self._comm, _lib.stream_ptr(env.device)), "cx_comm_sync")
        bits = int(env.lib.cx_comm_check(self._comm))
        if bits:
            raise ComprexError(f"rank {env.rank}: native allreduce: {_lib.decode_status(bits)}")

    def stats(self) -> dict:
        self.check()
        s = _lib.Stats()
        _lib.check(self._env.lib.cx_allreduce_stats(self._h, C.byref(s)), "cx_allreduce_stats")
        return {"n": int(s.n), "nnz": int(s.nnz), "nnz_found": int(s.nnz_found), "status": int(s.status),
                "threshold": float(s.threshold)}

    def state_dict(self) -> dict:
        self.check()
        step = C.c_uint64()
        res = torch.zeros(self.size if self.compressed else 0, dtype=torch.float32)
        _lib.check(self._env.lib.cx_allreduce_state(self._h, res.data_ptr() if self.compressed else None, self.size,
                                                    C.byref(step)), "cx_allreduce_state")
        return {"kind": self.kind, "size": self.size, "step": int(step.value), "residual": res if self.compressed else None}

    def load_state_dict(self, state) -> None:
        if state["kind"] != self.kind or state["size"] != self.size:
            raise ComprexError("state_dict belongs to a different allreduce")
        res = state["residual"]
        _lib.check(self._env.lib.cx_allreduce_load_state(self._h, res.contiguous().data_ptr() if res is not None else None,
                                                         self.size, state["step"]), "cx_allreduce_load_state")

    def __del__(self):
        try:
            if self._h:
                self._env.lib.cx_allreduce_destroy(self._h)
                self._h = None
        except Exception:
            pass
