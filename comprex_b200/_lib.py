"""ctypes binding of ``libcomprex_b200.so`` (flat C ABI, see csrc/cx_common.h).

The reference loads ``libPyGPI.so`` the same way (ComprEx.py:10, gpi.py:16-79);
here the library is built in-tree by :mod:`comprex_b200.build` and every call
that fails raises :class:`ComprexError` with the native error text.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

import torch

MAX_PEERS = 16
SUBTILE = 1024

DEV_HOST, DEV_CUDA = 0, 1
F32, BF16, F16 = 0, 1, 2
KIND_PAIRS, KIND_DENSE, KIND_RLE = 1, 2, 3
ST_TIMEOUT, ST_BAD_HEADER, ST_OVERFLOW, ST_BAD_INDEX = 1, 2, 4, 8
OP_ADD, OP_SET, OP_SGD, OP_MOMENTUM, OP_ADAMW = 0, 1, 2, 3, 4
TG_MULTICAST = 1      # Targets.pad flag: ep[count] is the multicast alias of the targets' slots

_DTYPES = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}


class ComprexError(RuntimeError):
    """Raised for native failures and for status words kernels leave behind."""


class Header(C.Structure):
    _fields_ = [("seq", C.c_uint64), ("bytes", C.c_uint64), ("n", C.c_uint32), ("nnz", C.c_uint32),
                ("nnz_found", C.c_uint32), ("kind", C.c_uint32), ("threshold", C.c_float),
                ("nsub", C.c_uint32), ("src_rank", C.c_uint32), ("dtype", C.c_uint32),
                ("pad", C.c_uint32 * 4)]


class Endpoint(C.Structure):
    _fields_ = [("hdr", C.c_void_p), ("table", C.c_void_p), ("pairs", C.c_void_p)]


class Targets(C.Structure):
    _fields_ = [("count", C.c_int32), ("pad", C.c_int32), ("ep", Endpoint * MAX_PEERS)]


class Sources(C.Structure):
    _fields_ = [("count", C.c_int32), ("pad", C.c_int32), ("ep", Endpoint * MAX_PEERS),
                ("seq", C.c_uint64 * MAX_PEERS), ("cap", C.c_uint32 * MAX_PEERS)]


class Stats(C.Structure):
    _fields_ = [("n", C.c_uint32), ("nnz", C.c_uint32), ("nnz_found", C.c_uint32),
                ("status", C.c_uint32), ("threshold", C.c_float), ("pad", C.c_uint32 * 3)]


class ApplyArgs(C.Structure):
    _fields_ = [("op", C.c_int32), ("out_dtype", C.c_int32), ("out", C.c_void_p),
                ("shadow", C.c_void_p), ("shadow_dtype", C.c_int32), ("pad", C.c_int32),
                ("m", C.c_void_p), ("v", C.c_void_p), ("scale", C.c_float), ("lr", C.c_float),
                ("beta1", C.c_float), ("beta2", C.c_float), ("eps", C.c_float), ("wd", C.c_float),
                ("bc1", C.c_float), ("bc2", C.c_float), ("momentum", C.c_float), ("pad2", C.c_float)]


OPK_THRESHOLD, OPK_COMPRESS, OPK_APPLY, OPK_DENSE_SEND, OPK_DENSE_REDUCE, OPK_UPDATE, OPK_MM_ALLREDUCE = 1, 2, 3, 4, 5, 6, 7


class Op(C.Structure):
    """One launch of a pre-built launch sequence (CxOp in csrc/cx_common.h)."""
    _fields_ = [("kind", C.c_int32), ("dev", C.c_int32), ("dtype", C.c_int32), ("has_ranges", C.c_int32),
                ("g", C.c_void_p), ("r", C.c_void_p), ("n", C.c_int64),
                ("ratio", C.c_float), ("default_subsamples", C.c_int32), ("subsample_factor", C.c_float),
                ("scale", C.c_float), ("thr", C.c_void_p), ("cap", C.c_uint32), ("src_rank", C.c_uint32),
                ("workspace", C.c_void_p), ("ws_bytes", C.c_int64), ("stats", C.c_void_p),
                ("out", C.c_void_p), ("own", C.c_void_p), ("status", C.c_void_p), ("timeout_ns", C.c_uint64),
                ("has_push", C.c_int32), ("lane", C.c_int32),
                ("starts", C.c_int64 * MAX_PEERS), ("lens", C.c_int64 * MAX_PEERS),
                ("tg", Targets), ("src", Sources), ("apply", ApplyArgs)]


assert C.sizeof(Header) == 64 and C.sizeof(Stats) == 32

_lock = threading.Lock()
_lib = None


def lib_path() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libcomprex_b200.so")


def _declare(lib) -> None:
    vp, i32, i64, u32, u64, f32 = C.c_void_p, C.c_int, C.c_int64, C.c_uint32, C.c_uint64, C.c_float
    P = C.POINTER
    sig = {
        "cx_last_error": (C.c_char_p, []),
        "cx_launch_count": (u64, []),
        "cx_reset_launch_count": (None, []),
        "cx_version": (i32, []),
        "cx_workspace_bytes": (i64, [i64]),
        "cx_threshold_plan": (None, [i64, f32, i32, f32, P(C.c_int32), P(C.c_int32), P(f32), P(C.c_int32)]),
        "cx_threshold_topk": (i32, [i32, i32, vp, vp, i64, f32, i32, f32, vp, vp]),
        "cx_threshold_workspace_bytes": (i64, []),
        "cx_threshold_select": (i32, [i32, i32, vp, vp, i64, f32, i32, f32, vp, vp, i64, vp]),
        "cx_compress": (i32, [i32, i32, vp, vp, i64, vp, u32, u64, P(Targets), vp, i64, vp, u32, vp]),
        "cx_apply": (i32, [i32, P(Sources), i64, P(ApplyArgs), vp, u64, vp]),
        "cx_update_dense": (i32, [i32, vp, i64, P(ApplyArgs), vp]),
        "cx_barrier": (i32, [i32, i32, i32, P(C.c_void_p), u64, vp, u64, vp]),
        "cx_mm_flag_bytes": (i64, []),
        "cx_mm_counter_bytes": (i64, []),
        "cx_mm_allreduce": (i32, [i32, vp, vp, vp, vp, i64, i64, i32, i32, C.c_float, i32, i64, u64,
                                  P(C.c_void_p), vp, vp, u64, vp]),
        "cx_forward": (i32, [i32, P(Endpoint), u64, P(Targets), u64, u32, vp, vp, u64, vp]),
        "cx_dense_send": (i32, [i32, i32, vp, vp, i64, u64, P(Targets), P(i64), P(i64), vp, u32, vp]),
        "cx_dense_reduce": (i32, [i32, i32, vp, vp, i64, P(Sources), f32, P(Targets), u64, P(i64), P(i64),
                                  vp, u32, vp, u64, vp]),
        "cx_run_ops": (i32, [P(Op), i32, u64, vp]),
        "cx_graph_build": (i32, [P(Op), i32, P(vp)]),
        "cx_graph_launch": (i32, [vp, u64, vp]),
        "cx_graph_free": (i32, [vp]),
        "cx_sizeof": (i64, [i32]),
        "cx_fold": (i32, [i32, i32, vp, vp, vp, vp, vp, vp, i32, vp, vp, f32, f32, f32, vp]),
        "cx_axpy": (i32, [i32, i32, vp, i32, vp, f32, i64, vp]),
        "cx_fill_zero": (i32, [i32, vp, i64, vp]),
        "cx_rle_compress_host": (i64, [vp, vp, i64, f32, vp, i64]),
        "cx_rle_decode_host": (i32, [vp, i64, vp, i64, i32]),
        "cx_rle_slot_bytes": (i64, [i64]),
        "cx_rle_workspace_bytes": (i64, [i64]),
        "cx_rle_send": (i32, [i32, i32, vp, vp, i64, vp, i64, u64, P(Targets), vp, i64, u32, vp]),
        "cx_rle_recv": (i32, [i32, P(Endpoint), u64, vp, i64, i32, i64, vp, i64, vp, u64, vp]),
        "cx_cuda_device_count": (i32, []),
        "cx_cuda_set_device": (i32, [i32]),
        "cx_cuda_malloc": (vp, [i64]),
        "cx_cuda_free": (i32, [vp]),
        "cx_cuda_ipc_get": (i32, [vp, vp]),
        "cx_cuda_ipc_open": (vp, [vp]),
        "cx_cuda_ipc_close": (i32, [vp]),
        "cx_cuda_can_access_peer": (i32, [i32, i32]),
        "cx_pinned_alloc": (vp, [i64, P(vp)]),
        "cx_pinned_free": (i32, [vp]),
        "cx_cuda_stream_sync": (i32, [vp]),
        "cx_cuda_memcpy": (i32, [vp, vp, i64, i32, vp]),
        "cx_shm_create": (vp, [C.c_char_p, i64]),
        "cx_shm_open": (vp, [C.c_char_p, i64]),
        "cx_shm_close": (i32, [vp, i64]),
        "cx_shm_unlink": (i32, [C.c_char_p]),
        "cx_host_alloc": (vp, [i64]),
        "cx_host_free": (i32, [vp]),
        "cx_host_wait_seq": (i32, [vp, u64, u64]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


def load():
    """Return the loaded native library, building it first when it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = lib_path()
        if not os.path.exists(path):
            from . import build as _build
            try:
                _build.build()
            except Exception as exc:  # no nvcc on this machine
                raise ComprexError(
                    f"native library {path} is missing and could not be built: {exc}") from exc
        lib = C.CDLL(path)
        _declare(lib)
        for what, mirror in enumerate((Op, Sources, Targets, ApplyArgs, None, Header)):
            if mirror is not None and lib.cx_sizeof(what) != C.sizeof(mirror):
                raise ComprexError(f"{path} does not match this binding ({mirror.__name__} is "
                                   f"{lib.cx_sizeof(what)} bytes there, {C.sizeof(mirror)} here): rebuild it")
        _lib = lib
    return _lib


def last_error() -> str:
    return load().cx_last_error().decode("utf-8", "replace")


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        raise ComprexError(f"{what or 'native call'} failed: {last_error()} (rc={rc})")


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _DTYPES[dt]
    except KeyError:
        raise ComprexError(f"unsupported dtype {dt}; use float32, bfloat16 or float16") from None


def dev_code(t: torch.Tensor) -> int:
    return DEV_CUDA if t.is_cuda else DEV_HOST


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_ptr(device: torch.device) -> int:
    """cudaStream_t of the current stream of ``device`` (0 on the host).  Called once per launch:
    the raw-pointer query avoids building a ``torch.cuda.Stream`` object each time."""
    if device.type != "cuda":
        return 0
    if _raw_stream is not None and device.index is not None:
        return _raw_stream(device.index)
    return torch.cuda.current_stream(device).cuda_stream


def decode_status(bits: int) -> str:
    names = []
    for bit, name in ((ST_TIMEOUT, "TIMEOUT"), (ST_BAD_HEADER, "BAD_HEADER"), (ST_OVERFLOW, "OVERFLOW"),
                      (ST_BAD_INDEX, "BAD_INDEX")):
        if bits & bit:
            names.append(name)
    return "|".join(names) or "OK"


def launch_count() -> int:
    """Number of kernels this library launched in this process so far."""
    return int(load().cx_launch_count())
