"""Allreduce objects as framework ops (reference: allreduceOp.py:8-143 and the TensorFlow
kernels in src/tf_ops/tfAllreduce.cc:11-149).

The reference registers nine TensorFlow ops (``*AllreduceApply`` for the six
collectives, ``Comprex*AllreduceFlush`` for the three compressed ones) that take
the C++ object's address as an integer attribute and run it in place on the
input tensor.  Here the same shape is expressed with ``torch.library``: two
in-place custom ops, ``comprex::allreduce_apply(Tensor(a!) t, int handle)`` and
``comprex::allreduce_flush(Tensor(a!) t, int handle)``, where ``handle`` names
an allreduce object in a process-local registry.  Being registered ops they can
be called from eager code, traced graphs and TorchScript-free export alike;
the work itself is this package's kernels on the tensor's stream.

The ``*Op`` wrapper classes keep the reference's interface: ``setup(size,
tag=0, ...)`` once, then ``apply(t)`` / ``op(t)``, and for the compressed ones
``flush(t)`` and ``set_compression_ratio(r)``.
"""
from __future__ import annotations

import itertools

import torch

from . import allreduce as _ar
from ._lib import ComprexError

_registry: dict[int, object] = {}
_next_handle = itertools.count(1)


def register(obj) -> int:
    """Give an allreduce object a handle usable as an op attribute."""
    h = next(_next_handle)
    _registry[h] = obj
    return h


def unregister(handle: int) -> None:
    _registry.pop(handle, None)


def _lookup(handle: int):
    try:
        return _registry[handle]
    except KeyError:
        raise ComprexError(f"no allreduce object registered under handle {handle}") from None


@torch.library.custom_op("comprex::allreduce_apply", mutates_args=("t",))
def allreduce_apply(t: torch.Tensor, handle: int) -> None:
    _lookup(handle).apply(t)


@torch.library.custom_op("comprex::allreduce_flush", mutates_args=("t",))
def allreduce_flush(t: torch.Tensor, handle: int) -> None:
    _lookup(handle).flush(t)


class AllreduceOp:
    """Base of the six wrappers (allreduceOp.py:8-19)."""
    _cls = None

    def __init__(self, gaspi_env):
        self.gaspi_env = gaspi_env
        self.allreduce = self._cls(gaspi_env)
        self.handle = register(self.allreduce)
        self.size = None

    def __del__(self):
        unregister(getattr(self, "handle", -1))

    def __call__(self, inputs):
        return self.apply(inputs)

    def get_size(self):
        return self.size

    def _setup(self, size, *args, **kw):
        if self.size is not None:
            if size > self.size:
                raise RuntimeError("Allreduce was already set up for size %d, cannot grow to %d" % (self.size, size))
            return
        self.size = size
        self.allreduce.setup_connections(size, *args, **kw)

    def apply(self, inputs: torch.Tensor) -> torch.Tensor:
        """In place on ``inputs``; returns it (the TF op forwards its input as output)."""
        allreduce_apply(inputs, self.handle)
        return inputs


class _CompressedOp(AllreduceOp):
    def flush(self, inputs: torch.Tensor) -> torch.Tensor:
        allreduce_flush(inputs, self.handle)
        return inputs

    def reset(self) -> None:
        self.allreduce.reset()

    def set_compression_ratio(self, compression_ratio: float) -> None:
        self.allreduce.set_compression_ratio(compression_ratio)


class AllToOneAllreduceOp(AllreduceOp):
    _cls = _ar.AllToOneAllreduce

    def setup(self, size, tag=0, chiefRank=0):
        self._setup(size, tag, chiefRank)


class Comprex_AllToOneAllreduceOp(_CompressedOp):
    _cls = _ar.Comprex_AllToOneAllreduce

    def setup(self, size, tag=0, chiefRank=0, compression_ratio=0.01, size_factor=1.0):
        self._setup(size, tag, chiefRank, compression_ratio, size_factor)


class RingAllreduceOp(AllreduceOp):
    _cls = _ar.RingAllreduce

    def setup(self, size, tag=0):
        self._setup(size, tag)


class Comprex_RingAllreduceOp(_CompressedOp):
    _cls = _ar.Comprex_RingAllreduce

    def setup(self, size, tag=0, compression_ratio=0.01, size_factor=1.0):
        self._setup(size, tag, compression_ratio, size_factor)


class BigRingAllreduceOp(AllreduceOp):
    _cls = _ar.BigRingAllreduce

    def setup(self, size, tag=0):
        self._setup(size, tag)


class Comprex_BigRingAllreduceOp(_CompressedOp):
    _cls = _ar.Comprex_BigRingAllreduce

    def setup(self, size, tag=0, compression_ratio=0.01, size_factor=1.0):
        self._setup(size, tag, compression_ratio, size_factor)
