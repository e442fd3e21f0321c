"""Initial weight broadcast and periodic re-synchronisation
(reference: keras/callbacks.py:8-90).

The chief flattens all weights into one fp32 blob and writes it to every
other rank through a ``GaspiEx``; here that is a single kernel launch that
stores the blob into all peers' slots over NVLink, and one launch per worker
that copies it out.  The callbacks are framework-neutral objects with the
Keras hook names, so a training loop calls ``on_train_begin(model)`` /
``on_epoch_begin(model)`` itself.
"""
from __future__ import annotations

import torch

from .GaspiEx import GaspiEx


def weights_to_blob(model: torch.nn.Module) -> torch.Tensor:
    """All parameters and buffers with floating dtype, flattened to one fp32 vector."""
    return torch.cat([t.detach().reshape(-1).float() for t in _tensors(model)])


def blob_to_weights(model: torch.nn.Module, blob: torch.Tensor) -> None:
    off = 0
    with torch.no_grad():
        for t in _tensors(model):
            k = t.numel()
            t.copy_(blob[off:off + k].view_as(t).to(t.dtype))
            off += k


def _tensors(model):
    seen = []
    for t in list(model.parameters()) + list(model.buffers()):
        if t.is_floating_point():
            seen.append(t)
    return seen


def _broadcast(comm: GaspiEx, model, env, src: int) -> None:
    me, nr = env.get_rank(), env.get_ranks()
    if nr == 1:
        return
    if me == src:
        blob = weights_to_blob(model)
        comm.writeRemote_multi(blob, [r for r in range(nr) if r != me])
    else:
        comm.connectRx(src, 0)
        blob_to_weights(model, comm.readRemote())
    env.flush()


def broadcast_parameters(model: torch.nn.Module, gaspi_env, src: int = 0) -> None:
    """Every rank's model takes rank ``src``'s weights (collective)."""
    env = gaspi_env.get()
    size = sum(t.numel() for t in _tensors(model))
    mark = env.heap_mark()
    comm = GaspiEx(env, size)
    _broadcast(comm, model, env, src)
    env.heap_release(mark)   # the blob-sized slots are only needed once


class BroadcastInitWeights:
    def __init__(self, srcRank: int, gaspi_env):
        self.srcRank, self.gaspi_env = srcRank, gaspi_env

    def on_train_begin(self, model, logs=None) -> None:
        broadcast_parameters(model, self.gaspi_env, self.srcRank)


class SynchWeights:
    """Every ``intervall`` epochs all ranks take ``srcRank``'s weights (local-SGD style)."""

    def __init__(self, intervall: int, srcRank: int, gaspi_env):
        self.intervall, self.srcRank, self.gaspi_env = intervall, srcRank, gaspi_env
        self.comm = None
        self.epoch_counter = 0

    def on_train_begin(self, model, logs=None) -> None:
        if self.comm is None:
            self.comm = GaspiEx(self.gaspi_env.get(), sum(t.numel() for t in _tensors(model)))

    def on_epoch_begin(self, model, epoch=None, logs=None) -> None:
        self.epoch_counter += 1
        if self.epoch_counter >= self.intervall:
            self.epoch_counter = 0
            _broadcast(self.comm, model, self.gaspi_env.get(), self.srcRank)
            self.gaspi_env.get().barrier()
