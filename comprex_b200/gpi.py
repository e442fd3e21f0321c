"""Runtime entry points with the reference's names (gpi.py:86-180).

``GaspiEnvironment`` is the handle every engine and collective takes.
``Gaspi_Runtime`` / ``Gaspi_Segment`` / ``initGaspiCxx`` exist so that scripts
written against the reference keep working: the runtime is
``torch.distributed`` (one process per GPU, ``torchrun`` instead of
``gaspi_run``), the segment is the environment's symmetric heap.
"""
from __future__ import annotations

import logging
import os

import torch
import torch.distributed as dist

from .parallel.env import GaspiEnvironment, LoopbackWorld  # noqa: F401

_log = logging.getLogger("comprex_b200")


def initGaspiCxx(backend: str | None = None) -> None:
    """Join the job started by ``torchrun`` (reads RANK / WORLD_SIZE / MASTER_*).

    A no-op when ``torch.distributed`` is already initialised or when the
    process was not started by a launcher (single rank).
    """
    if dist.is_initialized() or "RANK" not in os.environ:
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")) % torch.cuda.device_count())
    dist.init_process_group(backend=backend)


class Gaspi_Runtime:
    """Context manager with rank / size / barrier / flush (gpi.py:86-114)."""

    def __init__(self):
        initGaspiCxx()
        self._env = GaspiEnvironment(1 << 16)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self._env.close()

    def get(self):
        return self

    def getGlobalRank(self) -> int:
        return self._env.get_rank()

    def getGlobalSize(self) -> int:
        return self._env.get_ranks()

    def barrier(self) -> None:
        self._env.barrier()

    def flush(self) -> None:
        self._env.flush()


class Gaspi_Segment:
    """A heap of ``size`` bytes (gpi.py:119-135); wraps an environment."""

    def __init__(self, size: int):
        self.size = int(size)
        self._env = GaspiEnvironment(self.size)

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self._env.close()

    def get(self):
        return self._env


def gaspi_printf(message: str) -> None:
    """Rank-tagged log line (the reference forwards to ``gaspi_logger``, gpi.py:179-180)."""
    rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
    print(f"[rank {rank}] {message}", flush=True)
    _log.info("[rank %d] %s", rank, message)
