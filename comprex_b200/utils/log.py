"""Logging: one ``logging`` logger per rank and a JSON-lines metrics writer (the reference
prints through ``gaspi_printf`` to an external daemon, gpi.py:179-180, and writes CSV from
its benchmarks, examples/allreduce_speed.cpp:69-76)."""
from __future__ import annotations

import json
import logging
import os
import time


def get_logger(name: str = "comprex", rank: int | None = None) -> logging.Logger:
    """Logger whose records carry the rank; level from ``COMPREX_LOG`` (default WARNING)."""
    if rank is None:
        rank = int(os.environ.get("RANK", "0"))
    logger = logging.getLogger(f"{name}.r{rank}")
    if not logger.handlers:
        h = logging.StreamHandler()
        h.setFormatter(logging.Formatter(f"[%(asctime)s rank {rank}] %(levelname)s %(message)s"))
        logger.addHandler(h)
        logger.propagate = False
        logger.setLevel(os.environ.get("COMPREX_LOG", "WARNING").upper())
    return logger


class JsonlWriter:
    """Append one JSON object per line; ``None`` path keeps the records in memory only."""

    def __init__(self, path: str | None = None):
        self.path, self.records = path, []
        if path:
            os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)

    def write(self, **record) -> dict:
        record.setdefault("time", time.time())
        self.records.append(record)
        if self.path:
            with open(self.path, "a") as f:
                f.write(json.dumps(record) + "\n")
        return record


class StepLogger:
    """Per-step training metrics in the spirit of the reference's per-epoch TensorBoard
    scalars (LeNet/main.py:92-93): loss, throughput, and the compressor's counters
    (pairs sent, threshold, overflow) every ``every`` steps on rank 0."""

    def __init__(self, optimizer=None, every: int = 50, path: str | None = None, rank: int | None = None):
        self.opt, self.every, self.step = optimizer, max(int(every), 1), 0
        self.rank = int(os.environ.get("RANK", "0")) if rank is None else rank
        self.out = JsonlWriter(path if self.rank == 0 else None)
        self.log = get_logger(rank=self.rank)
        self._t = time.perf_counter()

    def __call__(self, loss=None, samples: int | None = None) -> dict | None:
        self.step += 1
        if self.step % self.every or self.rank != 0:
            return None
        now = time.perf_counter()
        rec = {"step": self.step}
        if loss is not None:
            rec["loss"] = float(loss)
        if samples is not None:
            rec["samples_per_s"] = samples * self.every / (now - self._t)
        if self.opt is not None and hasattr(self.opt, "stats"):
            rec.update({"comprex_" + k: v for k, v in self.opt.stats().items()})
        self._t = now
        self.log.info("%s", rec)
        return self.out.write(**rec)
