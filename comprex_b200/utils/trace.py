"""Tracing and per-phase timing (the reference has a host wall-clock ``TictocTimer``,
examples/tictocTimer.hxx, and nothing inside the library).

* ``nvtx_range(name)``: an NVTX range when ``COMPREX_NVTX=1`` (or ``enable_nvtx()``) and a
  CUDA device is present, otherwise a no-op; the optimizer wraps fold / send / receive of
  every bucket in one.
* ``PhaseTimer``: device time of named phases with CUDA events on the current stream
  (host monotonic clock on the CPU), read after a synchronise; ``summary()`` gives count,
  total and mean per phase.
* ``TictocTimer``: the reference's accumulating wall-clock timer, for host code.
"""
from __future__ import annotations

import contextlib
import os
import time

import torch

_nvtx_on = os.environ.get("COMPREX_NVTX", "0") == "1"


def enable_nvtx(on: bool = True) -> None:
    global _nvtx_on
    _nvtx_on = bool(on)


def nvtx_enabled() -> bool:
    return _nvtx_on and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    if not nvtx_enabled():
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


class PhaseTimer:
    """``with timer.phase("compress"): ...`` around launches on the current stream."""

    def __init__(self, device=None, enabled: bool = True):
        self.device = torch.device(device) if device is not None else None
        self.cuda = self.device is not None and self.device.type == "cuda"
        self.enabled = enabled
        self._open: list = []        # (name, start, end) not yet read
        self._acc: dict = {}

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if self.cuda:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                self._open.append((name, a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._add(name, (time.perf_counter() - t0) * 1e3)

    def _add(self, name: str, ms: float) -> None:
        cnt, tot = self._acc.get(name, (0, 0.0))
        self._acc[name] = (cnt + 1, tot + ms)

    def collect(self) -> None:
        """Synchronise and fold the finished events into the totals."""
        if self.cuda and self._open:
            torch.cuda.synchronize(self.device)
            for name, a, b in self._open:
                self._add(name, a.elapsed_time(b))
        self._open = []

    def summary(self) -> dict:
        self.collect()
        return {k: {"count": c, "total_ms": t, "mean_ms": t / c} for k, (c, t) in self._acc.items()}

    def reset(self) -> None:
        self._open, self._acc = [], {}


class TictocTimer:
    """Accumulating wall-clock timer (examples/tictocTimer.hxx): tic/toc pairs add up."""

    def __init__(self):
        self.elapsed, self._t0, self.laps = 0.0, None, 0

    def tic(self) -> None:
        self._t0 = time.perf_counter()

    def toc(self) -> float:
        if self._t0 is None:
            raise RuntimeError("toc without tic")
        dt = time.perf_counter() - self._t0
        self.elapsed += dt
        self.laps += 1
        self._t0 = None
        return dt

    def get_elapsed_time_in_sec(self) -> float:
        return self.elapsed

    def reset(self) -> None:
        self.elapsed, self._t0, self.laps = 0.0, None, 0
