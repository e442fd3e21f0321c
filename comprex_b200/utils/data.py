"""Host <-> device plumbing of a training loop: input prefetch and asynchronous scalar
read-back (the reference feeds Keras from in-memory NumPy arrays, LeNet/main.py:36-47, and has
no equivalent; on a GPU these two keep the copy engines busy while the SMs compute).

* ``DevicePrefetcher`` takes an iterable of batches whose tensors sit in pinned host memory
  and hands out device copies, always keeping the next batch's host-to-device copy in flight on
  a copy stream while the current batch is being used.
* ``AsyncScalar`` copies a 0-dim device tensor (the loss) into pinned host memory without
  blocking; ``value()`` waits for that one copy only, so a loop can log step k while step k+1
  is already queued.
"""
from __future__ import annotations

import torch


class DevicePrefetcher:
    def __init__(self, batches, device, depth: int = 1):
        self.device = torch.device(device)
        self.cuda = self.device.type == "cuda"
        self.it = iter(batches)
        self.depth = max(int(depth), 1)
        self.stream = torch.cuda.Stream(self.device) if self.cuda else None
        self.queue: list = []
        self.h2d_bytes = 0
        for _ in range(self.depth):
            self._issue()

    def _issue(self) -> None:
        try:
            batch = next(self.it)
        except StopIteration:
            return
        single = isinstance(batch, torch.Tensor)
        items = (batch,) if single else tuple(batch)
        if not self.cuda:
            self.queue.append((items, None, single))
            return
        with torch.cuda.stream(self.stream):
            out = tuple(t.to(self.device, non_blocking=True) for t in items)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.h2d_bytes += sum(t.numel() * t.element_size() for t in items)
        self.queue.append((out, ev, single))

    def __iter__(self):
        return self

    def __next__(self):
        if not self.queue:
            raise StopIteration
        out, ev, single = self.queue.pop(0)
        if ev is not None:
            cur = torch.cuda.current_stream(self.device)
            cur.wait_event(ev)                 # the consumer's stream, not the host, waits for the copy
            for t in out:
                t.record_stream(cur)           # the allocator must not reuse it while `cur` reads it
        self._issue()
        return out[0] if single else out

    next = __next__


class AsyncScalar:
    """``r = AsyncScalar(loss)`` right after the step; ``r.value()`` later."""

    def __init__(self, t: torch.Tensor):
        t = t.detach()
        if t.device.type != "cuda":
            self._host, self._ev = t.reshape(()).to(torch.float32).clone(), None
            return
        self._host = torch.empty((), dtype=torch.float32).pin_memory()
        self._host.copy_(t.reshape(()).to(torch.float32), non_blocking=True)
        self._ev = torch.cuda.Event()
        self._ev.record(torch.cuda.current_stream(t.device))

    def value(self) -> float:
        if self._ev is not None:
            self._ev.synchronize()
        return float(self._host)
