"""DistributedDataParallel communication hook with top-k compression and error feedback.

This is the PyTorch form of the reference's TensorFlow ops (src/tf_ops/tfAllreduce.cc:11-149,
allreduceOp.py:8-143), which run an allreduce object in place on a gradient tensor:

    state = ComprexHookState(env, compression_ratio=0.01)
    ddp_model.register_comm_hook(state, comprex_hook)

Per gradient bucket (``bucket_cap_mb`` of DDP, 25 MB by default) the hook keeps
a residual and a ``Comprex_BigRingAllreduce`` in replica-consistent mode.  On a
dedicated high-priority stream that first waits for the bucket's gradients it
launches: threshold estimate, fused residual-add / select / store-to-peers, and
the receive kernel that writes ``(1/P) * sum of all ranks' sparse
contributions`` back into the bucket.  The returned future completes on that
stream, so the exchange of one bucket overlaps the backward pass of the next.
Buckets below ``dense_fallback_bytes`` (64 KiB) use the dense one-shot
allreduce kernels instead.  No NCCL call is made on either path.

The state object is picklable (``__getstate__`` carries ratio, step counts and
the residuals by bucket key) so it can be saved next to the optimizer state.
"""
import torch
import torch.distributed as dist

from . import allreduce as _ar
from .ops import primitives as P


class ComprexHookState:
    def __init__(self, gaspi_env, compression_ratio: float = 0.01, capacity_slack: float = 2.0,
                 dense_fallback_bytes: int = 65536, min_capacity: int = 1024):
        self.env = gaspi_env.get()
        self.compression_ratio = float(compression_ratio)
        self.capacity_slack = float(capacity_slack)
        self.dense_fallback_bytes = int(dense_fallback_bytes)
        self.min_capacity = int(min_capacity)
        self.reducers: dict = {}
        self._pending: dict = {}
        self._stream = None
        self.steps = 0

    # ---- helpers ---------------------------------------------------------------------------------
    def stream(self):
        if self._stream is None and self.env.device.type == "cuda":
            self._stream = torch.cuda.Stream(self.env.device, priority=-1)
        return self._stream

    def _size_factor(self, n: int) -> float:
        cap = max(int(n * self.compression_ratio * self.capacity_slack), self.min_capacity)
        return (8.0 * cap + 16.0) / (4.0 * n)

    def reducer(self, index: int, n: int, dtype: torch.dtype):
        """Collective on first use of a (bucket index, size): DDP's bucket layout is the same on every rank."""
        key = (index, n, str(dtype))
        red = self.reducers.get(key)
        if red is None:
            if n * torch.empty(0, dtype=dtype).element_size() < self.dense_fallback_bytes:
                red = _ar.BigRingAllreduce(self.env)
                red.setup_connections(n, 1, dtype=dtype, ordered=True)   # the same bits on every rank
                red.result_scale = 1.0 / self.env.ranks        # the mean comes out of the reducing kernel
            else:
                red = _ar.Comprex_BigRingAllreduce(self.env)
                red.setup_connections(n, 1, self.compression_ratio, self._size_factor(n), consistent=True)
                saved = self._pending.pop(key, None)
                if saved is not None:
                    red.load_state_dict(saved)
            self.reducers[key] = red
        return red

    def set_compression_ratio(self, ratio: float) -> None:
        self.compression_ratio = float(ratio)
        for red in self.reducers.values():
            if red.compressed:
                red.set_compression_ratio(ratio)

    def stats(self) -> dict:
        return {k: r.stats() for k, r in self.reducers.items() if r.compressed}

    # ---- checkpoint ----------------------------------------------------------------------------------
    def __getstate__(self):
        return {"compression_ratio": self.compression_ratio, "capacity_slack": self.capacity_slack,
                "dense_fallback_bytes": self.dense_fallback_bytes, "min_capacity": self.min_capacity,
                "steps": self.steps,
                "residuals": {k: r.state_dict() for k, r in self.reducers.items() if r.compressed}}

    def __setstate__(self, state):
        self.compression_ratio = state["compression_ratio"]
        self.capacity_slack = state["capacity_slack"]
        self.dense_fallback_bytes = state["dense_fallback_bytes"]
        self.min_capacity = state["min_capacity"]
        self.steps = state["steps"]
        self.reducers, self._pending, self._stream, self.env = {}, dict(state["residuals"]), None, None

    def attach(self, gaspi_env) -> "ComprexHookState":
        """Bind an unpickled state to this process' environment; residuals are restored lazily."""
        self.env = gaspi_env.get()
        return self

    state_dict = __getstate__


def comprex_hook(state: ComprexHookState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    """Average the bucket's gradients over all ranks through the compressed exchange."""
    buf = bucket.buffer()
    env = state.env
    n = buf.numel()
    red = state.reducer(bucket.index(), n, buf.dtype)
    if bucket.is_last():
        state.steps += 1
    scale = 1.0 / env.ranks
    cuda = buf.is_cuda
    fut = torch.futures.Future(devices=[buf.device]) if cuda else torch.futures.Future()

    def run():
        if red.compressed:
            seq, par = red.send_fast(buf)
            red.recv_fast(seq, par, P.args_set(buf, scale))
        else:
            for phase in red._plan_apply(buf):
                phase()

    if cuda:
        comm = state.stream()
        comm.wait_stream(torch.cuda.current_stream(buf.device))
        with torch.cuda.stream(comm):
            run()
            buf.record_stream(comm)
            fut.set_result(buf)
    else:
        run()
        env.maybe_check()
        fut.set_result(buf)
    return fut
