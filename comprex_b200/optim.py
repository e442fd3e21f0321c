"""Compressed data-parallel optimizer (reference: keras/comprex_optimizer.py:8-170).

The reference hooks into Keras' ``_aggregate_gradients``: per tensor it clips
the gradient to an L2 norm of ``pre_clipnorm``, folds it into a *local*
momentum buffer scaled by the learning rate (``mom = m*mom + lr*g``),
concatenates everything into one blob, allreduces the blob with one of six
collectives (default ``comprex_bigring``), divides by the number of ranks and
applies ``var = (1-wd)*var - update``.  This class keeps those semantics for
PyTorch and maps a step onto five kernel launches per bucket:

1. per-tensor sums of squares and 2. clip + momentum fold, read straight from
   the gradient tensors autograd produced into the flat fp32 update vector,
3. threshold estimate of ``residual + update`` (device resident),
4. fused ``residual += update`` / select / store pairs into every peer's slot,
5. fused wait / scatter-add in rank order / average / parameter update, which
   also refreshes the low-precision copy of the weights when the model is held
   in bf16 or fp16.

The parameters live in one flat fp32 master buffer (the model's tensors are
views of it, or of its low-precision shadow, in their own memory order, so
channels-last weights stay channels-last); there is no flat gradient buffer,
no concatenation and no slicing copy.  The flat
buffers are laid out in reverse parameter order and cut into buckets of
``bucket_cap_mb``; with ``overlap=True`` (and more than one bucket) a bucket's steps 1-4 are launched on a
side stream from a post-accumulate-grad hook as soon as its last gradient is
produced, i.e. while backward is still running for earlier layers, and
``step()`` only launches the receive/update kernels.  Every rank, the sender
included, applies exactly what was transmitted (its own dense remainder stays
in its residual), so replicas stay bit-identical.  Unlike the reference the
single-rank case uses the same rule as the multi-rank case (the reference
drops the learning rate there, keras/comprex_optimizer.py:134-141).

``rule="adamw"`` exchanges the clipped gradient itself and runs AdamW in the
receive kernel.  Residuals, momentum and master weights travel in
``state_dict()`` under the key ``"comprex"``, keyed by parameter.

All six collectives of the reference (keras/comprex_optimizer.py:49-70) run through the same
bucketed, overlapped step.  ``comprex_bigring`` and ``comprex_ring`` (replica-consistent) fuse the
parameter update into their final decode; the other types, and ``consistent=False``, allreduce a
work copy of the bucket's vector in place and update from it with one dense kernel.
``allreduce_type="auto"`` picks per bucket between the dense kernels, the compressed BigRing and
the compressed Ring (``allreduce.select_schedule``).  ``aggregate_blob=False`` is the reference's
per-tensor mode (keras/comprex_optimizer.py:77-96): one allreducer per tensor.  A single rank
exchanges nothing (keras/comprex_optimizer.py:134-141): the clipped, folded gradient goes straight
into the dense update kernel.
"""
from __future__ import annotations

import warnings

import torch

from . import _lib, allreduce as _ar
from ._lib import ComprexError
from .ops import primitives as P
from .utils.trace import nvtx_range

_TYPES = {
    "alltoone": _ar.AllToOneAllreduce, "comprex_alltoone": _ar.Comprex_AllToOneAllreduce,
    "ring": _ar.RingAllreduce, "comprex_ring": _ar.Comprex_RingAllreduce,
    "bigring": _ar.BigRingAllreduce, "comprex_bigring": _ar.Comprex_BigRingAllreduce,
}


class _Bucket:
    __slots__ = ("start", "end", "params", "offsets", "ar", "ready", "sent", "seq", "par", "fold", "kind", "xbuf",
                 "plan", "u")

    def __init__(self, start):
        self.start, self.end = start, start
        self.params, self.offsets = [], []
        self.ar, self.ready, self.sent, self.fold = None, 0, False, None
        self.kind, self.xbuf, self.plan, self.u = None, None, None, None


_ITEM = 65536     # elements per fold work item
_ALIGN = 64       # tensors start on 128-byte (bf16) / 256-byte (fp32) boundaries of the flat buffers


def _dense_layout(p: torch.Tensor) -> bool:
    """True when p's elements occupy numel consecutive slots (any permutation, e.g. channels-last)."""
    if p.is_contiguous():
        return True
    size, stride = p.size(), p.stride()
    expect = 1
    for dim in sorted(range(p.dim()), key=lambda d: stride[d]):
        if size[dim] == 1:
            continue
        if stride[dim] != expect:
            return False
        expect *= size[dim]
    return True


def _same_layout(a: torch.Tensor, b: torch.Tensor) -> bool:
    return all(x == y for n, x, y in zip(a.size(), a.stride(), b.stride()) if n > 1)


class _FoldTable:
    """Static description of a bucket's tensors for the fold kernels plus the per-step
    table of gradient pointers (staged through a small ring of pinned buffers)."""

    def __init__(self, env, bucket):
        dev = env.device
        off, rel, ln, seg, first = [], [], [], [], [0]
        for si, (p, o) in enumerate(zip(bucket.params, bucket.offsets)):
            k = p.numel()
            for r in range(0, max(k, 1), _ITEM):
                off.append(o - bucket.start + r)
                rel.append(r)
                ln.append(min(_ITEM, k - r))
                seg.append(si)
            first.append(len(off))
        self.nitems, self.nseg = len(off), len(bucket.params)
        self.item_off = torch.tensor(off, dtype=torch.int64, device=dev)
        self.item_rel = torch.tensor(rel, dtype=torch.int64, device=dev)
        self.item_len = torch.tensor(ln, dtype=torch.int32, device=dev)
        self.item_seg = torch.tensor(seg, dtype=torch.int32, device=dev)
        self.seg_first = torch.tensor(first, dtype=torch.int32, device=dev)
        self.partial = torch.zeros(self.nitems, dtype=torch.float32, device=dev)
        self.ptrs = torch.zeros(self.nseg, dtype=torch.int64, device=dev)
        self.last = None
        self.cuda = dev.type == "cuda"
        if self.cuda:
            self.ring = [(torch.zeros(self.nseg, dtype=torch.int64).pin_memory(), torch.cuda.Event()) for _ in range(4)]
            self.turn = 0

    def stage(self, values) -> None:
        """Upload this step's gradient pointers (async on the current stream).  The caching
        allocator usually hands autograd the same blocks every step: an unchanged table is
        not uploaded again."""
        if values == self.last:
            return
        self.last = list(values)
        if not self.cuda:
            self.ptrs.copy_(torch.tensor(values, dtype=torch.int64))
            return
        host, ev = self.ring[self.turn]
        self.turn = (self.turn + 1) % len(self.ring)
        ev.synchronize()                      # the copy that last used this buffer has finished
        host.copy_(torch.tensor(values, dtype=torch.int64))
        self.ptrs.copy_(host, non_blocking=True)
        ev.record()



class ComprexOptimizer(torch.optim.Optimizer):
    def __init__(self, params, gaspi_env, lr=0.01, momentum=0.9, compression_ratio=0.01, nesterov=False,
                 allreduce_type="comprex_bigring", size_factor=1.0, logging=False, pre_clipnorm=5.0,
                 weight_decay=0.0, local_momentum=True, rule="sgd", betas=(0.9, 0.999), eps=1e-8,
                 learning_rate=None, bucket_cap_mb=None, overlap=False, consistent=True, aggregate_blob=True,
                 single_rank_bypass=True, name="ComprexOptimizer"):
        if learning_rate is not None:
            lr = learning_rate
        if not 0 <= momentum <= 1:
            raise ValueError("`momentum` must be between [0, 1].")
        if allreduce_type not in _TYPES and allreduce_type != "auto":
            raise ValueError("AllreduceOp with name %s is not known!" % allreduce_type)
        if rule not in ("sgd", "adamw"):
            raise ValueError("rule must be 'sgd' or 'adamw'")
        if nesterov:
            warnings.warn("ComprexOptimizer: nesterov=True is accepted for interface parity and has no effect "
                          "(the reference stores the flag and never reads it, keras/comprex_optimizer.py:33)")
        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.gaspi_env = gaspi_env
        self.name = name
        self._env = env = gaspi_env.get()
        self.compression_ratio = float(compression_ratio)
        self.nesterov = nesterov
        self.logging = logging
        self.allreduce_type = allreduce_type
        self.size_factor = float(size_factor)
        self.pre_clipnorm = pre_clipnorm
        self.local_momentum = bool(local_momentum)
        self.rule = rule
        self.betas, self.eps = betas, eps
        self.momentum_correction = 1.0
        self._t = 0
        # consistent=False is the reference's rule for the compressed collectives (a rank applies its
        # own update densely and the peers' sparsely, keras/comprex_optimizer.py:117-133 with
        # src/allreduce.tpp:649-681): replicas drift apart by what each keeps in its residual.
        self.consistent = bool(consistent)
        self.aggregate_blob = bool(aggregate_blob)
        # a job of one rank exchanges nothing (keras/comprex_optimizer.py:134-141)
        self._local = env.ranks == 1 and bool(single_rank_bypass)

        # keys: the names torch recorded when named parameters were passed, else the position
        keyed, pos = [], 0
        for g in self.param_groups:
            names = g.get("param_names")
            for i, p in enumerate(g["params"]):
                if p.requires_grad:
                    keyed.append((str(names[i]) if names else f"param{pos}", p))
                pos += 1
        if not keyed:
            raise ValueError("optimizer got an empty parameter list")
        plist = [p for _, p in keyed]
        dt = plist[0].dtype
        if any(p.dtype != dt or p.device != env.device for p in plist):
            raise ComprexError("all parameters must share one dtype and live on the environment's device")
        # reverse order: the gradients that backward produces first come first
        keyed = keyed[::-1]
        self._params = [p for _, p in keyed]
        self._keys = [k for k, _ in keyed]
        es = torch.empty(0, dtype=dt).element_size()
        cap_elems = int(bucket_cap_mb * (1 << 20) / es) if bucket_cap_mb else None
        self._buckets, self._offsets, off = [_Bucket(0)], [], 0
        for p in self._params:
            b = self._buckets[-1]
            full = cap_elems and (off - b.start) + p.numel() > cap_elems
            if b.params and (full or not self.aggregate_blob):
                off = (off + 1023) // 1024 * 1024          # buckets start on a sub-tile boundary
                b = _Bucket(off)
                self._buckets.append(b)
            self._offsets.append(off)
            b.params.append(p)
            b.offsets.append(off)
            off += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
            b.end = off
        self.blob_size = n = off
        dev = env.device
        self._dtype = dt
        self._master = torch.zeros(n, dtype=torch.float32, device=dev)
        self._shadow = torch.zeros(n, dtype=dt, device=dev) if dt != torch.float32 else None
        store = self._shadow if self._shadow is not None else self._master
        self._bucket_of = {}
        for b in self._buckets:
            for p, o in zip(b.params, b.offsets):
                k = p.numel()
                src = p.detach()
                if not _dense_layout(src):
                    src = src.contiguous()
                # the flat buffers keep the tensor's own memory order (e.g. channels-last weights)
                self._master[o:o + k].as_strided(src.size(), src.stride()).copy_(src)
                view = store[o:o + k].as_strided(src.size(), src.stride())
                view.copy_(src)
                p.data = view
                p.grad = None
                self._bucket_of[p] = b
        self._zeros = torch.zeros(max(p.numel() for p in plist), dtype=dt, device=dev)
        self._update = torch.zeros(n, dtype=torch.float32, device=dev)   # momentum_var / exchanged vector
        self._m = torch.zeros(n, dtype=torch.float32, device=dev) if rule == "adamw" or not local_momentum else None
        self._v = torch.zeros(n, dtype=torch.float32, device=dev) if rule == "adamw" else None
        self.comprex_allreducers = {}
        self._comm = None
        self._trace = None
        # with a single bucket there is nothing to overlap with: its last gradient appears when
        # backward ends, and the hooks and the side stream would only add latency
        self.overlap = bool(overlap) and dev.type == "cuda" and len(self._buckets) > 1 and not self._local
        self._armed = False
        self._hooks = []
        if self.overlap:
            for p in self._params:
                self._hooks.append(p.register_post_accumulate_grad_hook(self._on_grad))

    # ---- reference surface -----------------------------------------------------------------
    def set_compression_ratio(self, compression_ratio) -> None:
        self.compression_ratio = float(compression_ratio)
        for ar in self.comprex_allreducers.values():
            if hasattr(ar, "set_compression_ratio"):
                ar.set_compression_ratio(compression_ratio)

    def create_allreduce_op(self, name: str, size: int):
        """Collective; tag 1 and chief 0 like the reference (keras/comprex_optimizer.py:49-70)."""
        cls = _TYPES[name]
        ar = cls(self._env)
        if name == "comprex_bigring":
            ar.setup_connections(size, 1, self.compression_ratio, self.size_factor, consistent=self.consistent)
        elif name == "comprex_ring":
            ar.setup_connections(size, 1, self.compression_ratio, self.size_factor, consistent=self.consistent,
                                 chunk_align=4)
        elif name == "comprex_alltoone":
            ar.setup_connections(size, 1, 0, self.compression_ratio, self.size_factor)
        elif name == "alltoone":
            ar.setup_connections(size, 1, 0)
        elif name == "bigring":
            ar.setup_connections(size, 1, ordered=self.consistent)     # identical bits on every rank
        else:
            ar.setup_connections(size, 1)
        return ar

    def _ensure_allreducers(self) -> None:
        if self._armed:
            return
        dev = self._env.device
        for i, b in enumerate(self._buckets):
            n = b.end - b.start
            if self._local:
                b.kind = "local"
                continue
            name = self.allreduce_type
            if name == "auto":
                name = _ar.select_schedule(n, self.compression_ratio, self._env.ranks)
            b.ar = self.comprex_allreducers[i] = self.create_allreduce_op(name, n)
            if name == "comprex_bigring" and self.consistent:
                b.kind = "bigring"
            elif name == "comprex_ring" and self.consistent:
                b.kind = "ring"
            else:
                b.kind = "phased"
            if b.kind != "bigring":
                # the exchange works in place on a copy; for a dense allreduce through the switch the
                # copy lives in the symmetric heap, so that it is reduced there without staging
                in_heap = b.kind == "phased" and getattr(b.ar, "first_phase_waits", False)
                b.xbuf = self._env.empty(n) if in_heap else torch.empty(n, dtype=torch.float32, device=dev)
        self._armed = True

    def describe(self) -> str:
        """One line that names the exchange of every bucket (for logs and benchmark records)."""
        if self._local:
            return "single rank: no exchange, dense fused update"
        self._ensure_allreducers()
        kinds = {}
        for b in self._buckets:
            name = type(b.ar).__name__ + ("" if b.kind == "phased" else " (update fused into the decode)")
            kinds[name] = kinds.get(name, 0) + 1
        mode = "replica-consistent" if self.consistent else "reference semantics (own update dense)"
        return "; ".join(f"{v} x {k}" for k, v in kinds.items()) + f"; direct NVLink peer stores, {mode}"

    def zero_grad(self, set_to_none: bool = True) -> None:
        """Drop the gradients (autograd then writes fresh tensors, which the fold kernels read
        in place; no flat gradient buffer and no accumulate kernels are involved)."""
        for p in self._params:
            if set_to_none:
                p.grad = None
            elif p.grad is not None:
                p.grad.zero_()
        if getattr(self, "_trace", None) is not None:
            self._trace.clear()
            self._mark(("origin",))             # the step's timeline starts here

    # ---- the step ---------------------------------------------------------------------------------
    def _fold(self, b: _Bucket, lr: float, mu: float) -> torch.Tensor:
        """Clip per tensor and build the vector that is exchanged for one bucket: two launches
        that read the gradient tensors where autograd left them."""
        if b.fold is None:
            b.fold = _FoldTable(self._env, b)
        ft, ptrs = b.fold, []
        for p in b.params:
            g = p.grad
            if g is None:
                ptrs.append(self._zeros.data_ptr())
                continue
            if g.dtype != self._dtype or (g.stride() != p.stride() and not _same_layout(g, p)):
                g = torch.empty_strided(p.size(), p.stride(), dtype=self._dtype, device=p.device).copy_(g)  # rare
                p.grad = g
            ptrs.append(g.data_ptr())
        ft.stage(ptrs)
        u = self._update[b.start:b.end]
        local = self.rule == "sgd" and self.local_momentum
        env = self._env
        _lib.check(env.lib.cx_fold(env.dev, _lib.dtype_code(self._dtype), ft.ptrs.data_ptr(), ft.item_off.data_ptr(),
                                   ft.item_rel.data_ptr(), ft.item_len.data_ptr(), ft.item_seg.data_ptr(),
                                   ft.seg_first.data_ptr(), ft.nitems, u.data_ptr(), ft.partial.data_ptr(),
                                   float(self.pre_clipnorm) if self.pre_clipnorm is not None else 0.0,
                                   mu * self.momentum_correction if local else 0.0, lr if local else 1.0,
                                   _lib.stream_ptr(env.device)), "cx_fold")
        return u

    def _hyper(self):
        """The update kernels take one learning rate, momentum and weight decay for the whole flat
        buffer: parameter groups may exist (schedulers address them) but must agree."""
        group = self.param_groups[0]
        hyper = (float(group["lr"]), float(group["momentum"]), float(group["weight_decay"]))
        for other in self.param_groups[1:]:
            if (float(other["lr"]), float(other["momentum"]), float(other["weight_decay"])) != hyper:
                raise ComprexError("parameter groups with different lr / momentum / weight_decay are not "
                                   "supported: the fused update applies one setting to the flat buffer")
        return hyper

    def _comm_stream(self):
        if self._comm is None:
            self._comm = torch.cuda.Stream(self._env.device, priority=-1)
        return self._comm

    # ---- per-bucket timeline (CUDA events; for the overlap evidence, off by default) --------------
    def enable_timeline(self, on: bool = True) -> None:
        """Record CUDA events around every bucket's send and receive half and at the start of
        ``step`` (where backward has ended); :meth:`timeline` turns the last step's events into
        milliseconds.  Costs a few event records per bucket and step."""
        self._trace = {} if on and self._env.device.type == "cuda" else None

    def _mark(self, key) -> None:
        if getattr(self, "_trace", None) is not None:
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self._env.device))
            self._trace[key] = ev

    def timeline(self) -> dict:
        """Milliseconds since the first recorded event of the last step: per bucket
        ``send_start`` (its last gradient exists and the comm stream picks it up), ``send_end``,
        ``recv_start``, ``recv_end``; ``backward_end`` is the compute stream at the entry of
        ``step``, ``step_end`` the compute stream after it joined the comm stream."""
        tr = getattr(self, "_trace", None)
        if not tr:
            return {}
        torch.cuda.synchronize(self._env.device)
        origin = tr.get(("origin",)) or next(iter(tr.values()))     # zero_grad() marks the start of a step
        out = {"buckets": [dict(index=i, mbytes=round((b.end - b.start) * 4 / 2 ** 20, 2), kind=b.kind)
                           for i, b in enumerate(self._buckets)]}
        for key, ev in tr.items():
            ms = round(origin.elapsed_time(ev), 3)
            if len(key) == 2:
                out["buckets"][key[1]][key[0]] = ms
            elif key != ("origin",):
                out[key[0]] = ms
        return out

    def _send(self, b: _Bucket) -> None:
        """First half of a bucket's exchange: fold, then everything that waits for nobody."""
        lr, mu, _ = self._hyper()
        idx = self._buckets.index(b) if getattr(self, "_trace", None) is not None else -1
        self._mark(("send_start", idx))
        with nvtx_range("comprex.fold+send"):
            u = self._fold(b, lr, mu)
            if b.kind == "bigring":
                b.seq, b.par = b.ar.send_fast(u)
            elif b.kind == "ring":
                b.xbuf.copy_(u)
                b.seq, b.par = b.ar.send_fast(b.xbuf)
            elif b.kind == "phased":
                b.xbuf.copy_(u)
                b.plan = b.ar._plan_apply(b.xbuf)
                if b.plan and not b.ar.first_phase_waits:
                    b.plan[0]()                 # a first phase that only sends goes out right away
                    b.plan = b.plan[1:]
            else:
                b.u = u
        self._mark(("send_end", idx))
        b.sent = True

    def _recv(self, b: _Bucket, lr, mu, wd) -> None:
        """Second half: wait for the peers, reduce / decode, update the parameters."""
        env, n = self._env, b.end - b.start
        with nvtx_range("comprex.recv+update"):
            if b.kind == "bigring":
                b.ar.recv_fast(b.seq, b.par, self._args(b.start, n, lr, mu, wd, 1.0 / env.ranks))
            elif b.kind == "ring":
                b.ar.recv_fast(b.xbuf, b.seq, b.par,
                               lambda c, start, size: self._args(b.start + start, size, lr, mu, wd, 1.0 / env.ranks))
            elif b.kind == "phased":
                for phase in b.plan:
                    phase()
                b.plan = None
                P.update_dense(env, b.xbuf, n, self._args(b.start, n, lr, mu, wd, 1.0 / env.ranks))
            else:
                P.update_dense(env, b.u, n, self._args(b.start, n, lr, mu, wd, 1.0))

    def no_sync(self):
        """Context for gradient accumulation with ``overlap=True``: backward passes inside it
        only accumulate; the buckets go out during the first backward pass after it (or in
        ``step``)."""
        import contextlib

        @contextlib.contextmanager
        def ctx():
            armed, self._armed = self._armed, False
            try:
                yield
            finally:
                self._armed = armed
        return ctx()

    def _on_grad(self, p) -> None:
        if not self._armed:
            return
        b = self._bucket_of[p]
        b.ready += 1
        if b.ready < len(b.params) or b.sent:
            return
        comm = self._comm_stream()
        comm.wait_stream(torch.cuda.current_stream(self._env.device))
        with torch.cuda.stream(comm):
            self._send(b)

    def _args(self, start: int, n: int, lr, mu, wd, scale: float):
        """Receive-side update of the flat range [start, start + n): the rule and its state."""
        sl = slice(start, start + n)
        sh = None if self._shadow is None else self._shadow[sl]
        if self.rule == "adamw":
            return P.args_update(_lib.OP_ADAMW, self._master[sl], scale, shadow=sh, m=self._m[sl], v=self._v[sl],
                                 lr=lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, wd=wd, step=self._t)
        if self.local_momentum:
            return P.args_update(_lib.OP_SGD, self._master[sl], scale, shadow=sh, wd=wd)
        return P.args_update(_lib.OP_MOMENTUM, self._master[sl], scale, shadow=sh, m=self._m[sl], lr=lr,
                             momentum=mu * self.momentum_correction, wd=wd)

    def _recv_args(self, b: _Bucket, lr, mu, wd):
        return self._args(b.start, b.end - b.start, lr, mu, wd, 1.0 / self._env.ranks)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        lr, mu, wd = self._hyper()
        self._t += 1
        first = not self._armed
        self._ensure_allreducers()
        use_side = self.overlap and not first
        self._mark(("backward_end",))
        if use_side:
            comm = self._comm_stream()
            comm.wait_stream(torch.cuda.current_stream(self._env.device))
            ctx = torch.cuda.stream(comm)
        else:
            import contextlib
            ctx = contextlib.nullcontext()
        with ctx:
            for b in self._buckets:          # everything that the hooks did not send yet
                if not b.sent:
                    self._send(b)
            for i, b in enumerate(self._buckets):   # then receive: all peers' payloads are on their way
                self._mark(("recv_start", i))
                self._recv(b, lr, mu, wd)
                self._mark(("recv_end", i))
                b.sent, b.ready = False, 0
        if use_side:
            torch.cuda.current_stream(self._env.device).wait_stream(comm)
        self._mark(("step_end",))
        self._env.maybe_check()
        return loss

    def apply_gradients(self, grads_and_vars, *args, **kwargs):
        """Keras-style entry (keras/comprex_optimizer.py:144-145): ``(gradient, variable)`` pairs are
        installed as the variables' ``.grad`` and one step is taken."""
        for g, v in grads_and_vars:
            v.grad = g
        return self.step()

    def refresh_master(self) -> None:
        """Take the model's current tensors as the master weights: call it after the parameters
        were overwritten from outside (a weight broadcast, a manual edit).  With fp32 parameters
        the model's tensors are the master buffer itself and nothing needs to happen."""
        if self._shadow is not None:
            self._master.copy_(self._shadow)

    def flush(self) -> None:
        """Apply everything still held in residuals (end of training)."""
        if not self.comprex_allreducers:
            return
        for b in self._buckets:
            ar = b.ar
            if ar is None or not ar.compressed:
                continue
            buf = torch.zeros(ar.size, dtype=torch.float32, device=self._env.device)
            ar.flush(buf)
            if self.rule == "sgd" and self.local_momentum:
                # residuals hold lr-scaled updates: apply them like a received update
                sl = slice(b.start, b.start + ar.size)
                self._master[sl].sub_(buf / self._env.ranks)
                if self._shadow is not None:
                    self._shadow[sl].copy_(self._master[sl])

    def stats(self) -> dict:
        """Statistics of the first bucket's last compression (synchronises)."""
        ar = self._buckets[0].ar
        return ar.stats() if ar is not None and ar.compressed else {}

    # ---- checkpoint ---------------------------------------------------------------------------------
    def _layout(self):
        """(key, offset, numel) of every parameter in the flat buffers."""
        return [(k, int(o), int(p.numel())) for k, o, p in zip(self._keys, self._offsets, self._params)]

    def _residual_flat(self):
        """The buckets' main residuals as one vector in the layout of the flat buffers."""
        if not self.comprex_allreducers:
            return None
        flat = torch.zeros(self.blob_size, dtype=torch.float32)
        for b in self._buckets:
            r = getattr(b.ar, "rests", None) if b.ar is not None else None
            if r is not None:
                flat[b.start:b.start + r.numel()] = r.detach().cpu()
        return flat

    def state_dict(self):
        sd = super().state_dict()
        self._env.flush()
        ars = [b.ar for b in self._buckets]
        sd["comprex"] = {
            "version": 2, "world_size": self._env.ranks, "rank": self._env.rank, "ratio": self.compression_ratio,
            "topology": self.allreduce_type, "step": self._t, "rule": self.rule,
            "layout": self._layout(), "buckets": [(b.start, b.end, type(b.ar).__name__) for b in self._buckets],
            "master": self._master.detach().cpu().clone(), "update": self._update.detach().cpu().clone(),
            "m": None if self._m is None else self._m.detach().cpu().clone(),
            "v": None if self._v is None else self._v.detach().cpu().clone(),
            "residual": self._residual_flat(),
            "allreduce": [a.state_dict() if a is not None and a.compressed else None for a in ars],
        }
        return sd

    def _remap(self, flat, layout):
        """A flat vector saved under ``layout`` rearranged into this optimizer's layout, by key."""
        if flat is None:
            return None
        saved = {k: (o, n) for k, o, n in layout}
        out = torch.zeros(self.blob_size, dtype=flat.dtype)
        for k, o, n in self._layout():
            if k not in saved or saved[k][1] != n:
                raise ComprexError(f"checkpoint has no parameter '{k}' of {n} elements: it was written for another model")
            so = saved[k][0]
            out[o:o + n] = flat[so:so + n]
        return out

    def load_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        cs = state_dict.pop("comprex", None)
        layout, mine = None, self._layout()
        if cs is not None:
            layout = cs.get("layout")
            if layout is None:                              # version 1: flat vectors in this layout or nothing
                if cs["master"].numel() != self.blob_size:
                    raise ComprexError("checkpoint belongs to a model of a different size")
                layout = mine
            if len(layout) != len(mine) or {k for k, _, _ in layout} != {k for k, _, _ in mine}:
                raise ComprexError("checkpoint was written for other parameters (names or count differ)")
        super().load_state_dict(state_dict)
        if cs is None:
            return
        same_layout = [tuple(x) for x in layout] == mine
        pick = (lambda t: t) if same_layout else (lambda t: self._remap(t, layout))
        dev = self._env.device
        self._t = cs["step"]
        # Weights and the Adam moments are replicated, so any rank's file restores them.  The
        # local momentum and the residuals are this rank's own: a file written by another rank
        # (a new rank of a larger job, or everybody loading rank 0's file) starts them at zero.
        foreign = int(cs.get("rank", self._env.rank)) != self._env.rank
        self._master.copy_(pick(cs["master"]).to(dev))
        if foreign:
            self._update.zero_()
        else:
            self._update.copy_(pick(cs["update"]).to(dev))
        if self._m is not None and cs["m"] is not None:
            self._m.copy_(pick(cs["m"]).to(dev))
        if self._v is not None and cs["v"] is not None:
            self._v.copy_(pick(cs["v"]).to(dev))
        if self._shadow is not None:
            self._shadow.copy_(self._master)
        if any(s is not None for s in cs["allreduce"]) and not self._local:
            self._ensure_allreducers()
            saved_buckets = cs.get("buckets")
            same_buckets = (same_layout and cs["world_size"] == self._env.ranks and
                            (saved_buckets is None or [tuple(x) for x in saved_buckets] ==
                             [(b.start, b.end, type(b.ar).__name__) for b in self._buckets]))
            residual = None if cs.get("residual") is None else pick(cs["residual"])
            for i, b in enumerate(self._buckets):
                if b.ar is None or not b.ar.compressed:
                    continue
                if foreign:
                    b.ar.reset()
                elif same_buckets and i < len(cs["allreduce"]) and cs["allreduce"][i] is not None:
                    b.ar.load_state_dict(cs["allreduce"][i])
                else:
                    # another bucket layout, schedule or world size: every parameter keeps what this
                    # rank had not sent yet (the residual follows the parameter, not the bucket);
                    # secondary residuals (a ring owner's) start at zero
                    b.ar.reset()
                    r = getattr(b.ar, "rests", None)
                    if r is not None and residual is not None:
                        r.copy_(residual[b.start:b.start + r.numel()].to(dev))
                    elif r is not None and i < len(cs["allreduce"]) and cs["allreduce"][i] is not None:
                        src = cs["allreduce"][i]["residuals"][0]          # version 1 file, same buckets
                        if src.numel() == r.numel():
                            r.copy_(src.to(dev))
        # every reducer, restored or reset, selects with the checkpoint's ratio from here on
        self.set_compression_ratio(cs["ratio"])
