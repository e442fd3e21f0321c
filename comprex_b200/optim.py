"""Compressed data-parallel optimizer (reference: keras/comprex_optimizer.py:8-170).

The reference hooks into Keras' ``_aggregate_gradients``: per tensor it clips
the gradient to an L2 norm of ``pre_clipnorm``, folds it into a *local*
momentum buffer scaled by the learning rate (``mom = m*mom + lr*g``),
concatenates everything into one blob, allreduces the blob with one of six
collectives (default ``comprex_bigring``), divides by the number of ranks and
applies ``var = (1-wd)*var - update``.  This class keeps those semantics for
PyTorch and maps them onto three kernel launches per step and blob:

1. threshold estimate of ``residual + update`` (device resident),
2. fused ``residual += update`` / select / store pairs into every peer's slot,
3. fused wait / scatter-add in rank order / average / parameter update, which
   also refreshes the low-precision copy of the weights when the model is held
   in bf16 or fp16.

The parameters live in one flat fp32 master buffer (the model's tensors are
views of it, or of its low-precision shadow), gradients accumulate directly
into one flat buffer, so no concatenation or slicing copy happens.  Every
rank, the sender included, applies exactly what was transmitted (its own dense
remainder stays in its residual), so replicas stay bit-identical.  Unlike the
reference the single-rank case uses the same rule as the multi-rank case (the
reference drops the learning rate there, keras/comprex_optimizer.py:134-141).

``rule="adamw"`` exchanges the clipped gradient itself and runs AdamW in the
receive kernel.  Residuals, momentum and master weights travel in
``state_dict()`` under the key ``"comprex"``.
"""
from __future__ import annotations

import torch

from . import _lib, allreduce as _ar
from ._lib import ComprexError
from .ops import primitives as P

_TYPES = {
    "alltoone": _ar.AllToOneAllreduce, "comprex_alltoone": _ar.Comprex_AllToOneAllreduce,
    "ring": _ar.RingAllreduce, "comprex_ring": _ar.Comprex_RingAllreduce,
    "bigring": _ar.BigRingAllreduce, "comprex_bigring": _ar.Comprex_BigRingAllreduce,
}


class ComprexOptimizer(torch.optim.Optimizer):
    def __init__(self, params, gaspi_env, lr=0.01, momentum=0.9, compression_ratio=0.01, nesterov=False,
                 allreduce_type="comprex_bigring", size_factor=1.0, logging=False, pre_clipnorm=5.0,
                 weight_decay=0.0, local_momentum=True, rule="sgd", betas=(0.9, 0.999), eps=1e-8,
                 learning_rate=None):
        if learning_rate is not None:
            lr = learning_rate
        if not 0 <= momentum <= 1:
            raise ValueError("`momentum` must be between [0, 1].")
        if allreduce_type not in _TYPES:
            raise ValueError("AllreduceOp with name %s is not known!" % allreduce_type)
        if rule not in ("sgd", "adamw"):
            raise ValueError("rule must be 'sgd' or 'adamw'")
        defaults = dict(lr=lr, momentum=momentum, weight_decay=weight_decay)
        super().__init__(params, defaults)
        self.gaspi_env = gaspi_env
        self._env = env = gaspi_env.get()
        self.compression_ratio = float(compression_ratio)
        self.nesterov = nesterov          # accepted and unused, like the reference
        self.logging = logging
        self.allreduce_type = allreduce_type
        self.size_factor = float(size_factor)
        self.pre_clipnorm = pre_clipnorm
        self.local_momentum = bool(local_momentum)
        self.rule = rule
        self.betas, self.eps = betas, eps
        self.momentum_correction = 1.0
        self._t = 0

        plist = [p for g in self.param_groups for p in g["params"] if p.requires_grad]
        if not plist:
            raise ValueError("optimizer got an empty parameter list")
        dt = plist[0].dtype
        if any(p.dtype != dt or p.device != env.device for p in plist):
            raise ComprexError("all parameters must share one dtype and live on the environment's device")
        self._params = plist
        # 16-byte aligned segments keep every tensor view vectorisable
        self._offsets, off = [], 0
        for p in plist:
            self._offsets.append(off)
            off += (p.numel() + 3) // 4 * 4
        self.blob_size = n = off
        dev = env.device
        self._master = torch.zeros(n, dtype=torch.float32, device=dev)
        self._shadow = torch.zeros(n, dtype=dt, device=dev) if dt != torch.float32 else None
        self._grad = torch.zeros(n, dtype=dt, device=dev)
        store = self._shadow if self._shadow is not None else self._master
        for p, o in zip(plist, self._offsets):
            k = p.numel()
            self._master[o:o + k].copy_(p.detach().reshape(-1))
            store[o:o + k].copy_(p.detach().reshape(-1))
            p.data = store[o:o + k].view_as(p)
            p.grad = self._grad[o:o + k].view_as(p)
        self._grad_views = [self._grad[o:o + p.numel()] for p, o in zip(plist, self._offsets)]
        self._update = torch.zeros(n, dtype=torch.float32, device=dev)   # momentum_var / exchanged vector
        self._m = torch.zeros(n, dtype=torch.float32, device=dev) if rule == "adamw" or not local_momentum else None
        self._v = torch.zeros(n, dtype=torch.float32, device=dev) if rule == "adamw" else None
        self.comprex_allreducers = {}
        self._allreduce = None

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
            ar.setup_connections(size, 1, self.compression_ratio, self.size_factor, consistent=True)
        elif name == "comprex_ring":
            ar.setup_connections(size, 1, self.compression_ratio, self.size_factor)
        elif name == "comprex_alltoone":
            ar.setup_connections(size, 1, 0, self.compression_ratio, self.size_factor)
        elif name == "alltoone":
            ar.setup_connections(size, 1, 0)
        else:
            ar.setup_connections(size, 1)
        return ar

    def zero_grad(self, set_to_none: bool = False) -> None:
        """Zero the flat gradient buffer; the per-parameter views stay attached."""
        self._grad.zero_()
        for p, o in zip(self._params, self._offsets):
            if p.grad is None or p.grad.data_ptr() != self._grad.data_ptr() + o * self._grad.element_size():
                p.grad = self._grad[o:o + p.numel()].view_as(p)

    # ---- the step ---------------------------------------------------------------------------------
    def _clip_coefficients(self):
        if self.pre_clipnorm is None:
            return None
        norms = torch._foreach_norm(self._grad_views)
        clip = float(self.pre_clipnorm)
        # tf.clip_by_norm: g * clip / max(norm, clip)
        return [clip / torch.clamp(nrm.float(), min=clip) for nrm in norms]

    def _fold(self, lr: float, mu: float) -> torch.Tensor:
        """Clip per tensor and build the vector that is exchanged."""
        coefs = self._clip_coefficients()
        if coefs is not None:
            torch._foreach_mul_(self._grad_views, [c.to(self._grad.dtype) for c in coefs])
        if self.rule == "sgd" and self.local_momentum:
            self._update.mul_(mu * self.momentum_correction).add_(self._grad, alpha=lr)
            return self._update
        if self._grad.dtype == torch.float32:
            return self._grad
        self._update.copy_(self._grad)
        return self._update

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        group = self.param_groups[0]
        lr, mu, wd = float(group["lr"]), float(group["momentum"]), float(group["weight_decay"])
        self._t += 1
        x = self._fold(lr, mu)
        if self._allreduce is None:
            self._allreduce = self.comprex_allreducers[0] = self.create_allreduce_op(self.allreduce_type, self.blob_size)
        ar, nr = self._allreduce, self._env.ranks
        if self.rule == "adamw":
            args = P.args_update(_lib.OP_ADAMW, self._master, 1.0 / nr, shadow=self._shadow, m=self._m, v=self._v,
                                 lr=lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, wd=wd, step=self._t)
        elif self.local_momentum:
            args = P.args_update(_lib.OP_SGD, self._master, 1.0 / nr, shadow=self._shadow, wd=wd)
        else:
            args = P.args_update(_lib.OP_MOMENTUM, self._master, 1.0 / nr, shadow=self._shadow, m=self._m, lr=lr,
                                 momentum=mu * self.momentum_correction, wd=wd)
        if isinstance(ar, _ar.Comprex_BigRingAllreduce):
            for phase in ar._plan_apply(x, recv_args=args):
                phase()
        else:
            self._generic_step(ar, x, lr, mu, wd)
        self._env.maybe_check()
        return loss

    def _generic_step(self, ar, x, lr, mu, wd) -> None:
        """Other collectives: allreduce a copy of the vector in place, then update with tensor ops."""
        if getattr(self, "_xbuf", None) is None:
            self._xbuf = torch.empty(self.blob_size, dtype=torch.float32, device=self._env.device)
        buf = self._xbuf
        buf.copy_(x)
        ar.apply(buf)
        avg = buf.div_(self._env.ranks)
        if self.rule == "adamw":
            b1, b2 = self.betas
            self._m.mul_(b1).add_(avg, alpha=1 - b1)
            self._v.mul_(b2).addcmul_(avg, avg, value=1 - b2)
            mh = self._m / (1 - b1 ** self._t)
            vh = self._v / (1 - b2 ** self._t)
            self._master.mul_(1 - lr * wd).addcdiv_(mh, vh.sqrt_().add_(self.eps), value=-lr)
        elif self.local_momentum:
            self._master.mul_(1 - wd).sub_(avg)
        else:
            self._m.mul_(mu * self.momentum_correction).add_(avg, alpha=lr)
            self._master.mul_(1 - wd).sub_(self._m)
        if self._shadow is not None:
            self._shadow.copy_(self._master)

    def flush(self) -> None:
        """Apply everything still held in residuals (end of training)."""
        if self._allreduce is None or not self._allreduce.compressed:
            return
        buf = torch.zeros(self.blob_size, dtype=torch.float32, device=self._env.device)
        self._allreduce.flush(buf)
        if self.rule == "sgd" and self.local_momentum:
            # residuals hold lr-scaled updates: apply them like a received update
            self._master.sub_(buf / self._env.ranks)
            if self._shadow is not None:
                self._shadow.copy_(self._master)

    def stats(self) -> dict:
        return self._allreduce.stats() if self._allreduce is not None and self._allreduce.compressed else {}

    # ---- checkpoint ---------------------------------------------------------------------------------
    def state_dict(self):
        sd = super().state_dict()
        ar = self._allreduce
        sd["comprex"] = {
            "version": 1, "world_size": self._env.ranks, "rank": self._env.rank, "ratio": self.compression_ratio,
            "topology": self.allreduce_type, "step": self._t, "rule": self.rule,
            "master": self._master.detach().cpu().clone(), "update": self._update.detach().cpu().clone(),
            "m": None if self._m is None else self._m.detach().cpu().clone(),
            "v": None if self._v is None else self._v.detach().cpu().clone(),
            "allreduce": ar.state_dict() if ar is not None and ar.compressed else None,
        }
        return sd

    def load_state_dict(self, state_dict):
        state_dict = dict(state_dict)
        cs = state_dict.pop("comprex", None)
        super().load_state_dict(state_dict)
        if cs is None:
            return
        if cs["master"].numel() != self.blob_size:
            raise ComprexError("checkpoint belongs to a model of a different size")
        dev = self._env.device
        self._t = cs["step"]
        self.compression_ratio = cs["ratio"]
        self._master.copy_(cs["master"].to(dev))
        self._update.copy_(cs["update"].to(dev))
        if self._m is not None and cs["m"] is not None:
            self._m.copy_(cs["m"].to(dev))
        if self._v is not None and cs["v"] is not None:
            self._v.copy_(cs["v"].to(dev))
        if self._shadow is not None:
            self._shadow.copy_(self._master)
        if cs["allreduce"] is not None:
            if self._allreduce is None:
                self._allreduce = self.comprex_allreducers[0] = self.create_allreduce_op(self.allreduce_type, self.blob_size)
            if cs["world_size"] == self._env.ranks:
                self._allreduce.load_state_dict(cs["allreduce"])
            else:
                # residuals are rank-local errors: a restart with another world size keeps
                # what this rank had and starts the new ranks from zero
                for dst, src in zip(self._allreduce._residuals(), cs["allreduce"]["residuals"]):
                    if dst.numel() == src.numel():
                        dst.copy_(src.to(dev))
