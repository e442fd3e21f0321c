"""Data-parallel training in one object (the reference wires the same pieces by hand in
LeNet/main.py:36-129: a data shard per rank, ``BroadcastInitWeights``, the compressed optimizer,
optionally ``SynchWeights`` every few epochs).

    dp = DataParallel(model, env, config=ComprexConfig(compression_ratio=0.01), lr=0.01 * env.get_ranks(),
                      momentum=0.9, sync_every=0)
    idx = dp.shard(len(dataset))                 # this rank's slice of the sample indices
    for epoch in range(epochs):
        dp.on_epoch_begin()
        for x, y in batches(idx):
            dp.zero_grad(); loss_fn(model(x), y).backward(); dp.step()
    torch.save(dp.state_dict(), path)
"""
from __future__ import annotations

import torch

from ..callbacks import SynchWeights, broadcast_parameters
from ..utils.config import ComprexConfig


class DataParallel:
    def __init__(self, model: torch.nn.Module, gaspi_env, config: ComprexConfig | None = None, src: int = 0,
                 sync_every: int = 0, **optimizer_kwargs):
        self.model, self.env = model, gaspi_env.get()
        self.config = config or ComprexConfig()
        broadcast_parameters(model, self.env, src)                 # same initial weights everywhere
        self.optimizer = self.config.optimizer(model.parameters(), self.env, **optimizer_kwargs)
        self._sync = SynchWeights(sync_every, src, self.env) if sync_every > 0 else None
        if self._sync is not None:
            self._sync.on_train_begin(model)

    # ---- data --------------------------------------------------------------------------------------
    def shard(self, n: int) -> range:
        """This rank's contiguous share of ``n`` samples (equal sizes, the remainder is dropped
        like in LeNet/main.py:42-47)."""
        per = n // self.env.ranks
        return range(self.env.rank * per, (self.env.rank + 1) * per)

    # ---- step ---------------------------------------------------------------------------------------
    def zero_grad(self) -> None:
        self.optimizer.zero_grad()

    def step(self, closure=None):
        return self.optimizer.step(closure)

    def no_sync(self):
        return self.optimizer.no_sync()

    def on_epoch_begin(self) -> None:
        """Periodic weight synchronisation (``sync_every`` epochs; 0 = never)."""
        if self._sync is None:
            return
        before = self._sync.epoch_counter
        self._sync.on_epoch_begin(self.model)
        if self._sync.epoch_counter < before + 1:                   # a broadcast happened
            self.optimizer.refresh_master()

    def flush(self) -> None:
        """Apply everything still held in residuals (end of training)."""
        self.optimizer.flush()

    # ---- checkpoint -----------------------------------------------------------------------------------
    def state_dict(self) -> dict:
        return {"model": self.model.state_dict(), "optimizer": self.optimizer.state_dict(),
                "config": self.config.to_dict()}

    def load_state_dict(self, state: dict) -> None:
        """Restore model and optimizer.  The model's own state goes in first: its buffers
        (BatchNorm running statistics and the like) live only there; its parameters are views of
        the optimizer's flat weights, which the optimizer state then sets authoritatively."""
        if state.get("model") is not None:
            self.model.load_state_dict(state["model"])
        self.optimizer.load_state_dict(state["optimizer"])
