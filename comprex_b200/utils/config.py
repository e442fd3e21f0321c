"""One configuration object for the library (the reference has none: its knobs are CMake
options, constructor arguments and module constants, see keras/comprex_optimizer.py:11-46
and LeNet/main.py:16-24).

``ComprexConfig`` gathers them, takes overrides from ``COMPREX_<FIELD>`` environment
variables (upper-case field name) and from an ``argparse`` namespace, and builds the
objects that consume them::

    cfg = ComprexConfig.from_env(compression_ratio=0.001)
    env = cfg.environment()
    opt = cfg.optimizer(model.parameters(), env, lr=0.1)
    model.register_comm_hook(cfg.hook_state(env), comprex_hook)
"""
from __future__ import annotations

import argparse
import dataclasses
import os
from dataclasses import dataclass

_TOPOLOGIES = ("comprex_bigring", "comprex_ring", "comprex_alltoone", "bigring", "ring", "alltoone", "auto")


@dataclass
class ComprexConfig:
    # what is sent
    compression_ratio: float = 0.01          # top-k fraction
    threshold: str = "topk"                  # "topk" | "const" | "none"
    threshold_value: float = 0.0             # for threshold == "const"
    default_subsamples: int = 1000           # sampling of the top-k estimate (src/threshold.hxx:182-205)
    subsample_factor: float = 10.0
    compressor: str = "pairs"                # "pairs" | "rle" | "none"
    size_factor: float = 1.0                 # receive slot = size * 4 * size_factor bytes (src/comprEx.tpp:61)
    # how it is exchanged
    topology: str = "comprex_bigring"
    consistent: bool = True                  # replicas apply exactly what was transmitted (bit-identical)
    stale: bool = False                      # FastComprEx semantics: payloads arrive one call late
    ring_schedule: str = "direct"            # compressed Ring: "direct" stores or the reference's "hops"
    exact_topk: bool = False                 # threshold from a select over the whole vector
    two_shot_bytes: int = 1 << 20            # dense BigRing: reduce-scatter + allgather above this size
    dense_fallback_bytes: int = 64 << 10     # DDP hook: buckets below this go out dense
    capacity_slack: float = 2.0              # DDP hook: slot room over the expected survivors
    # optimizer
    rule: str = "sgd"                        # "sgd" | "adamw"
    local_momentum: bool = True
    pre_clipnorm: float = 5.0
    bucket_cap_mb: float = 25.0
    overlap: bool = True
    aggregate_blob: bool = True              # False: one allreducer per tensor (keras/comprex_optimizer.py:77-96)
    # runtime
    segment_bytes: int = 1 << 30             # symmetric heap per rank
    timeout_ms: int = 10000                  # budget of every device-side wait
    sync_check: bool = False                 # synchronise and check the status words after every call
    dtype_policy: str = "fp32_master"        # fp32 master weights with a low-precision shadow

    def __post_init__(self) -> None:
        if not 0.0 <= self.compression_ratio <= 1.0:
            raise ValueError("compression_ratio must be between 0 and 1")
        if self.topology not in _TOPOLOGIES:
            raise ValueError(f"topology must be one of {_TOPOLOGIES}")
        if self.threshold not in ("topk", "const", "none"):
            raise ValueError("threshold must be 'topk', 'const' or 'none'")
        if self.compressor not in ("pairs", "rle", "none"):
            raise ValueError("compressor must be 'pairs', 'rle' or 'none'")
        if self.rule not in ("sgd", "adamw"):
            raise ValueError("rule must be 'sgd' or 'adamw'")
        if self.ring_schedule not in ("direct", "hops"):
            raise ValueError("ring_schedule must be 'direct' or 'hops'")

    # ---- sources of overrides -------------------------------------------------------------------
    @staticmethod
    def _coerce(field: dataclasses.Field, text: str):
        kind = field.type if isinstance(field.type, str) else field.type.__name__
        if kind == "bool":
            return text.strip().lower() in ("1", "true", "yes", "on")
        if kind == "int":
            return int(float(text)) if any(c in text for c in ".eE") else int(text, 0)
        if kind == "float":
            return float(text)
        return text

    @classmethod
    def from_env(cls, environ=None, **overrides) -> "ComprexConfig":
        """Defaults, then ``COMPREX_<FIELD>`` variables, then keyword arguments."""
        environ = os.environ if environ is None else environ
        values = {}
        for f in dataclasses.fields(cls):
            text = environ.get("COMPREX_" + f.name.upper())
            if text is not None:
                values[f.name] = cls._coerce(f, text)
        values.update(overrides)
        return cls(**values)

    @classmethod
    def add_arguments(cls, parser: argparse.ArgumentParser) -> argparse.ArgumentParser:
        """One ``--comprex-<field>`` option per field (defaults stay with the dataclass)."""
        group = parser.add_argument_group("comprex")
        for f in dataclasses.fields(cls):
            group.add_argument("--comprex-" + f.name.replace("_", "-"), dest="comprex_" + f.name, default=None,
                               metavar=str(f.type), help=f"default {f.default!r}")
        return parser

    @classmethod
    def from_args(cls, namespace: argparse.Namespace, environ=None) -> "ComprexConfig":
        overrides = {}
        for f in dataclasses.fields(cls):
            text = getattr(namespace, "comprex_" + f.name, None)
            if text is not None:
                overrides[f.name] = cls._coerce(f, text) if isinstance(text, str) else text
        return cls.from_env(environ, **overrides)

    def to_dict(self) -> dict:
        return dataclasses.asdict(self)

    # ---- builders -------------------------------------------------------------------------------------
    def environment(self, device=None):
        from ..parallel.env import GaspiEnvironment
        env = GaspiEnvironment(self.segment_bytes, device=device, timeout_ms=self.timeout_ms)
        if self.sync_check:
            env.sync_check = True
        return env

    def threshold_object(self):
        from .. import ComprEx as E
        if self.threshold == "topk":
            return E.ThresholdTopK(self.compression_ratio, self.default_subsamples, self.subsample_factor,
                                   exact=self.exact_topk)
        if self.threshold == "const":
            return E.ThresholdConst(self.threshold_value)
        return E.ThresholdNone()

    def compressor_object(self):
        from .. import ComprEx as E
        return {"pairs": E.CompressorIndexPairs, "rle": E.CompressorRLE, "none": E.CompressorNone}[self.compressor]()

    def engine(self, env, size: int):
        """A point-to-point engine (``Comprex`` or, with ``stale``, ``FastComprex``)."""
        from .. import ComprEx as E
        eng = (E.FastComprex if self.stale else E.Comprex)(env, size, self.size_factor)
        eng.setThreshold(self.threshold_object())
        if self.compressor != "pairs":
            eng.setCompressor(self.compressor_object())
        return eng

    def allreduce(self, env, size: int, tag: int = 0):
        """An allreduce object of the configured topology, connections set up."""
        from .. import allreduce as A
        cls = {"comprex_bigring": A.Comprex_BigRingAllreduce, "comprex_ring": A.Comprex_RingAllreduce,
               "comprex_alltoone": A.Comprex_AllToOneAllreduce, "bigring": A.BigRingAllreduce,
               "ring": A.RingAllreduce, "alltoone": A.AllToOneAllreduce, "auto": A.AutoAllreduce}[self.topology]
        ar = cls(env)
        if self.topology == "comprex_bigring":
            ar.setup_connections(size, tag, self.compression_ratio, self.size_factor, consistent=self.consistent)
        elif self.topology == "auto":
            ar.setup_connections(size, tag, self.compression_ratio, self.size_factor, consistent=self.consistent)
        elif self.topology == "comprex_ring":
            # the hop-by-hop ring is the reference's schedule with the reference's semantics
            ar.setup_connections(size, tag, self.compression_ratio, self.size_factor,
                                 consistent=self.consistent and self.ring_schedule == "direct",
                                 schedule=self.ring_schedule)
        elif self.topology == "comprex_alltoone":
            ar.setup_connections(size, tag, 0, self.compression_ratio, self.size_factor, stale=self.stale)
        elif self.topology == "alltoone":
            ar.setup_connections(size, tag, 0)
        elif self.topology == "bigring":
            ar.setup_connections(size, tag, two_shot_bytes=self.two_shot_bytes)
        else:
            ar.setup_connections(size, tag)
        if self.exact_topk and ar.compressed:
            getattr(ar, "impl", ar).set_exact_topk(True)
        return ar

    def optimizer(self, params, env, **kwargs):
        from ..optim import ComprexOptimizer
        args = dict(compression_ratio=self.compression_ratio, allreduce_type=self.topology,
                    size_factor=self.size_factor, pre_clipnorm=self.pre_clipnorm,
                    local_momentum=self.local_momentum, rule=self.rule, consistent=self.consistent,
                    bucket_cap_mb=self.bucket_cap_mb, overlap=self.overlap, aggregate_blob=self.aggregate_blob)
        args.update(kwargs)
        return ComprexOptimizer(params, env, **args)

    def hook_state(self, env):
        from ..ddp_hook import ComprexHookState
        return ComprexHookState(env, compression_ratio=self.compression_ratio, capacity_slack=self.capacity_slack,
                                dense_fallback_bytes=self.dense_fallback_bytes)
