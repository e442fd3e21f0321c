"""Configuration object, timers and logging helpers."""
import argparse
import json

import pytest
import torch

import comprex_b200 as cx
from comprex_b200.utils import ComprexConfig, JsonlWriter, PhaseTimer, StepLogger, TictocTimer, nvtx_range


def test_config_defaults_env_and_args():
    cfg = ComprexConfig()
    assert (cfg.compression_ratio, cfg.dense_fallback_bytes, cfg.bucket_cap_mb) == (0.01, 64 << 10, 25.0)
    env = {"COMPREX_COMPRESSION_RATIO": "0.001", "COMPREX_OVERLAP": "0", "COMPREX_TIMEOUT_MS": "250",
           "COMPREX_TOPOLOGY": "comprex_ring", "COMPREX_TWO_SHOT_BYTES": "1e6"}
    cfg = ComprexConfig.from_env(env, size_factor=3.0)
    assert cfg.compression_ratio == 0.001 and cfg.overlap is False and cfg.timeout_ms == 250
    assert cfg.topology == "comprex_ring" and cfg.size_factor == 3.0 and cfg.two_shot_bytes == 1000000
    ap = ComprexConfig.add_arguments(argparse.ArgumentParser())
    ns = ap.parse_args(["--comprex-compression-ratio", "0.1", "--comprex-rule", "adamw"])
    cfg = ComprexConfig.from_args(ns, env)
    assert cfg.compression_ratio == 0.1 and cfg.rule == "adamw" and cfg.timeout_ms == 250
    with pytest.raises(ValueError):
        ComprexConfig(topology="tree")
    with pytest.raises(ValueError):
        ComprexConfig(compression_ratio=1.5)
    assert ComprexConfig(**cfg.to_dict()) == cfg


def test_config_builds_objects(device):
    cfg = ComprexConfig(compression_ratio=0.05, size_factor=3.0, segment_bytes=8 << 20, timeout_ms=500,
                        bucket_cap_mb=0.004, overlap=False)
    env = cfg.environment(device)
    assert isinstance(cfg.threshold_object(), cx.ThresholdTopK) and cfg.threshold_object().getTopK() == 0.05
    ar = cfg.allreduce(env, 5000)
    x = torch.ones(5000, device=device)
    ar.apply(x)
    assert torch.isfinite(x).all()
    params = [torch.nn.Parameter(torch.randn(300, 7, device=device)), torch.nn.Parameter(torch.randn(999, device=device))]
    opt = cfg.optimizer(params, env, lr=0.1)
    assert len(opt._buckets) > 1 and opt.compression_ratio == 0.05
    for p in params:
        p.grad = torch.ones_like(p)
    opt.step()
    eng = ComprexConfig(compressor="rle", threshold="const", threshold_value=0.5, segment_bytes=8 << 20).engine(env, 100)
    assert eng.compressor.kind == "rle" and eng.threshold.getThreshold() == 0.5
    ring = ComprexConfig(topology="comprex_ring", ring_schedule="hops", exact_topk=True, segment_bytes=8 << 20)
    ar2 = ring.allreduce(env, 3000)
    assert ar2.schedule == "hops" and ar2._subsamples > 10 ** 9 and ring.threshold_object().exact
    a2o = ComprexConfig(topology="comprex_alltoone", stale=True, segment_bytes=8 << 20).allreduce(env, 3000)
    assert a2o.stale
    with pytest.raises(ValueError):
        ComprexConfig(ring_schedule="tree")
    state = cfg.hook_state(env)
    assert state.compression_ratio == 0.05 and state.dense_fallback_bytes == 64 << 10
    env.close()


def test_timers_and_logging(tmp_path, device):
    t = PhaseTimer(device)
    for _ in range(3):
        with t.phase("work"), nvtx_range("work"):
            torch.ones(1000, device=device).sum()
    s = t.summary()
    assert s["work"]["count"] == 3 and s["work"]["total_ms"] >= 0.0
    tt = TictocTimer()
    tt.tic(); tt.toc(); tt.tic(); tt.toc()
    assert tt.laps == 2 and tt.get_elapsed_time_in_sec() >= 0.0
    with pytest.raises(RuntimeError):
        tt.toc()
    path = tmp_path / "m" / "metrics.jsonl"
    w = JsonlWriter(str(path))
    w.write(step=1, loss=0.5)
    w.write(step=2, loss=0.25)
    rows = [json.loads(line) for line in open(path)]
    assert [r["step"] for r in rows] == [1, 2] and "time" in rows[0]
    log = StepLogger(None, every=2, path=str(tmp_path / "steps.jsonl"), rank=0)
    assert log(loss=1.0, samples=8) is None
    rec = log(loss=0.5, samples=8)
    assert rec["step"] == 2 and rec["loss"] == 0.5 and rec["samples_per_s"] > 0


def test_prefetcher_and_async_scalar(device):
    from comprex_b200.utils import AsyncScalar, DevicePrefetcher
    pin = device != "cpu" and torch.cuda.is_available()
    host = [(torch.full((4, 3), float(i)), torch.tensor([i])) for i in range(5)]
    if pin:
        host = [(a.pin_memory(), b.pin_memory()) for a, b in host]
    feed = DevicePrefetcher(host, device, depth=2)
    seen, readers = [], []
    for x, y in feed:
        assert x.device.type == torch.device(device).type
        readers.append(AsyncScalar(x.sum() + y.sum()))
        seen.append(int(y.item()))
    assert seen == [0, 1, 2, 3, 4]
    assert [r.value() for r in readers] == [13.0 * i for i in range(5)]
    single = list(DevicePrefetcher([torch.ones(2), torch.zeros(2)], device))
    assert len(single) == 2 and float(single[0].sum()) == 2.0
    if pin:
        assert feed.h2d_bytes == 5 * (12 * 4 + 8)
