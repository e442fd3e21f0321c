"""Plain PyTorch / Python restatements used as oracles by the tests."""

import numpy as np
import torch


def ref_threshold_topk(x: torch.Tensor, ratio: float, default_subsamples=1000, subsample_factor=10.0) -> float:
    """ThresholdTopK of the reference (src/threshold.hxx:182-240) on x = rests + input (fp32, CPU)."""
    x = x.detach().float().cpu().numpy()
    n = x.size
    subs = default_subsamples
    if ratio > 0:
        req = np.float32(subsample_factor) / np.float32(ratio)
        if req > default_subsamples:
            subs = int(req)
    if n < subs:
        sample = np.abs(x)
    else:
        step = np.float32(n) / np.float32(subs)
        pos = (np.arange(subs, dtype=np.float32) * step).astype(np.int64)
        pos = np.minimum(pos, n - 1)
        sample = np.abs(x[pos])
    topk_pos = int(np.ceil(np.float32(sample.size) * np.float32(ratio)) - 1)
    if topk_pos <= 0:
        return float(np.float32(sample.max()) + np.float32(1.0))
    return float(np.sort(sample)[::-1][topk_pos])


def ref_compress(g, r, thr, cap=None):
    """IndexPairs compress_add_update (src/compressor.hxx:568-581) with a capacity limit.
    Returns (idx, val, new_r)."""
    v = (r if r is not None else 0) + (g.float() if g is not None else 0)
    sel = v.abs() > thr
    idx = torch.nonzero(sel).flatten()
    if cap is not None and idx.numel() > cap:
        idx = idx[:cap]
    val = v[idx]
    new_r = v.clone()
    new_r[idx] = 0
    return idx.to(torch.int32), val, new_r


def alt_ramp(n, device="cpu"):
    """values[i] = i * (1 - 2*(i % 2)), the reference tests' data (test/comprex.cpp:44-47)."""
    i = torch.arange(n, device=device)
    return (i * (1 - 2 * (i % 2))).float()
