"""Single-GPU timing of the exchange kernels against their memory roofline.

For every (n, ratio, dtype) it times, with CUDA events on the launching stream
after warm-up and with an L2 flush between iterations:

* ``threshold``  - sampled top-k threshold estimate,
* ``compress``   - fused residual add / select / per-sub-tile compaction / store into
                   ``--targets`` slots (local memory stands in for peers),
* ``residual_add_torch`` - ``torch.add(r, g, out=r)``: the same dense traffic through torch's own
                   elementwise kernel, as the size-matched reference for the compress rows,
* ``apply_add``  - wait + scatter-add of ``--sources`` payloads,
* ``apply_set``  - wait + dense result (sum of the payloads, zero elsewhere): the receive side of
                   the replica-consistent allreduce,
* ``apply_sgd`` / ``apply_adamw`` - the same fused with the parameter update.

Algorithmic bytes: compress reads g and r and writes r (plus 8 B per pair and
target); apply reads the pairs and touches one 32-byte sector per pair (sparse
ops) or reads/writes the dense state once (dense ops).  Fractions are "of
measured": the copy bandwidth in MEASURED_PEAKS.json at the repository root
when present (6.65 TB/s otherwise, "of fallback").

Below about 2^24 elements the figures are bound by the host's launch path (one ctypes
call per timed launch), not by the kernels.

    python bench/kernel_bench.py --out results/kernel_bench.jsonl
"""
import argparse
import json
import os
import statistics
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import comprex_b200 as cx  # noqa: E402
from comprex_b200 import _lib  # noqa: E402
from comprex_b200.ops import primitives as P  # noqa: E402


def peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def timed(fn, iters, flush, reps=1):
    """Median / best device time of one launch in microseconds.

    ``reps`` > 1 queues that many launches behind a long-running filler kernel, so the
    events bracket back-to-back kernels and not the host's launch latency (used for
    vectors that fit in L2 anyway, where a flush between launches would not be the
    situation a training step sees)."""
    times = []
    for _ in range(iters):
        flush.add_(1)          # flushes L2 and keeps the GPU busy while the launches queue up
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b) * 1e3 / reps)
    return statistics.median(times), min(times)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", type=int, nargs="+", default=[1 << 20, 1 << 24, 1 << 26, 1 << 28])
    ap.add_argument("--ratios", type=float, nargs="+", default=[0.001, 0.01, 0.1])
    ap.add_argument("--dtypes", nargs="+", default=["fp32", "bf16"])
    ap.add_argument("--targets", type=int, default=7)
    ap.add_argument("--sources", type=int, default=7)
    ap.add_argument("--iters", type=int, default=7)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--kernels", nargs="+", default=None, help="only these rows (threshold, compress, apply_add, ...)")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    peak, how = peak_gbs()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)  # larger than the 126 MB L2
    rows = []
    for n in args.sizes:
        for ratio in args.ratios:
            cap = int(n * ratio * 2) + 1024
            env = cx.GaspiEnvironment(1 << 20, device=dev)
            nslots = max(args.targets, args.sources)
            slots = [P.SparseSlot.create(env, n, cap) for _ in range(nslots)]
            comp = P.Compressor(env, n)
            st = env.new_status("bench")
            for dname in args.dtypes:
                dt = torch.float32 if dname == "fp32" else torch.bfloat16
                g = torch.randn(n, device=dev).to(dt)
                r = torch.randn(n, device=dev) * 0.5
                w = torch.randn(n, device=dev)
                m = torch.zeros(n, device=dev)
                v = torch.zeros(n, device=dev)
                out = torch.zeros(n, device=dev)
                tg = P.make_targets([s.endpoint(env) for s in slots[: args.targets]])
                seq = [0]

                def k_thr():
                    comp.threshold_topk(g, r, n, ratio)

                def k_comp():
                    seq[0] += 1
                    comp.compress(g, r, n, cap, seq[0], tg)

                def k_stream():
                    # torch's elementwise kernel with the compress kernel's dense traffic (read g and r,
                    # write r): what a plain streaming kernel reaches at this size, cold caches included
                    torch.add(r, g, out=r)

                def k_add():
                    src = P.make_sources([s.endpoint(env) for s in slots[: args.sources]], [1] * args.sources)
                    P.apply_sparse(env, src, n, P.args_add(out, 1.0 / 8), st)

                def k_set():
                    src = P.make_sources([s.endpoint(env) for s in slots[: args.sources]], [1] * args.sources)
                    P.apply_sparse(env, src, n, P.args_set(out, 1.0 / 8), st)

                def k_sgd():
                    src = P.make_sources([s.endpoint(env) for s in slots[: args.sources]], [1] * args.sources)
                    P.apply_sparse(env, src, n, P.args_update(_lib.OP_SGD, w, 1.0 / 8), st)

                def k_adamw():
                    src = P.make_sources([s.endpoint(env) for s in slots[: args.sources]], [1] * args.sources)
                    P.apply_sparse(env, src, n, P.args_update(_lib.OP_ADAMW, w, 1.0 / 8, m=m, v=v, lr=1e-3, wd=0.01), st)

                gb = torch.empty(0, dtype=dt).element_size()
                for _ in range(args.warmup):
                    k_thr(); k_comp(); k_add()
                nnz = comp.last_stats()["nnz"]
                kernels = {
                    "threshold": (k_thr, 0),
                    "compress": (k_comp, n * (gb + 8) + 8 * nnz * args.targets),
                    "residual_add_torch": (k_stream, n * (gb + 8)),
                    "apply_add": (k_add, args.sources * nnz * (8 + 64)),
                    "apply_set": (k_set, args.sources * nnz * 8 + 4 * n),
                    "apply_sgd": (k_sgd, args.sources * nnz * (8 + 64)),
                    "apply_adamw": (k_adamw, args.sources * nnz * 8 + 24 * n),
                }
                r0 = r.clone()
                for name, (fn, nbytes) in kernels.items():
                    if name not in ("compress", "residual_add_torch") and dname != args.dtypes[0]:
                        continue   # only the compress kernel reads the gradient dtype
                    if args.kernels and name not in args.kernels:
                        continue
                    if name == "apply_add":
                        # the receive kernels see a payload of the nominal density again: the timed
                        # compress calls above fed the same gradient into a growing residual
                        r.copy_(r0)
                        k_thr()
                        k_comp()
                        nnz = comp.last_stats()["nnz"]
                        for key in ("apply_add", "apply_sgd"):
                            kernels[key] = (kernels[key][0], args.sources * nnz * (8 + 64))
                        kernels["apply_set"] = (kernels["apply_set"][0], args.sources * nnz * 8 + 4 * n)
                        kernels["apply_adamw"] = (kernels["apply_adamw"][0], args.sources * nnz * 8 + 24 * n)
                        nbytes = kernels[name][1]
                    for _ in range(args.warmup):
                        fn()
                    reps = 10 if n * 12 < (100 << 20) else 1
                    med, best = timed(fn, args.iters, flush, reps)
                    row = {"kernel": name, "n": n, "ratio": ratio, "dtype": dname, "nnz": nnz, "reps": reps,
                           "targets": args.targets, "sources": args.sources, "us_median": round(med, 2),
                           "us_min": round(best, 2), "algo_bytes": nbytes,
                           "gbs": round(nbytes / med / 1e3, 1) if nbytes else None,
                           "frac_of_" + how: round(nbytes / med / 1e3 / peak, 3) if nbytes else None}
                    rows.append(row)
                    print(json.dumps(row), flush=True)
                env.flush()
                del g, r, w, m, v, out
            env.close()
            torch.cuda.empty_cache()
    if args.out:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            for row in rows:
                f.write(json.dumps(row) + "\n")


if __name__ == "__main__":
    main()
