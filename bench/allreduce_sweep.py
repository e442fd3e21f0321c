"""Allreduce time vs size and top-k ratio on P GPUs, against dense NCCL.

The counterpart of the reference's examples/allreduce_speed.cpp (variants
AllToOne / Ring / BigRing, dense and compressed, mean time per size), measured
the way this package's numbers are defined: device time of ``apply`` with CUDA
events on the launching stream, after warm-up, ranks aligned by a barrier before
every repetition, an L2 flush between repetitions, and the MAX over ranks of
every repetition before the median is taken.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench/allreduce_sweep.py \
        --out results/sweep_p8.jsonl

Every row carries the dense ``torch.distributed.all_reduce`` (NCCL) time of the
same tensor, the speed-up against it, the fraction of the vector that was sent,
and for the compressed BigRing the roofline fraction: the slower of (bytes the
compress kernel must move through HBM) / (measured copy bandwidth) and (bytes
that must leave over NVLink) / (770 GB/s per direction), divided by the time.
"""
import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import comprex_b200 as cx  # noqa: E402

NVLINK_GBS = 770.0


def hbm_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def time_op(fn, reps, warmup, flush, dev, after=None, samples=None):
    """Median and minimum over the repetitions of the MAX over ranks; ``after`` runs outside the
    timed region of every repetition, ``samples`` receives the individual times."""
    out = []
    for i in range(warmup + reps):
        if flush is not None:
            flush.add_(1)
        torch.cuda.synchronize(dev)
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize(dev)
        t = torch.tensor([a.elapsed_time(b) * 1e3], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if after is not None and i >= warmup:
            after()
        if i >= warmup:
            out.append(float(t.item()))
    if samples is not None:
        samples.extend(out)
    return statistics.median(out), min(out)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--log2-sizes", type=int, nargs="+", default=[16, 18, 20, 22, 24, 26, 28])
    ap.add_argument("--ratios", type=float, nargs="+", default=[0.001, 0.01, 0.1])
    ap.add_argument("--variants", nargs="+", default=["comprex_bigring", "comprex_ring", "comprex_alltoone",
                                                      "bigring", "ring", "alltoone"])
    ap.add_argument("--dtypes", nargs="+", default=["fp32", "bf16"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--max-log2-onetoall", type=int, default=26,
                    help="largest size for the schedules that hold P full-size slots (dense BigRing, AllToOne)")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--out", default=None)
    ap.add_argument("--csv", default=None,
                    help="also write the reference benchmark's table (examples/allreduce_speed.cpp:182-184): "
                         "variant;size(MB);compression;time_mean(us);time_stddev(us);sparsity_mean;sparsity_stddev")
    args = ap.parse_args()

    cx.initGaspiCxx("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    env = cx.GaspiEnvironment(256 << 20, device=dev)
    flush = None if args.no_flush else torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    peak, how = hbm_gbs()
    rows = []

    def emit(row):
        rows.append(row)
        if rank == 0:
            print(json.dumps({k: v for k, v in row.items() if k != "csv"}), flush=True)

    for lg in args.log2_sizes:
        n = 1 << lg
        for dname in args.dtypes:
            dt = torch.float32 if dname == "fp32" else torch.bfloat16
            torch.manual_seed(1000 + rank)
            x = torch.randn(n, device=dev).to(dt)
            work = x.clone()
            nccl_med, nccl_min = time_op(lambda: dist.all_reduce(work), args.reps, args.warmup, flush, dev)
            emit({"variant": "nccl_dense", "n": n, "dtype": dname, "ranks": world, "us_median": round(nccl_med, 2),
                  "us_min": round(nccl_min, 2),
                  "busbw_gbs": round(2 * (world - 1) / world * n * x.element_size() / nccl_med / 1e3, 1)})
            for variant in args.variants:
                compressed = variant.startswith("comprex")
                if compressed and dname != "fp32":
                    continue   # compressed payloads and residuals are fp32; bf16 enters through the optimizer
                if variant in ("bigring", "alltoone", "comprex_alltoone") and lg > args.max_log2_onetoall:
                    continue
                for ratio in (args.ratios if compressed else [1.0]):
                    mark = env.heap_mark()
                    cls = {"comprex_bigring": cx.Comprex_BigRingAllreduce, "comprex_ring": cx.Comprex_RingAllreduce,
                           "comprex_alltoone": cx.Comprex_AllToOneAllreduce, "bigring": cx.BigRingAllreduce,
                           "ring": cx.RingAllreduce, "alltoone": cx.AllToOneAllreduce}[variant]
                    ar = cls(env)
                    sf = max(4.0 * ratio, 2e-3)     # slots hold twice the expected survivors
                    if variant == "comprex_bigring":
                        ar.setup_connections(n, 1, ratio, sf, consistent=True)
                    elif variant == "comprex_ring":
                        ar.setup_connections(n, 1, ratio, sf)
                    elif variant == "comprex_alltoone":
                        ar.setup_connections(n, 1, 0, ratio, sf)
                    elif variant == "alltoone":
                        ar.setup_connections(n, 1, 0, dtype=dt)
                    else:
                        ar.setup_connections(n, 1, dtype=dt)
                    buf = x.clone()

                    def run():
                        buf.copy_(x)
                        ar.apply(buf)

                    def copy_only():
                        buf.copy_(x)
                    times, sparsity = [], []
                    med, best = time_op(run, args.reps, args.warmup, flush, dev, samples=times,
                                        after=(lambda: sparsity.append(float((buf == 0).float().mean()))) if args.csv else None)
                    res_sparsity = round(float((buf == 0).float().mean()), 4)   # of the last result
                    cmed, _ = time_op(copy_only, 3, 1, flush, dev)   # the input reset is not part of the allreduce
                    med, best = max(med - cmed, 0.01), max(best - cmed, 0.01)
                    env.flush()
                    row = {"variant": variant, "n": n, "dtype": dname, "ranks": world, "ratio": ratio,
                           "us_median": round(med, 2), "us_min": round(best, 2), "nccl_us": round(nccl_med, 2),
                           "speedup_vs_nccl": round(nccl_med / med, 2)}
                    if compressed:
                        st = ar.stats()
                        row["sent_fraction"] = round(st["nnz"] / max(st["n"], 1), 5)
                        row["overflow"] = bool(st["status"] & 4)
                        row["result_sparsity"] = res_sparsity
                        if variant == "comprex_bigring":
                            hbm_b = 12.0 * n
                            link_b = (world - 1) * (8.0 * st["nnz"] + 8.0 * n / 1024)
                            roof_us = max(hbm_b / (peak * 1e3), link_b / (NVLINK_GBS * 1e3))
                            row["roofline_us"] = round(roof_us, 2)
                            row["frac_of_roofline_" + how] = round(roof_us / med, 3)
                    if args.csv:
                        ts = [max(t - cmed, 0.01) for t in times]
                        row["csv"] = (variant, n * x.element_size() / 1e6, ratio, statistics.mean(ts),
                                      statistics.pstdev(ts), statistics.mean(sparsity), statistics.pstdev(sparsity))
                    emit(row)
                    del ar, buf
                    env.heap_release(mark)
            del x, work
            torch.cuda.empty_cache()
    if args.csv and rank == 0:
        os.makedirs(os.path.dirname(os.path.abspath(args.csv)), exist_ok=True)
        with open(args.csv, "w") as f:
            f.write("variant;size(MB);compression;time_mean(us);time_stddev(us);sparsity_mean;sparsity_stddev\n")
            for row in rows:
                if "csv" in row:
                    v = row["csv"]
                    f.write(f"{v[0]};{v[1]:.6g};{v[2]:g};{v[3]:.2f};{v[4]:.2f};{v[5]:.5f};{v[6]:.5f}\n")
    for row in rows:
        row.pop("csv", None)
    if args.out and rank == 0:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            for row in rows:
                f.write(json.dumps(row) + "\n")
    env.barrier()
    env.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
