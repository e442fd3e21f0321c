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
same tensor, the speed-up against it, the nominal top-k and the fraction of the
vector that was actually sent, and the roofline fraction: the slower of (bytes
the kernels must move through HBM) / (measured copy bandwidth) and (bytes that
must cross this GPU's NVLink port in one direction) / (the peer-store bandwidth
measured at the start of the run: one kernel storing 256 MiB into one peer and
into all peers), divided by the time.  ``--exact-control`` adds, for every
compressed cell, a run with the exact top-k threshold (``set_exact_topk``) so
that speed-ups can be read at the nominal ratio too.
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

NVLINK_GBS = 770.0        # peer-copy rate of this pool; replaced by the store bandwidth measured in the run


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


def measure_store_bandwidth(env, dev, world, rank, flush, nbytes=256 << 20):
    """One kernel storing ``nbytes`` into one peer's memory, then into every peer's: GB/s out of
    this GPU (CUDA events, max over ranks of the time; all ranks store at the same moment, so the
    figure is what a port sustains in both directions at once)."""
    from comprex_b200.ops import primitives as P
    n = nbytes // 4
    x = torch.ones(n, device=dev)
    mark = env.heap_mark()
    slots = [P.DenseSlot.create(env, nbytes) for _ in range(world)]      # slot r: what rank r sends
    counters = env.scratch(64)
    peers = [r for r in range(world) if r != rank]
    seq = [0]

    def send(targets):
        seq[0] += 1
        P.dense_send(env, x, None, n, seq[0], targets, counters)
    one = P.make_targets([slots[rank].endpoint(env, (rank + 1) % world)])
    every = P.make_targets([slots[rank].endpoint(env, r) for r in peers])          # plain stores, P-1 copies
    t_one, _ = time_op(lambda: send(one), 5, 2, flush, dev)
    t_all, _ = time_op(lambda: send(every), 5, 2, flush, dev)
    row = {"variant": "p2p_store_bandwidth", "bytes": nbytes, "ranks": world,
           "one_peer_gbs": round(nbytes / t_one / 1e3, 1),
           "all_peers_egress_gbs": round((world - 1) * nbytes / t_all / 1e3, 1)}
    mc = slots[rank].mc_endpoint(env)
    if mc is not None and world > 2:
        multi = P.make_targets([slots[rank].endpoint(env, r) for r in peers], mc=mc)  # one multimem store
        t_mc, _ = time_op(lambda: send(multi), 5, 2, flush, dev)
        row["multicast_ingress_gbs"] = round((world - 1) * nbytes / t_mc / 1e3, 1)
    env.flush()
    del slots
    env.heap_release(mark)
    return row


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--log2-sizes", type=int, nargs="+", default=[16, 18, 20, 22, 24, 26, 28])
    ap.add_argument("--ratios", type=float, nargs="+", default=[0.001, 0.01, 0.1])
    ap.add_argument("--variants", nargs="+", default=["comprex_bigring", "comprex_ring", "comprex_alltoone",
                                                      "bigring", "ring", "ring_inplace", "alltoone", "auto"])
    ap.add_argument("--dtypes", nargs="+", default=["fp32", "bf16"])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--max-log2-onetoall", type=int, default=26,
                    help="largest size for the schedules that hold P full-size slots (dense BigRing, AllToOne)")
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--heap-gb", type=float, default=16.0, help="upper bound of the first heap segment")
    ap.add_argument("--no-p2p", action="store_true", help="skip the peer-store bandwidth measurement")
    ap.add_argument("--exact-control", action="store_true",
                    help="also run every compressed cell with the exact top-k threshold")
    ap.add_argument("--out", default=None)
    ap.add_argument("--csv", default=None,
                    help="also write the reference benchmark's table (examples/allreduce_speed.cpp:182-184): "
                         "variant;size(MB);compression;time_mean(us);time_stddev(us);sparsity_mean;sparsity_stddev")
    args = ap.parse_args()

    cx.initGaspiCxx("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    # one heap segment that holds the largest cell (2 P slots of 8 B x 0.2 n pairs for the compressed
    # BigRing at 10 %): cells then reuse it instead of mapping fresh peer / multicast memory each time
    nmax = 1 << max(args.log2_sizes)
    # the dense AllToOne keeps 2 P + 2 full-size slots (two parities per sender at the chief, two for
    # the broadcast): with --max-log2-onetoall raised, the heap has to hold them
    n_one = 1 << min(max(args.log2_sizes), args.max_log2_onetoall)
    need_one = (2 * world + 2) * 4 * n_one + 2 * 4 * n_one if "alltoone" in args.variants else 0
    heap = int(min(args.heap_gb * (1 << 30), max(256 << 20, 2 * world * 1.7 * nmax + 3 * 4 * nmax, need_one)))
    env = cx.GaspiEnvironment(heap, device=dev)
    flush = None if args.no_flush else torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    peak, how = hbm_gbs()
    rows = []

    def emit(row):
        rows.append(row)
        if rank == 0:
            print(json.dumps({k: v for k, v in row.items() if k != "csv"}), flush=True)

    link_gbs, link_how = NVLINK_GBS, "peer-copy figure"
    if world > 1 and not args.no_p2p:
        bw = measure_store_bandwidth(env, dev, world, rank, flush)
        emit(bw)
        link_gbs, link_how = max(bw["one_peer_gbs"], bw["all_peers_egress_gbs"]), "measured store bandwidth"

    def roofline(variant, n, es, sent, mm):
        """(HBM bytes, link bytes in the busier direction) of one call on one GPU."""
        p = world
        pairs = 8.0 * sent * n + 8.0 * n / 1024           # one rank's payload: pairs + table
        if variant == "comprex_bigring":
            return 12.0 * n, (p - 1) * pairs                # compress pass; everyone's payload comes in
        if variant == "comprex_ring":
            return 16.0 * n, 2.0 * (p - 1) / p * pairs      # two compress passes over n(P-1)/P + n/P, decode; two exchanges
        if variant == "comprex_alltoone":
            return 24.0 * n, (p - 1) * pairs                # the chief: decode, compress, P-1 payloads in and out
        if variant == "alltoone":
            return 3.0 * n * es, (p - 1) * n * es           # the chief's port carries every worker's vector
        if mm:
            return 2.0 * n * es, (p + 1.0) / p * n * es     # in-switch reduction: n out, n/P + n in (staging copies not counted)
        return 3.0 * n * es, 2.0 * (p - 1) / p * n * es     # reduce-scatter + allgather

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
                compressed = variant.startswith("comprex") or variant == "auto"
                # the schedules that keep P full-size slots (or a full-size residual per rank at the
                # chief) stop where those no longer fit next to the vector
                if variant in ("alltoone", "comprex_alltoone") and lg > args.max_log2_onetoall:
                    emit({"variant": variant, "n": n, "dtype": dname, "ranks": world, "skipped": "slots do not fit"})
                    continue
                for ratio, exact in [(r, e) for r in (args.ratios if compressed else [1.0])
                                     for e in ((False, True) if compressed and args.exact_control else (False,))]:
                    mark = env.heap_mark()
                    cls = {"comprex_bigring": cx.Comprex_BigRingAllreduce, "comprex_ring": cx.Comprex_RingAllreduce,
                           "comprex_alltoone": cx.Comprex_AllToOneAllreduce, "bigring": cx.BigRingAllreduce,
                           "ring": cx.RingAllreduce, "ring_inplace": cx.RingAllreduce,
                           "alltoone": cx.AllToOneAllreduce, "auto": cx.AutoAllreduce}[variant]
                    ar = cls(env)
                    sf = max(4.0 * ratio, 2e-3)     # slots hold twice the expected survivors
                    if variant == "comprex_bigring":
                        ar.setup_connections(n, 1, ratio, sf, consistent=True)
                    elif variant == "comprex_ring":
                        ar.setup_connections(n, 1, ratio, sf, chunk_align=8)
                    elif variant == "comprex_alltoone":
                        ar.setup_connections(n, 1, 0, ratio, sf)
                    elif variant == "alltoone":
                        ar.setup_connections(n, 1, 0, dtype=dt)
                    elif variant == "auto":
                        ar.setup_connections(n, 1, ratio, sf, dtype=dt)
                    else:
                        ar.setup_connections(n, 1, dtype=dt)
                    if exact:
                        (ar.impl if variant == "auto" else ar).set_exact_topk() if getattr(ar, "compressed", False) else None
                    # "ring_inplace": the vector lives in the symmetric heap (env.empty), like the
                    # reference's buffers live in its registered segment: no staging copies
                    buf = env.empty(n, dt) if variant == "ring_inplace" else x.clone()

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
                    kind, sent = ("ring" if variant == "ring_inplace" else variant), 1.0
                    if variant == "auto":
                        kind = row["chosen"] = ar.choice
                    st = ar.stats() if getattr(ar, "compressed", False) else None
                    if st:
                        sent = st["nnz"] / max(st["n"], 1)
                        row["nominal_topk"] = ratio
                        row["exact_topk"] = exact
                        row["sent_fraction"] = round(sent, 5)
                        row["overflow"] = bool(st["status"] & 4)
                        row["result_sparsity"] = res_sparsity
                    mm = bool(getattr(getattr(ar, "impl", ar), "_mm", None))
                    if mm:
                        row["through_switch"] = True
                    hbm_b, link_b = roofline(kind, n, x.element_size(), sent, mm)
                    roof_us = max(hbm_b / (peak * 1e3), link_b / (link_gbs * 1e3))
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
