"""Two-rank exchange ping-pong: time and bandwidth vs size (the reference's
examples/comprex_speed.cpp: ``writeRemote`` + ``readRemote_add`` each way, sizes
1e5 ... 5e8 bytes, top-k 10 % / 1 % / 0.1 %, bandwidth ``2*n*4/t``), dense GaspiEx and
compressed Comprex, device-timed with CUDA events, max over the two ranks.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 bench/p2p_pingpong.py --out results/p2p.jsonl
"""
import argparse
import json
import os
import statistics
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import comprex_b200 as cx  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=float, nargs="+", default=[1e5, 1e6, 1e7, 1e8, 5e8])
    ap.add_argument("--ratios", type=float, nargs="+", default=[0.1, 0.01, 0.001])
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    cx.initGaspiCxx("nccl")
    rank = dist.get_rank()
    if dist.get_world_size() != 2:
        raise SystemExit("run with exactly two ranks")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    env = cx.GaspiEnvironment(256 << 20, device=dev)
    peer = 1 - rank
    rows = []
    for nbytes in args.bytes:
        n = int(nbytes) // 4
        x = torch.randn(n, device=dev)
        acc = torch.zeros(n, device=dev)
        for ratio in [1.0] + args.ratios:
            mark = env.heap_mark()
            if ratio == 1.0:
                comm = cx.GaspiEx(env, n)
            else:
                comm = cx.Comprex(env, n, max(4 * ratio, 2e-3))
                comm.setThreshold(cx.ThresholdTopK(ratio))
            comm.connectTo(peer, peer, 1)
            times = []
            for i in range(args.reps + 3):
                torch.cuda.synchronize(dev)
                dist.barrier()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                comm.writeRemote(x)
                comm.readRemote_add(acc)
                b.record()
                torch.cuda.synchronize(dev)
                t = torch.tensor([a.elapsed_time(b) * 1e3], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                if i >= 3:
                    times.append(float(t.item()))
            med = statistics.median(times)
            row = {"bytes": int(nbytes), "ratio": ratio, "engine": "GaspiEx" if ratio == 1.0 else "Comprex",
                   "us_median": round(med, 2), "effective_MBps": round(2 * n * 4 / med, 1)}
            rows.append(row)
            if rank == 0:
                print(json.dumps(row), flush=True)
            del comm
            env.heap_release(mark)
    if args.out and rank == 0:
        os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
        with open(args.out, "w") as f:
            for row in rows:
                f.write(json.dumps(row) + "\n")
    env.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
