"""Where the time of one compress launch goes: %globaltimer stamps taken inside the kernel.

Needs the library built with the stamps compiled in (they are off by default):

    COMPREX_NVCC_EXTRA="-DCX_COMPRESS_TRACE" python -m comprex_b200.build --force
    python bench/compress_phases.py [--log2-sizes 20 22 24 26] [--ratio 0.01] [--no-flush]

Thread 0 of every CTA stamps: entry, start of the sub-tile loop, end of the loop, arrival at the
completion counter, and (in the CTA that arrives last) regions summed, headers published, end.
Printed per size: the CUDA-event time of the launch and the stamps in nanoseconds since the first
CTA's entry (median over the timed launches; L2 flushed before every launch unless --no-flush).
"""
import argparse
import ctypes as C
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import comprex_b200 as cx  # noqa: E402
from comprex_b200.ops import primitives as P  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--log2-sizes", type=int, nargs="+", default=[20, 22, 24, 26])
    ap.add_argument("--ratio", type=float, default=0.01)
    ap.add_argument("--targets", type=int, default=7)
    ap.add_argument("--iters", type=int, default=8)
    ap.add_argument("--no-flush", action="store_true")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    for lg in args.log2_sizes:
        n = 1 << lg
        cap = max(int(2 * args.ratio * n), 1024)
        env = cx.GaspiEnvironment(int(args.targets * (8 * cap + 8 * (n // 1024 + 1) + 4096) + (64 << 20)), device=dev)
        lib = env.lib
        if not hasattr(lib, "cx_compress_trace"):
            raise SystemExit("the library was built without -DCX_COMPRESS_TRACE (see the docstring)")
        lib.cx_compress_trace.argtypes = [C.c_void_p, C.c_int]
        lib.cx_compress_trace.restype = C.c_int
        slots = [P.SparseSlot.create(env, n, cap) for _ in range(args.targets)]
        tg = P.make_targets([s.endpoint(env) for s in slots])
        comp = P.Compressor(env, n)
        g = torch.randn(n, device=dev)
        r = torch.randn(n, device=dev) * 0.5
        flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
        res = []
        nb = min(2 * torch.cuda.get_device_properties(dev).multi_processor_count, (n // 1024 + 7) // 8)
        for it in range(args.iters):
            comp.threshold_topk(g, r, n, args.ratio)
            torch.cuda.synchronize()
            if not args.no_flush:
                flush.add_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            comp.compress(g, r, n, cap, it + 1, tg)
            b.record()
            torch.cuda.synchronize()
            buf = (C.c_ulonglong * (8 * nb))()
            if lib.cx_compress_trace(buf, 8 * nb) != 0:
                raise SystemExit("reading the stamps failed")
            t = [[buf[8 * i + k] for i in range(nb)] for k in range(8)]
            t0 = min(t[0])
            last = max(range(nb), key=lambda i: t[3][i])        # the CTA that arrived last
            if it >= 3:
                res.append((a.elapsed_time(b) * 1e3, statistics.median(t[1]) - t0, min(t[2]) - t0, max(t[2]) - t0,
                            statistics.median(t[3]) - t0, t[3][last] - t0, t[4][last] - t0, t[5][last] - t0,
                            t[6][last] - t0))
        m = [statistics.median(x[i] for x in res) for i in range(9)]
        print(f"n=2^{lg} ctas={nb} event_us={m[0]:.1f} | ns since the first entry: loop start {m[1]:.0f}, loop end "
              f"{m[2]:.0f}..{m[3]:.0f}, arrived median {m[4]:.0f} last {m[5]:.0f}, regions summed {m[6]:.0f}, "
              f"published {m[7]:.0f}, end {m[8]:.0f}", flush=True)
        env.close()


if __name__ == "__main__":
    main()
