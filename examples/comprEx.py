"""Compressed exchange demo (the reference's examples/comprEx.py / comprEx.cpp): top-k 1 %
with residual accumulation, the last round flushes the residual; the receiver's sum must
equal ``runs * values`` exactly, i.e. thresholding loses nothing.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/comprEx.py
"""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import comprex_b200 as cx  # noqa: E402


def main():
    cx.initGaspiCxx()
    env = cx.GaspiEnvironment(64 << 20)
    rank, n, runs = env.get_rank(), 100_000, 100  # runs * n < 2^24: exact in fp32
    i = torch.arange(n, device=env.device)
    values = (i * (1 - 2 * (i % 2))).float()
    comm = cx.Comprex(env, n, 3.0)
    comm.setThreshold(cx.ThresholdTopK(0.01))
    comm.setCompressor(cx.CompressorIndexPairs())
    t0 = time.time()
    if rank == 0:
        comm.connectTx(1, 1)
        for _ in range(runs - 1):
            comm.writeRemote(values)
            env.barrier()
        comm.flushRests()
        env.barrier()
    elif rank == 1:
        comm.connectRx(0, 1)
        acc = torch.zeros(n, device=env.device)
        for _ in range(runs):
            comm.readRemote_add(acc)
            env.barrier()
        ok = torch.equal(acc, (runs - 1) * values)
        cx.gaspi_printf("+++ PASSED +++" if ok else "--- FAILED ---")
    else:
        for _ in range(runs):
            env.barrier()
    env.barrier()
    cx.gaspi_printf("Runtime: %.1f ms" % ((time.time() - t0) * 1e3))
    env.close()


if __name__ == "__main__":
    main()
