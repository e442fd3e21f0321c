"""Dense exchange demo (the reference's examples/gaspiEx.py): rank 0 sends a vector to
rank 1 many times, rank 1 accumulates; at the end the sum must be exact.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/gaspiEx.py
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
    comm = cx.GaspiEx(env, n)
    t0 = time.time()
    if rank == 0:
        comm.connectTx(1, 1)
        for _ in range(runs):
            comm.writeRemote(values)
            env.barrier()
    elif rank == 1:
        comm.connectRx(0, 1)
        acc = torch.zeros(n, device=env.device)
        for _ in range(runs):
            comm.readRemote_add(acc)
            env.barrier()
        ok = torch.equal(acc, runs * values)
        cx.gaspi_printf("+++ PASSED +++" if ok else "--- FAILED ---")
    else:
        for _ in range(runs):
            env.barrier()
    env.barrier()
    cx.gaspi_printf("Runtime: %.1f ms" % ((time.time() - t0) * 1e3))
    env.close()


if __name__ == "__main__":
    main()
