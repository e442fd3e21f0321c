"""DistributedDataParallel with the compressed communication hook and a stock torch optimizer.

The other way to use the library: keep ``torch.optim`` and let DDP's gradient buckets go
through top-k compression with error feedback (the PyTorch form of the reference's
TensorFlow allreduce ops, allreduceOp.py:8-143).  The hook state is picklable, so the
residuals are saved next to the model and the optimizer.

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/ddp_hook_train.py --steps 200

Runs on GPUs (one process per GPU, NCCL only for DDP's own rendezvous) or on CPU ranks (gloo).
"""
import argparse
import os
import pickle
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch.nn.parallel import DistributedDataParallel as DDP

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import comprex_b200 as cx  # noqa: E402
from comprex_b200.ddp_hook import ComprexHookState, comprex_hook  # noqa: E402
from comprex_b200.models.lenet import LeNet5  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--ratio", type=float, default=0.01)
    ap.add_argument("--checkpoint", default=None, help="file to save model, optimizer and hook state to")
    args = ap.parse_args()
    cx.initGaspiCxx()
    env = cx.GaspiEnvironment(64 << 20)
    rank, ranks, dev = env.get_rank(), env.get_ranks(), env.device
    torch.manual_seed(0)
    model = LeNet5().to(dev)
    ddp = DDP(model, device_ids=[dev.index] if dev.type == "cuda" else None)
    state = ComprexHookState(env, compression_ratio=args.ratio, dense_fallback_bytes=64 << 10)
    ddp.register_comm_hook(state, comprex_hook)
    opt = torch.optim.SGD(ddp.parameters(), lr=0.01 * ranks, momentum=0.9)
    gen = torch.Generator().manual_seed(rank)
    templates = torch.rand(10, 1, 28, 28, generator=torch.Generator().manual_seed(123))
    for step in range(args.steps):
        y = torch.randint(0, 10, (64,), generator=gen)
        x = (0.6 * templates[y] + 0.4 * torch.rand(64, 1, 28, 28, generator=gen)).to(dev)
        opt.zero_grad()
        loss = F.cross_entropy(ddp(x), y.to(dev))
        loss.backward()
        opt.step()
        if rank == 0 and (step + 1) % 50 == 0:
            print(f"step {step + 1}: loss {loss.item():.4f} compressor {state.stats()}", flush=True)
    if args.checkpoint and rank == 0:
        torch.save({"model": model.state_dict(), "optimizer": opt.state_dict(), "hook": pickle.dumps(state)},
                   args.checkpoint)
    final = torch.tensor([loss.item()], device=dev)
    dist.all_reduce(final)
    if rank == 0:
        print(f"mean final loss over {ranks} ranks: {final.item() / ranks:.4f}", flush=True)
    env.barrier()
    env.close()


if __name__ == "__main__":
    main()
