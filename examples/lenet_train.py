"""Data-parallel LeNet training with the compressed optimizer (the reference's LeNet/main.py).

Sweeps the reference's settings: dense ``ring`` and ``bigring``, then ``comprex_ring`` and
``comprex_bigring`` at top-k 1 % and 0.1 %, momentum 0.9, learning rate ``0.01 * ranks``,
batch 64 per rank, ``size_factor`` 3, initial weights broadcast from rank 0.  MNIST is read
from ``--data`` (a directory with ``mnist.npz``) when given; without it a synthetic
28x28x1 data set of the same shape is used (ten fixed random class templates buried in
uniform noise, so that there is something to learn).

    torchrun --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 examples/lenet_train.py --epochs 2
"""
import argparse
import os
import sys
import time

import numpy as np
import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import comprex_b200 as cx  # noqa: E402
from comprex_b200.callbacks import BroadcastInitWeights  # noqa: E402
from comprex_b200.models.lenet import LeNet5, LeNetReference  # noqa: E402
from comprex_b200.optim import ComprexOptimizer  # noqa: E402


def load_data(path, n_train, n_test, device):
    if path:
        d = np.load(os.path.join(path, "mnist.npz"))
        xtr, ytr, xte, yte = d["x_train"], d["y_train"], d["x_test"], d["y_test"]
        xtr = torch.from_numpy(xtr[:n_train]).float().div(255).unsqueeze(1)
        xte = torch.from_numpy(xte[:n_test]).float().div(255).unsqueeze(1)
        return xtr.to(device), torch.from_numpy(ytr[:n_train]).long().to(device), \
            xte.to(device), torch.from_numpy(yte[:n_test]).long().to(device)
    g = torch.Generator().manual_seed(0)
    # ten fixed random templates, one per class, buried in uniform noise
    templates = torch.rand(10, 1, 28, 28, generator=g)
    y = torch.randint(0, 10, (n_train + n_test,), generator=g)
    x = 0.6 * templates[y] + 0.4 * torch.rand(n_train + n_test, 1, 28, 28, generator=g)
    x, y = x.to(device), y.to(device)
    return x[:n_train], y[:n_train], x[n_train:], y[n_train:]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--data", default=None)
    ap.add_argument("--epochs", type=int, default=5)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--train-samples", type=int, default=60000)
    ap.add_argument("--model", default="lenet5", choices=["lenet5", "reference"])
    ap.add_argument("--reference-semantics", action="store_true",
                    help="also run comprex_bigring the reference's way (own update dense, peers' sparse)")
    args = ap.parse_args()
    cx.initGaspiCxx()
    env = cx.GaspiEnvironment(64 << 20)
    rank, ranks, dev = env.get_rank(), env.get_ranks(), env.device
    xtr, ytr, xte, yte = load_data(args.data, args.train_samples, 10000, dev)
    shard = slice(rank * (len(xtr) // ranks), (rank + 1) * (len(xtr) // ranks))   # one shard per rank
    xtr, ytr = xtr[shard], ytr[shard]
    runs = [("ring", 1.0), ("bigring", 1.0)] + [(k, r) for r in (1e-2, 1e-3) for k in ("comprex_ring", "comprex_bigring")]
    runs = [(k, r, True) for k, r in runs]
    if args.reference_semantics:
        runs += [("comprex_bigring", r, False) for r in (1e-2, 1e-3)]
    for kind, ratio, consistent in runs:
        torch.manual_seed(0)
        model = (LeNet5() if args.model == "lenet5" else LeNetReference()).to(dev)
        BroadcastInitWeights(0, env).on_train_begin(model)
        opt = ComprexOptimizer(model.parameters(), env, lr=0.01 * ranks, momentum=0.9, compression_ratio=ratio,
                               allreduce_type=kind, size_factor=3.0, local_momentum=kind.startswith("comprex"),
                               consistent=consistent)
        t0 = time.time()
        for epoch in range(args.epochs):
            perm = torch.randperm(len(xtr), device=dev, generator=torch.Generator(device=dev).manual_seed(epoch))
            for b in range(0, len(xtr) - args.batch + 1, args.batch):
                idx = perm[b:b + args.batch]
                opt.zero_grad()
                loss = F.cross_entropy(model(xtr[idx]), ytr[idx])
                loss.backward()
                opt.step()
            with torch.no_grad():
                acc = float((model(xte).argmax(1) == yte).float().mean())
            if rank == 0:
                tag = kind if consistent else kind + " (reference semantics)"
                print(f"{tag} ratio {ratio:g} epoch {epoch + 1}: loss {loss.item():.4f} test accuracy {acc:.4f} "
                      f"time {time.time() - t0:.1f} s", flush=True)
        env.barrier()
    env.close()


if __name__ == "__main__":
    main()
