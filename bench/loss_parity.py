"""Training-loss curves at a fixed step count: compressed optimizer against dense DDP.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench/loss_parity.py --model resnet50 --steps 300

Every arm trains the same randomly initialised model on the same fixed set of synthetic batches
(``--batches`` per rank, cycled; the labels are random, so the loss falls by memorisation) with
the same hyper-parameters:

* ``dense``          stock DistributedDataParallel + NCCL + the torch optimizer,
* ``ours``           ComprexOptimizer, replica-consistent (the default),
* ``ours_reference`` ComprexOptimizer(consistent=False): the reference's rule (own update dense,
                     peers' sparse, keras/comprex_optimizer.py:117-133),
* ``ours_exact``     like ``ours`` with the exact top-k threshold instead of the sampled estimate.

Printed per arm: the mean loss over all ranks every ``--every`` steps, the nominal top-k and the
fraction actually sent in the last step (first bucket).  One JSON object on rank 0.
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import comprex_b200 as cx  # noqa: E402
from comprex_b200.callbacks import broadcast_parameters  # noqa: E402
from comprex_b200.optim import ComprexOptimizer  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "gpt2", "lenet"])
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--every", type=int, default=25)
    ap.add_argument("--batches", type=int, default=8)
    ap.add_argument("--ratio", type=float, default=None)
    ap.add_argument("--arms", nargs="+", default=["dense", "ours", "ours_reference"])
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    dev = torch.device("cuda", local) if cuda else torch.device("cpu")
    if world > 1:
        dist.init_process_group("nccl" if cuda else "gloo", **({"device_id": dev} if cuda else {}))
    torch.backends.cudnn.benchmark = True

    def make_model():
        torch.manual_seed(1234)
        if args.model == "resnet50":
            from comprex_b200.models.resnet import resnet50
            return resnet50().to(dev).to(torch.bfloat16).to(memory_format=torch.channels_last)
        if args.model == "gpt2":
            from comprex_b200.models.gpt2 import gpt2_medium
            return gpt2_medium().to(dev).to(torch.bfloat16)
        from comprex_b200.models.lenet import LeNet5
        return LeNet5().to(dev)

    gen = torch.Generator().manual_seed(100 + rank)
    if args.model == "resnet50":
        data = [(torch.randn(128, 3, 224, 224, generator=gen).to(torch.bfloat16).contiguous(memory_format=torch.channels_last).to(dev),
                 torch.randint(0, 1000, (128,), generator=gen).to(dev)) for _ in range(args.batches)]
        ratio, kw = args.ratio or 0.01, dict(lr=0.01, momentum=0.9)
        loss_of = lambda net, b: F.cross_entropy(net(b[0]).float(), b[1])            # noqa: E731
    elif args.model == "gpt2":
        toks = [torch.randint(0, 50257, (8, 1025), generator=gen).to(dev) for _ in range(args.batches)]
        data = [(t[:, :-1].contiguous(), t[:, 1:].contiguous()) for t in toks]
        ratio, kw = args.ratio or 0.001, dict(lr=3e-4, rule="adamw", weight_decay=0.1, betas=(0.9, 0.95))
        loss_of = lambda net, b: net(b[0], b[1])                                      # noqa: E731
    else:
        data = [(torch.rand(64, 1, 28, 28, generator=gen).to(dev), torch.randint(0, 10, (64,), generator=gen).to(dev))
                for _ in range(args.batches)]
        ratio, kw = args.ratio or 0.01, dict(lr=0.01, momentum=0.0)
        loss_of = lambda net, b: F.cross_entropy(net(b[0]), b[1])                     # noqa: E731

    def mean_over_ranks(v):
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t)
        return float(t) / world

    result = {"model": args.model, "ranks": world, "steps": args.steps, "nominal_topk": ratio, "arms": {}}
    for arm in args.arms:
        model = make_model()
        env = cx.GaspiEnvironment(256 << 20, device=dev)
        broadcast_parameters(model, env, 0)
        net = model
        if arm == "dense":
            if args.model == "gpt2":
                opt = torch.optim.AdamW(model.parameters(), lr=kw["lr"], betas=kw["betas"], weight_decay=kw["weight_decay"],
                                        fused=cuda)
            else:
                opt = torch.optim.SGD(model.parameters(), lr=kw["lr"], momentum=kw.get("momentum", 0.0))
            if world > 1:
                from torch.nn.parallel import DistributedDataParallel as DDP
                net = DDP(model, device_ids=[local] if cuda else None, bucket_cap_mb=25.0)
        else:
            opt = ComprexOptimizer(model.parameters(), env, compression_ratio=ratio, size_factor=max(4 * ratio, 1e-3) + 1e-4,
                                   bucket_cap_mb=25.0, overlap=cuda, consistent=(arm != "ours_reference"), **kw)
        curve = []
        for i in range(args.steps):
            opt.zero_grad()
            loss = loss_of(net, data[i % len(data)])
            loss.backward()
            if arm == "ours_exact" and i == 0:
                opt._ensure_allreducers()
                for ar in opt.comprex_allreducers.values():
                    if ar.compressed:
                        ar.set_exact_topk()
            opt.step()
            if i % args.every == 0 or i == args.steps - 1:
                curve.append((i, round(mean_over_ranks(float(loss)), 4)))
        row = {"loss": curve}
        if arm != "dense":
            st = opt.stats()
            if st:
                row["sent_fraction_last_step"] = round(st["nnz"] / max(st["n"], 1), 5)
        result["arms"][arm] = row
        if rank == 0:
            print(arm, json.dumps(row), flush=True)
        del opt, net, model
        env.close()
        if cuda:
            torch.cuda.empty_cache()
    if rank == 0:
        print(json.dumps(result))
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as f:
                f.write(json.dumps(result, indent=1) + "\n")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
