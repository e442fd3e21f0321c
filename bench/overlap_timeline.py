"""Per-bucket timeline of one training step and the overlap A/B.

    torchrun --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 bench/overlap_timeline.py --model resnet50

For one step of the benchmark workload (after warm-up) it prints, from CUDA events, when every
gradient bucket became ready and its send half started and ended on the communication stream,
when backward ended, and when every bucket's receive/update half ran; then it times the same
workload with ``overlap=False`` (all exchange work after backward) for comparison.  Times are
milliseconds on the device, max over ranks for the step times.
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
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "gpt2"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--allreduce", default="comprex_bigring")
    ap.add_argument("--out", default=None)
    args = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.backends.cudnn.benchmark = True

    def build(overlap):
        torch.manual_seed(1234)
        if args.model == "resnet50":
            from comprex_b200.models.resnet import resnet50
            model = resnet50().to(dev).to(torch.bfloat16).to(memory_format=torch.channels_last)
            x = torch.randn(128, 3, 224, 224, device=dev).to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
            y = torch.randint(0, 1000, (128,), device=dev)
            kw, ratio = dict(lr=0.01, momentum=0.9), 0.01
            loss_fn = lambda: F.cross_entropy(model(x).float(), y)     # noqa: E731
        else:
            from comprex_b200.models.gpt2 import gpt2_medium
            model = gpt2_medium().to(dev).to(torch.bfloat16)
            t = torch.randint(0, 50257, (8, 1025), device=dev)
            kw, ratio = dict(lr=3e-4, rule="adamw", weight_decay=0.1, betas=(0.9, 0.95)), 0.001
            loss_fn = lambda: model(t[:, :-1].contiguous(), t[:, 1:].contiguous())   # noqa: E731
        env = cx.GaspiEnvironment(256 << 20, device=dev)
        broadcast_parameters(model, env, 0)
        opt = ComprexOptimizer(model.parameters(), env, compression_ratio=ratio, size_factor=max(4 * ratio, 1e-3) + 1e-4,
                               bucket_cap_mb=25.0, overlap=overlap, allreduce_type=args.allreduce, **kw)
        return env, opt, loss_fn

    def step(opt, loss_fn):
        opt.zero_grad()
        loss_fn().backward()
        opt.step()

    def timed(opt, loss_fn):
        for _ in range(4):
            step(opt, loss_fn)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(args.steps):
            step(opt, loss_fn)
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / args.steps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(float(t), 3)

    out = {"model": args.model, "ranks": world, "allreduce": args.allreduce}
    env, opt, loss_fn = build(True)
    out["ms_per_step_overlap"] = timed(opt, loss_fn)
    opt.enable_timeline()
    step(opt, loss_fn)
    step(opt, loss_fn)
    out["timeline_ms"] = opt.timeline()
    opt.enable_timeline(False)
    del opt
    env.close()
    env, opt, loss_fn = build(False)
    out["ms_per_step_no_overlap"] = timed(opt, loss_fn)
    del opt
    env.close()
    if rank == 0:
        print(json.dumps(out))
        if args.out:
            os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
            with open(args.out, "w") as f:
                f.write(json.dumps(out, indent=1) + "\n")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
