"""Headline benchmark: data-parallel training throughput with the compressed optimizer.

    python bench.py --gpus N --steps K --warmup W            # N == 1: plain python
    torchrun ... bench.py --gpus N --steps K --warmup W       # N > 1: one rank per GPU

Default workload: ResNet-50 (25.6 M parameters) in bf16, channels-last, synthetic
224x224x3 inputs, batch 128 per GPU, momentum SGD (0.9) through
``ComprexOptimizer``: gradients in 25 MB buckets, top-k 1 % with error feedback,
exchanged by this package's kernels (peer stores over NVLink) and overlapped
with backward.  ``--model gpt2`` runs GPT-2 medium (seq 1024, micro-batch 8,
AdamW, top-k 0.1 %), ``--model lenet`` LeNet-5 (batch 64, SGD 0.01, top-k 1 %).

Prints ONE JSON line on rank 0.  ``value`` is samples/s of the whole job,
device-timed with CUDA events over exactly K steps after W warm-up steps,
bracketed by barrier + synchronize, max over ranks.  ``e2e`` is the same metric
through the public API with, every step, the host-to-device copy of that
step's inputs from pinned memory and a device-to-host read of the loss inside
the timed region.  ``gpu_launches`` counts this library's kernel launches inside
the device-timed region (rank 0).  Clocks are sampled with nvidia-smi during the
timed region.

``--impl reference`` reports why the reference cannot run here.  ``--impl dense`` runs the
comparison arm on the same model and data: stock DistributedDataParallel (dense NCCL allreduce)
with the stock torch optimizer; ``--impl hook`` the same with this package's compressed DDP
communication hook in place of the NCCL allreduce.

The default arm (``ours``) also runs that dense arm afterwards in the same invocation, on the
same batches, for the same steps and warm-up: the reference publishes no number, so
``vs_baseline`` is ``value`` divided by the dense arm's value and ``baseline`` holds the dense
arm's figures (``--skip-baseline`` leaves both out).  With N > 1 the line also carries an
``allreduce`` block: compressed BigRing, compressed Ring and the automatic choice for one
2^24-element fp32 vector at top-k 1 % (achieved sent fraction stated) next to
``torch.distributed.all_reduce`` of the same tensor, CUDA-event microseconds, max over ranks.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

REFERENCE_UNAVAILABLE = ("the metric needs the reference's Keras optimizer and TF custom ops: TensorFlow 2.3 is not on this "
                         "image and cannot be installed offline; pip cannot install the tree either (no setup.py/pyproject.toml; "
                         "GPI-2 and GaspiCxx absent). Its Python package and allreduce benchmark do run from baseline/_ref on a "
                         "shared-memory GaspiCxx stand-in (baseline/README.md), on CPU only")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "dense", "hook"])
    ap.add_argument("--model", default="resnet50", choices=["resnet50", "gpt2", "lenet"])
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch (default: the named config)")
    ap.add_argument("--ratio", type=float, default=None)
    ap.add_argument("--bucket-mb", type=float, default=25.0)
    ap.add_argument("--no-overlap", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-baseline", action="store_true", help="do not run the dense DDP comparison arm afterwards")
    ap.add_argument("--skip-allreduce", action="store_true", help="N > 1: do not time the compressed allreduce block")
    ap.add_argument("--allreduce", default="comprex_bigring",
                    help="allreduce_type of the compressed optimizer (comprex_bigring, comprex_ring, auto, ...)")
    return ap.parse_args()


class ClockSampler:
    """nvidia-smi in the background during the timed region; summary afterwards."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.path = gpu_index, None, f"/tmp/cx_clocks_{os.getpid()}.csv"

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.idx)],
                                         stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.remove(self.path)
        except Exception:
            pass
        busy = [s for s in sm if s > 0]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_workload(args, torch, F, dev, world):
    """Model, per-rank host batch maker, loss function and the config block of the named workload."""
    if args.model == "resnet50":
        from comprex_b200.models.resnet import resnet50
        batch = args.batch or 128
        ratio = args.ratio or 0.01
        model = resnet50().to(dev).to(torch.bfloat16).to(memory_format=torch.channels_last)
        opt_kw = dict(lr=0.01, momentum=0.9, rule="sgd", weight_decay=0.0)

        def host_batch(g):
            return (torch.randn(batch, 3, 224, 224, generator=g).to(torch.bfloat16)
                    .contiguous(memory_format=torch.channels_last).pin_memory(),
                    torch.randint(0, 1000, (batch,), generator=g).pin_memory())

        def loss_of(net, x, y):
            return F.cross_entropy(net(x).float(), y)
        cfg = {"model": "resnet50", "global_batch": batch * world, "seq_len": None, "image": "224x224x3",
               "optimizer": "sgd momentum 0.9 (local momentum, fused update)"}
    elif args.model == "gpt2":
        from comprex_b200.models.gpt2 import gpt2_medium
        batch = args.batch or 8
        ratio = args.ratio or 0.001
        model = gpt2_medium().to(dev).to(torch.bfloat16)
        opt_kw = dict(lr=3e-4, rule="adamw", weight_decay=0.1, betas=(0.9, 0.95))

        def host_batch(g):
            t = torch.randint(0, 50257, (batch, 1025), generator=g)
            return t[:, :-1].contiguous().pin_memory(), t[:, 1:].contiguous().pin_memory()

        def loss_of(net, x, y):
            return net(x, y)
        cfg = {"model": "gpt2-medium", "global_batch": batch * world, "seq_len": 1024, "optimizer": "adamw (fused)"}
    else:
        from comprex_b200.models.lenet import LeNet5
        batch = args.batch or 64
        ratio = args.ratio or 0.01
        model = LeNet5().to(dev)
        opt_kw = dict(lr=0.01, momentum=0.0, rule="sgd")

        def host_batch(g):
            return (torch.rand(batch, 1, 28, 28, generator=g).pin_memory(),
                    torch.randint(0, 10, (batch,), generator=g).pin_memory())

        def loss_of(net, x, y):
            return F.cross_entropy(net(x), y)
        cfg = {"model": "lenet5", "global_batch": batch * world, "seq_len": None, "optimizer": "sgd 0.01"}
    return model, batch, ratio, opt_kw, host_batch, loss_of, cfg


def run_arm(args, impl, rank, world, local):
    """One arm (``ours`` or ``dense``) of the training benchmark: fresh model and optimizer, warm-up,
    the device-timed loop, then the end-to-end loop.  Returns the numbers of that arm."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    import comprex_b200 as cx
    from comprex_b200 import _lib
    from comprex_b200.callbacks import broadcast_parameters
    from comprex_b200.optim import ComprexOptimizer

    dev = torch.device("cuda", local)
    torch.manual_seed(1234)
    model, batch, ratio, opt_kw, host_batch, loss_of, cfg = build_workload(args, torch, F, dev, world)
    nparams = sum(p.numel() for p in model.parameters())
    env = cx.GaspiEnvironment(256 << 20, device=dev)
    broadcast_parameters(model, env, 0)
    # slots sized for 2x the expected survivors (what does not fit stays in the residual)
    size_factor = max(4.0 * ratio, 1e-3) + 1e-4
    dense = impl in ("dense", "hook")
    net = model
    if dense:
        # comparison arm: stock DistributedDataParallel (dense NCCL allreduce, 25 MB buckets) and
        # the stock torch optimizer on the same model, data and step structure
        from torch.nn.parallel import DistributedDataParallel as DDP
        if args.model == "gpt2":
            opt = torch.optim.AdamW(model.parameters(), lr=opt_kw["lr"], betas=opt_kw["betas"],
                                    weight_decay=opt_kw["weight_decay"], fused=True)
        else:
            opt = torch.optim.SGD(model.parameters(), lr=opt_kw["lr"], momentum=opt_kw.get("momentum", 0.0))
        if world > 1:
            net = DDP(model, device_ids=[local], bucket_cap_mb=args.bucket_mb, gradient_as_bucket_view=True)
            if impl == "hook":
                # stock DDP and optimizer, the gradient buckets exchanged by this package's DDP hook
                from comprex_b200.ddp_hook import ComprexHookState, comprex_hook
                hook_state = ComprexHookState(env, compression_ratio=ratio)
                net.register_comm_hook(hook_state, comprex_hook)
    else:
        opt = ComprexOptimizer(model.parameters(), env, compression_ratio=ratio, size_factor=size_factor,
                               bucket_cap_mb=args.bucket_mb, overlap=not args.no_overlap,
                               allreduce_type=args.allreduce, **opt_kw)

    def loss_fn(x, y):
        return loss_of(net, x, y)

    gen = torch.Generator().manual_seed(100 + rank)
    host = [host_batch(gen) for _ in range(4)]
    dev_batches = [(x.to(dev, non_blocking=True), y.to(dev, non_blocking=True)) for x, y in host]
    torch.cuda.synchronize()

    def step_device(i):
        x, y = dev_batches[i % len(dev_batches)]
        opt.zero_grad()
        loss = loss_fn(x, y)
        loss.backward()
        opt.step()
        return loss

    def e2e_loop(nsteps):
        """nsteps training steps fed from pinned host memory: the next batch's host-to-device copy
        runs on a copy stream while this batch trains, and the loss of step k is read on the host
        while step k+1 is queued (every step's copy and read-back happen inside this loop)."""
        from comprex_b200.utils import AsyncScalar, DevicePrefetcher
        feed = DevicePrefetcher((host[i % len(host)] for i in range(nsteps)), dev)
        pending, last = None, 0.0
        for x, y in feed:
            opt.zero_grad()
            loss = loss_fn(x, y)
            loss.backward()
            opt.step()
            reader = AsyncScalar(loss)
            if pending is not None:
                last = pending.value()
            pending = reader
        if pending is not None:
            last = pending.value()
        return last

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    warm = max(args.warmup, 3)
    for i in range(warm):
        step_device(i)
    env.flush()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    l0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        loss = step_device(i)
    e1.record()
    barrier()
    launches = _lib.launch_count() - l0
    ms = max_over_ranks(e0.elapsed_time(e1))
    clocks = sampler.stop() if rank == 0 else None
    env.check()
    final_loss = float(loss.item())

    e2e = None
    if not args.skip_e2e:
        e2e_loop(2)
        barrier()
        t0 = time.perf_counter()
        e2e_loop(args.steps)
        barrier()
        sec = max_over_ranks(time.perf_counter() - t0)
        hx, hy = host[0]
        e2e = {"value": round(batch * world * args.steps / sec, 2), "unit": "samples/s",
               "h2d_bytes_per_step": hx.numel() * hx.element_size() + hy.numel() * hy.element_size(),
               "d2h_bytes_per_step": 4, "ms_per_step": round(sec * 1e3 / args.steps, 3)}
    stats = {} if dense else opt.stats()
    cfg.update({"parallelism": f"dp{world}", "per_gpu_batch": batch, "params": nparams,
                "compression_ratio": None if dense else ratio, "bucket_mb": args.bucket_mb,
                "overlap": not args.no_overlap,
                "allreduce": ("DistributedDataParallel with the compressed communication hook, stock torch optimizer"
                              if impl == "hook" else
                              "dense NCCL allreduce (DistributedDataParallel), stock torch optimizer" if dense else
                              getattr(opt, "describe", lambda: args.allreduce)()),
                "cache": "inputs_larger_than_L2 (activations + weights per step exceed 126 MB)",
                "first_bucket_nnz": stats.get("nnz"), "first_bucket_n": stats.get("n"), "final_loss": final_loss})
    out = {"impl": "ddp_comprex_hook" if impl == "hook" else "dense_nccl_ddp" if dense else "ours", "value": round(batch * world * args.steps / (ms / 1e3), 2),
           "ms_per_step": round(ms / args.steps, 3), "warm": warm, "config": cfg, "clocks": clocks, "e2e": e2e,
           "gpu_launches": int(launches), "final_loss": final_loss, "dtype": "fp32" if args.model == "lenet" else "bf16"}
    del opt, net, model, dev_batches
    env.close()
    torch.cuda.empty_cache()
    return out


def allreduce_block(rank, world, local, log2n=24, ratio=0.01, reps=10, warmup=3):
    """Compressed allreduce of one fp32 vector against ``torch.distributed.all_reduce`` of the same
    tensor (the reference's examples/allreduce_speed.cpp:259-279 protocol, device-timed): CUDA-event
    microseconds, ranks aligned by a barrier before every repetition, L2 flushed between repetitions,
    MAX over ranks per repetition, median over repetitions."""
    import torch
    import torch.distributed as dist
    import comprex_b200 as cx

    dev = torch.device("cuda", local)
    n = 1 << log2n
    env = cx.GaspiEnvironment(256 << 20, device=dev)
    flush = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    torch.manual_seed(1000 + rank)
    x = torch.randn(n, device=dev)

    def time_op(fn):
        out = []
        for i in range(warmup + reps):
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
            if i >= warmup:
                out.append(float(t.item()))
        return statistics.median(out)

    work = x.clone()
    block = {"n": n, "dtype": "fp32", "nominal_topk": ratio, "ranks": world,
             "nccl_all_reduce_us": round(time_op(lambda: dist.all_reduce(work)), 2)}
    sf = max(4.0 * ratio, 2e-3)
    for name, cls, kw in (("comprex_bigring", cx.Comprex_BigRingAllreduce, {"consistent": True}),
                          ("comprex_ring", cx.Comprex_RingAllreduce, {"consistent": True, "chunk_align": 4}),
                          ("auto", cx.AutoAllreduce, {})):
        mark = env.heap_mark()
        ar = cls(env)
        ar.setup_connections(n, 1, ratio, sf, **kw)
        buf = x.clone()
        # the input is not reset between repetitions: the residual carries what was not sent, as in training
        us = time_op(lambda: ar.apply(buf))
        st = ar.stats()
        block[name] = {"us": round(us, 2), "sent_fraction": round(st["nnz"] / max(st["n"], 1), 5) if st else None,
                       "speedup_vs_nccl": round(block["nccl_all_reduce_us"] / us, 2)}
        if name == "auto":
            block[name]["chosen"] = ar.choice
        del ar, buf
        env.heap_release(mark)
    env.barrier()
    env.close()
    return block


def main():
    args = parse()
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) == 0:          # one line per job, also under torchrun
            print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0

    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torchrun --nproc-per-node {args.gpus}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    torch.backends.cudnn.benchmark = True
    torch.backends.cuda.matmul.allow_tf32 = True
    torch.backends.cudnn.allow_tf32 = True

    main_arm = run_arm(args, args.impl, rank, world, local)
    base = None
    notes = {}
    if args.impl == "ours" and not args.skip_baseline:
        # the comparison arm in the same invocation, on the same batches: stock DDP + NCCL + torch optimizer
        try:
            base = run_arm(args, "dense", rank, world, local)
        except Exception as e:                               # the headline number stands without it
            notes["baseline_error"] = f"{type(e).__name__}: {e}"[:300]
    ar_block = None
    if world > 1 and args.impl == "ours" and not args.skip_allreduce:
        try:
            ar_block = allreduce_block(rank, world, local)
        except Exception as e:
            notes["allreduce_error"] = f"{type(e).__name__}: {e}"[:300]
    if rank == 0:
        line = {"metric": "train samples/sec", "value": main_arm["value"], "unit": "samples/s", "n_gpus": world,
                "steps": args.steps, "warmup": main_arm["warm"], "ms_per_step": main_arm["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": main_arm["dtype"],
                "data": "synthetic", "impl": main_arm["impl"], "config": main_arm["config"],
                "clocks": main_arm["clocks"], "e2e": main_arm["e2e"], "gpu_launches": main_arm["gpu_launches"]}
        if base is not None:
            # no published reference number exists: the baseline is the dense arm measured just now
            line["vs_baseline"] = round(main_arm["value"] / base["value"], 4)
            bl = {"impl": base["impl"], "value": base["value"], "ms_per_step": base["ms_per_step"],
                  "e2e": base["e2e"], "final_loss": base["final_loss"], "clocks": base["clocks"],
                  "ratio": line["vs_baseline"], "what": base["config"]["allreduce"]}
            if base["e2e"] and main_arm["e2e"]:
                bl["e2e_ratio"] = round(main_arm["e2e"]["value"] / base["e2e"]["value"], 4)
            line["baseline"] = bl
        if ar_block is not None:
            line["allreduce"] = ar_block
        line.update(notes)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
