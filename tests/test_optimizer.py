"""ComprexOptimizer and the DDP hook: update rule vs a plain restatement of
keras/comprex_optimizer.py:97-133,150-163, conservation through flush,
bucketed layout, checkpoint/resume, replica consistency across real ranks.
"""
import copy

import pytest
import torch
import torch.distributed as dist

import comprex_b200 as cx
from comprex_b200.models.lenet import LeNet5
from comprex_b200.optim import ComprexOptimizer

from test_multiprocess import gpu_world, run_ranks


def _const_grad_model(device, seed=0):
    torch.manual_seed(seed)
    return torch.nn.ParameterList([torch.nn.Parameter(torch.randn(s, device=device)) for s in
                                   [(300, 7), (1000,), (5,), (64, 64)]])


def _set_grads(opt, params, cs):
    opt.zero_grad()
    for p, c in zip(params, cs):
        p.grad = c.clone()


@pytest.mark.parametrize("buckets", [None, 0.004])
@pytest.mark.parametrize("local_momentum", [True, False])
def test_sgd_rule_matches_reference_after_flush(device, buckets, local_momentum):
    env = cx.GaspiEnvironment(8 << 20, device=device)
    params = _const_grad_model(device)
    w0 = [p.detach().clone() for p in params]
    cs = [torch.randn_like(p) * 3 for p in params]
    lr, mu, wd, clip, steps = 0.1, 0.9, 0.0, 5.0, 7
    opt = ComprexOptimizer(params, env, single_rank_bypass=False, lr=lr, momentum=mu, compression_ratio=0.05, size_factor=3.0,
                           pre_clipnorm=clip, weight_decay=wd, local_momentum=local_momentum, bucket_cap_mb=buckets)
    if buckets:
        assert len(opt._buckets) > 1
    for _ in range(steps):
        _set_grads(opt, params, cs)
        opt.step()
    # restatement: clip_by_norm, mom = mu*mom + lr*g, w -= mom  (all of it arrives once residuals are flushed)
    if local_momentum:
        opt.flush()
        for p, w, c in zip(params, w0, cs):
            g = c * clip / max(float(c.norm()), clip)
            mom, ref = torch.zeros_like(w), w.clone()
            for _ in range(steps):
                mom = mu * mom + lr * g
                ref = ref - mom
            torch.testing.assert_close(p.detach(), ref, rtol=1e-4, atol=1e-4)
    else:
        assert all(torch.isfinite(p).all() for p in params)
    env.close()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_fold_clips_per_tensor_and_keeps_memory_format(device, dtype):
    """The fold kernels against clip_by_norm + momentum in plain fp32, on tensors that are
    larger than one work item, channels-last, unaligned in length, or without a gradient."""
    env = cx.GaspiEnvironment(8 << 20, device=device)
    torch.manual_seed(3)
    conv = torch.randn(96, 24, 3, 3, device=device).to(memory_format=torch.channels_last)
    shapes = [torch.randn(70001, device=device), conv, torch.randn(7, device=device), torch.randn(33, 5, device=device)]
    params = [torch.nn.Parameter(t.to(dtype)) for t in shapes]
    w0 = [p.detach().float().clone() for p in params]
    lr, mu, clip = 0.05, 0.9, 2.0
    opt = ComprexOptimizer(params, env, single_rank_bypass=False, lr=lr, momentum=mu, compression_ratio=1.0, size_factor=1.0, pre_clipnorm=clip)
    assert params[1].is_contiguous(memory_format=torch.channels_last) and not params[1].is_contiguous()
    for p, w in zip(params, w0):
        torch.testing.assert_close(p.detach().float(), w)
    gs = [(torch.randn_like(p.float()) * s).to(dtype) for p, s in zip(params, (0.001, 1.0, 3.0, 0.2))]
    gs[1] = gs[1].contiguous(memory_format=torch.channels_last)
    mom = [torch.zeros_like(w) for w in w0]
    for step in range(3):
        opt.zero_grad()
        for i, (p, g) in enumerate(zip(params, gs)):
            if not (step == 1 and i == 3):          # one step without a gradient for the last tensor
                p.grad = g.clone()
        b = opt._buckets[0]
        u = opt._fold(b, lr, mu).clone()
        for i, (g, o) in enumerate(zip(gs, b.offsets[::-1])):
            gf = g.float() if not (step == 1 and i == 3) else torch.zeros_like(g.float())
            mom[i] = mu * mom[i] + lr * gf * (clip / max(float(gf.norm()), clip))
        for p, o, i in zip(b.params, b.offsets, range(len(params) - 1, -1, -1)):
            got = u[o:o + p.numel()].as_strided(p.size(), p.stride())
            torch.testing.assert_close(got, mom[i], rtol=2e-5, atol=1e-7)
    env.close()


def test_training_reduces_loss_and_bf16_shadow(device):
    torch.manual_seed(0)
    env = cx.GaspiEnvironment(8 << 20, device=device)
    model = LeNet5().to(device).to(torch.bfloat16)
    opt = ComprexOptimizer(model.parameters(), env, single_rank_bypass=False, lr=0.05, momentum=0.9, compression_ratio=0.1, size_factor=1.0)
    x = torch.rand(64, 1, 28, 28, device=device).to(torch.bfloat16)
    y = torch.randint(0, 10, (64,), device=device)
    losses = []
    for _ in range(40):
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(x).float(), y)
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert losses[-1] < losses[0] - 0.05
    for p in model.parameters():   # the model's tensors are views of the bf16 shadow of the fp32 master
        assert p.dtype == torch.bfloat16
    assert torch.equal(opt._shadow, opt._master.to(torch.bfloat16))
    st = opt.stats()
    assert 0 < st["nnz"] < st["n"]
    env.close()


@pytest.mark.parametrize("rule", ["sgd", "adamw"])
def test_checkpoint_resume_is_bit_exact(device, rule):
    def make(seed=0):
        torch.manual_seed(seed)
        env = cx.GaspiEnvironment(8 << 20, device=device)
        # linear layers only: cuDNN's convolution backward is not run-to-run deterministic
        model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, 96), torch.nn.ReLU(),
                                    torch.nn.Linear(96, 10)).to(device)
        opt = ComprexOptimizer(model.parameters(), env, single_rank_bypass=False, lr=0.02, momentum=0.9, compression_ratio=0.02,
                               size_factor=1.0, rule=rule, weight_decay=0.01, bucket_cap_mb=0.05)
        return env, model, opt

    def run(model, opt, steps, start):
        for i in range(start, start + steps):
            g = torch.Generator().manual_seed(i)
            x = torch.rand(16, 1, 28, 28, generator=g).to(device)
            y = torch.randint(0, 10, (16,), generator=g).to(device)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()

    env_a, model_a, opt_a = make()
    run(model_a, opt_a, 5, 0)
    sd = copy.deepcopy(opt_a.state_dict())
    assert sd["comprex"]["step"] == 5 and sd["comprex"]["allreduce"][0]["residuals"][0].abs().sum() > 0
    run(model_a, opt_a, 4, 5)
    env_b, model_b, opt_b = make(seed=99)          # fresh objects, different init
    opt_b.load_state_dict(sd)
    run(model_b, opt_b, 4, 5)
    assert torch.equal(opt_a._master, opt_b._master)
    for pa, pb in zip(model_a.parameters(), model_b.parameters()):
        assert torch.equal(pa, pb)
    env_a.close()
    env_b.close()


def test_reference_semantics_option(device):
    """consistent=False: the reference's rule for the compressed BigRing - the rank's own update is
    applied densely (nothing of it waits in a residual for the weights of this rank)."""
    env = cx.GaspiEnvironment(8 << 20, device=device)
    params = _const_grad_model(device)
    w0 = [p.detach().clone() for p in params]
    cs = [torch.randn_like(p) for p in params]
    opt = ComprexOptimizer(params, env, single_rank_bypass=False, lr=0.1, momentum=0.0, compression_ratio=0.01, size_factor=3.0,
                           pre_clipnorm=None, consistent=False)
    opt._ensure_allreducers()
    assert opt._buckets[0].kind == "phased"
    _set_grads(opt, params, cs)
    opt.step()
    for p, w, c in zip(params, w0, cs):          # single rank: w -= lr * g, in full, immediately
        torch.testing.assert_close(p.detach(), w - 0.1 * c, rtol=1e-6, atol=1e-6)
    env.close()


def test_parameter_groups_must_agree(device):
    env = cx.GaspiEnvironment(8 << 20, device=device)
    a = torch.nn.Parameter(torch.randn(100, device=device))
    b = torch.nn.Parameter(torch.randn(50, device=device))
    opt = ComprexOptimizer([{"params": [a]}, {"params": [b]}], env, lr=0.1, momentum=0.9, compression_ratio=1.0)
    for p in (a, b):
        p.grad = torch.ones_like(p)
    opt.step()                                   # two groups, same settings: fine
    sched = torch.optim.lr_scheduler.StepLR(opt, step_size=1, gamma=0.5)
    sched.step()                                 # schedulers change every group alike
    for p in (a, b):
        p.grad = torch.ones_like(p)
    opt.step()
    assert opt.param_groups[0]["lr"] == opt.param_groups[1]["lr"] == 0.05
    opt.param_groups[1]["lr"] = 0.5
    with pytest.raises(cx.ComprexError, match="parameter groups"):
        opt.step()
    env.close()


def test_other_allreduce_types_and_validation(device):
    env = cx.GaspiEnvironment(8 << 20, device=device)
    with pytest.raises(ValueError):
        ComprexOptimizer(_const_grad_model(device), env, allreduce_type="nope")
    with pytest.raises(ValueError):
        ComprexOptimizer(_const_grad_model(device), env, momentum=1.5)
    for kind in ["ring", "bigring", "alltoone", "comprex_ring", "comprex_alltoone"]:
        params = _const_grad_model(device)
        w0 = [p.detach().clone() for p in params]
        cs = [torch.randn_like(p) for p in params]
        opt = ComprexOptimizer(params, env, single_rank_bypass=False, lr=0.1, momentum=0.0, compression_ratio=0.5, size_factor=3.0,
                               allreduce_type=kind, pre_clipnorm=None)
        _set_grads(opt, params, cs)
        opt.step()
        if not kind.startswith("comprex"):   # single rank, dense: exactly one SGD step
            for p, w, c in zip(params, w0, cs):
                torch.testing.assert_close(p.detach(), w - 0.1 * c)
        opt.set_compression_ratio(0.25)
    env.close()


# ---- real ranks -------------------------------------------------------------------------------------
def scenario_optimizer_ranks(rank, world, device, overlap):
    env = cx.GaspiEnvironment(16 << 20, device=device)
    torch.manual_seed(7)                      # same initial weights everywhere
    model = LeNet5().to(device)
    opt = ComprexOptimizer(model.parameters(), env, lr=0.05, momentum=0.9, compression_ratio=0.05, size_factor=1.0,
                           bucket_cap_mb=0.05, overlap=overlap)
    first = None
    for i in range(12):
        g = torch.Generator().manual_seed(1000 * rank + i)
        x = torch.rand(32, 1, 28, 28, generator=g).to(device)
        y = (x.mean(dim=(1, 2, 3)) * 20).long().clamp(0, 9).to(device)
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        opt.step()
        first = first if first is not None else float(loss)
        flat = opt._master.detach().cpu()
        got = [None] * world
        dist.all_gather_object(got, flat)
        for other in got[1:]:
            assert torch.equal(other, got[0]), "replicas diverged"
    env.barrier()
    env.close()
    return first, float(loss)


def scenario_optimizer_kinds(rank, world, device, kind, aggregate_blob, overlap):
    """Every collective through the bucketed step.  Replica-consistent kinds keep all ranks'
    weights bit-identical; for the fused Ring the decode-with-update must give the bits of the
    two-stage path (allreduce into a work vector, then the dense update kernel)."""
    env = cx.GaspiEnvironment(16 << 20, device=device)

    def make(force_phased=False):
        torch.manual_seed(7)
        model = LeNet5().to(device)
        opt = ComprexOptimizer(model.parameters(), env, lr=0.05, momentum=0.9, compression_ratio=0.05, size_factor=1.0,
                               bucket_cap_mb=0.05 if aggregate_blob else None, overlap=overlap, allreduce_type=kind,
                               aggregate_blob=aggregate_blob)
        if force_phased:
            opt._ensure_allreducers()
            for b in opt._buckets:
                if b.kind == "ring":
                    b.kind = "phased"
        return model, opt
    arms = [make()] + ([make(True)] if kind == "comprex_ring" else [])
    first = last = None
    for i in range(8):
        g = torch.Generator().manual_seed(1000 * rank + i)
        x = torch.rand(32, 1, 28, 28, generator=g).to(device)
        y = (x.mean(dim=(1, 2, 3)) * 20).long().clamp(0, 9).to(device)
        model, opt = arms[0]
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(model(x), y)
        loss.backward()
        if len(arms) == 2:      # the second arm gets the very same gradients (GPU convolutions are not
            arms[1][1].zero_grad()   # bit-reproducible from one backward pass to the next)
            for p0, p1 in zip(model.parameters(), arms[1][0].parameters()):
                p1.grad = p0.grad.clone()
        for _, o in arms:
            o.step()
        first = first if first is not None else float(loss)
        last = float(loss)
        env.flush()
        if len(arms) == 2:
            assert torch.equal(arms[0][1]._master, arms[1][1]._master), "fused ring differs from the two-stage path"
        if kind in ("comprex_bigring", "comprex_ring", "auto", "ring", "alltoone", "bigring"):
            got = [None] * world
            dist.all_gather_object(got, arms[0][1]._master.detach().cpu())
            for other in got[1:]:
                assert torch.equal(other, got[0]), f"replicas diverged ({kind})"
    assert "x " in arms[0][1].describe()
    assert len(arms[0][1]._buckets) > 1
    env.barrier()
    env.close()
    return first, last


def _toy_step(model, opt, rank, i, device):
    g = torch.Generator().manual_seed(1000 * rank + i)
    x = torch.rand(16, 1, 28, 28, generator=g).to(device)
    y = (x.mean(dim=(1, 2, 3)) * 20).long().clamp(0, 9).to(device)
    opt.zero_grad()
    torch.nn.functional.cross_entropy(model(x), y).backward()
    opt.step()


def scenario_elastic_restart(rank, world, device, folder, phase):
    """Save with two ranks, restart with three: old ranks keep their residual and momentum, the
    new rank starts from another rank's file with both at zero; replicas stay identical."""
    import os
    env = cx.GaspiEnvironment(16 << 20, device=device)
    torch.manual_seed(3)
    model = LeNet5().to(device)
    opt = ComprexOptimizer(model.parameters(), env, lr=0.05, momentum=0.9, compression_ratio=0.02, size_factor=1.0)
    if phase == "save":
        for i in range(5):
            _toy_step(model, opt, rank, i, device)
        torch.save(opt.state_dict(), os.path.join(folder, f"opt_{rank}.pt"))
        out = (float(opt._buckets[0].ar.rests.abs().sum()), float(opt._update.abs().sum()))
    else:
        src = rank if os.path.exists(os.path.join(folder, f"opt_{rank}.pt")) else 0
        sd = torch.load(os.path.join(folder, f"opt_{src}.pt"), weights_only=False)
        assert sd["comprex"]["world_size"] == 2 and world == 3
        opt.load_state_dict(sd)
        rests, mom = float(opt._buckets[0].ar.rests.abs().sum()), float(opt._update.abs().sum())
        if src == rank:
            assert rests > 0 and mom > 0                  # this rank's own state came back
            assert torch.equal(opt._buckets[0].ar.rests.cpu(), sd["comprex"]["allreduce"][0]["residuals"][0])
        else:
            assert rests == 0.0 and mom == 0.0            # a new rank starts clean
        got = [None] * world
        dist.all_gather_object(got, opt._master.detach().cpu())
        assert all(torch.equal(g, got[0]) for g in got)   # same weights everywhere
        for i in range(5, 9):
            _toy_step(model, opt, rank, i, device)
        dist.all_gather_object(got, opt._master.detach().cpu())
        assert all(torch.equal(g, got[0]) for g in got), "replicas diverged after the restart"
        out = (rests, mom)
    env.barrier()
    env.close()
    return out


def scenario_data_parallel(rank, world, device):
    """DataParallel wrapper: same weights after construction although every rank initialised
    differently, disjoint shards, replicas stay identical, periodic sync repairs a perturbed rank
    (bf16 model: the fp32 master follows the synchronised weights)."""
    from comprex_b200.parallel.data_parallel import DataParallel
    from comprex_b200.utils import ComprexConfig
    env = cx.GaspiEnvironment(16 << 20, device=device)
    torch.manual_seed(100 + rank)                     # different initial weights on purpose
    model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, 64), torch.nn.ReLU(),
                                torch.nn.Linear(64, 10)).to(device).to(torch.bfloat16)
    dp = DataParallel(model, env, config=ComprexConfig(compression_ratio=0.05, overlap=False, bucket_cap_mb=25.0),
                      lr=0.05, momentum=0.9, sync_every=1)

    def same_everywhere(t):
        got = [None] * world
        dist.all_gather_object(got, t.detach().float().cpu())
        return all(torch.equal(g, got[0]) for g in got)

    assert same_everywhere(dp.optimizer._master)
    shards = [None] * world
    dist.all_gather_object(shards, list(dp.shard(1003)))
    flat = sum(shards, [])
    assert len(flat) == len(set(flat)) == (1003 // world) * world
    for i in range(4):
        g = torch.Generator().manual_seed(50 * rank + i)
        x = torch.rand(16, 1, 28, 28, generator=g).to(device).to(torch.bfloat16)
        y = torch.randint(0, 10, (16,), generator=g).to(device)
        dp.zero_grad()
        torch.nn.functional.cross_entropy(model(x).float(), y).backward()
        dp.step()
    assert same_everywhere(dp.optimizer._master)
    if rank == 1:                                      # someone tampers with one replica
        with torch.no_grad():
            model[1].weight.add_(1.0)
    dp.on_epoch_begin()                                # sync_every=1: rank 0's weights everywhere
    assert same_everywhere(model[1].weight) and same_everywhere(dp.optimizer._master)
    assert torch.equal(dp.optimizer._master.to(torch.bfloat16), dp.optimizer._shadow)
    sd = dp.state_dict()
    assert set(sd) == {"model", "optimizer", "config"} and sd["config"]["compression_ratio"] == 0.05
    env.barrier()
    env.close()
    return True


def scenario_ddp_hook(rank, world, device):
    from torch.nn.parallel import DistributedDataParallel as DDP
    from comprex_b200.ddp_hook import ComprexHookState, comprex_hook
    import pickle
    env = cx.GaspiEnvironment(16 << 20, device=device)
    torch.manual_seed(3)
    base = torch.nn.Sequential(torch.nn.Linear(50, 200), torch.nn.ReLU(), torch.nn.Linear(200, 10)).to(device)
    ids = [rank] if device == "cuda" else None
    # dense fallback for every bucket: must equal the stock averaging allreduce
    m_ref, m_dense = copy.deepcopy(base), copy.deepcopy(base)
    ddp_ref = DDP(m_ref, device_ids=ids)
    ddp_dense = DDP(m_dense, device_ids=ids)
    ddp_dense.register_comm_hook(ComprexHookState(env, dense_fallback_bytes=1 << 40), comprex_hook)
    g = torch.Generator().manual_seed(rank)
    x, y = torch.randn(16, 50, generator=g).to(device), torch.randint(0, 10, (16,), generator=g).to(device)
    for ddp in (ddp_ref, ddp_dense):
        torch.nn.functional.cross_entropy(ddp(x), y).backward()
    if device == "cuda":
        torch.cuda.synchronize()
    for a, b in zip(m_ref.parameters(), m_dense.parameters()):
        torch.testing.assert_close(a.grad, b.grad, rtol=1e-5, atol=1e-6)
    # compressed: what arrives over the steps plus the residuals is the true average gradient sum
    m_c = copy.deepcopy(base)
    ddp_c = DDP(m_c, device_ids=ids)
    state = ComprexHookState(env, compression_ratio=0.05, dense_fallback_bytes=0, capacity_slack=4.0)
    ddp_c.register_comm_hook(state, comprex_hook)
    applied = [torch.zeros_like(p) for p in m_c.parameters()]
    true_sum = [torch.zeros_like(p) for p in m_c.parameters()]
    for step in range(5):
        for p in list(m_c.parameters()) + list(m_ref.parameters()):
            p.grad = None
        torch.nn.functional.cross_entropy(ddp_c(x), y).backward()
        torch.nn.functional.cross_entropy(ddp_ref(x), y).backward()
        if device == "cuda":
            torch.cuda.synchronize()
        for acc, p in zip(applied, m_c.parameters()):
            acc += p.grad
        for acc, p in zip(true_sum, m_ref.parameters()):
            acc += p.grad
        got = [None] * world
        dist.all_gather_object(got, torch.cat([p.grad.reshape(-1).cpu() for p in m_c.parameters()]))
        for other in got[1:]:
            assert torch.equal(other, got[0])
    res_total = 0.0
    for red in state.reducers.values():
        if red.compressed:
            r = red.rests.clone()
            dist.all_reduce(r)
            res_total += float(r.double().sum()) / world
    lhs = sum(float(a.double().sum()) for a in applied) + res_total
    rhs = sum(float(t.double().sum()) for t in true_sum)
    assert abs(lhs - rhs) < 1e-3 * max(1.0, abs(rhs)), (lhs, rhs)
    blob = pickle.dumps(state)
    restored = pickle.loads(blob).attach(env)
    assert restored.compression_ratio == state.compression_ratio and len(restored._pending) > 0
    env.barrier()
    env.close()
    return True


@pytest.mark.parametrize("world", [2, 3])
def test_optimizer_replicas_stay_identical_cpu(world):
    out = run_ranks(world, "test_optimizer:scenario_optimizer_ranks", args=(False,))
    assert all(last < first for first, last in out)


def test_restart_with_more_ranks_cpu(tmp_path):
    saved = run_ranks(2, "test_optimizer:scenario_elastic_restart", args=(str(tmp_path), "save"))
    assert all(r > 0 and m > 0 for r, m in saved)
    loaded = run_ranks(3, "test_optimizer:scenario_elastic_restart", args=(str(tmp_path), "load"))
    assert loaded[2] == (0.0, 0.0) and loaded[0][0] == saved[0][0]


def test_data_parallel_wrapper_cpu():
    assert all(run_ranks(2, "test_optimizer:scenario_data_parallel"))


def test_ddp_hook_cpu():
    run_ranks(2, "test_optimizer:scenario_ddp_hook")


@pytest.mark.parametrize("kind,blob", [("comprex_ring", True), ("auto", True), ("comprex_alltoone", True),
                                       ("ring", True), ("bigring", True), ("alltoone", True),
                                       ("comprex_bigring", False), ("comprex_ring", False)])
def test_every_collective_runs_bucketed_cpu(kind, blob):
    out = run_ranks(2 if kind not in ("comprex_ring", "auto", "bigring") else 3, "test_optimizer:scenario_optimizer_kinds",
                    args=(kind, blob, False))
    assert all(last < first for first, last in out)


def test_single_rank_bypass_is_plain_momentum_sgd(device):
    """One rank exchanges nothing: the step is clip + local momentum + dense update, every step
    (with compression the same total would only arrive after a flush)."""
    env = cx.GaspiEnvironment(8 << 20, device=device)
    params = _const_grad_model(device)
    w0 = [p.detach().clone() for p in params]
    cs = [torch.randn_like(p) * 3 for p in params]
    lr, mu, clip = 0.1, 0.9, 5.0
    opt = ComprexOptimizer(params, env, lr=lr, momentum=mu, compression_ratio=0.01, pre_clipnorm=clip)
    assert opt._local and "single rank" in opt.describe()
    moms, refs = [torch.zeros_like(w) for w in w0], [w.clone() for w in w0]
    for _ in range(4):
        _set_grads(opt, params, cs)
        opt.step()
        for k, c in enumerate(cs):
            g = c * clip / max(float(c.norm()), clip)
            moms[k] = mu * moms[k] + lr * g
            refs[k] = refs[k] - moms[k]
        for p, ref in zip(params, refs):
            torch.testing.assert_close(p.detach(), ref, rtol=1e-5, atol=1e-5)
    assert opt.stats() == {} and not opt.comprex_allreducers
    sd = opt.state_dict()
    opt.load_state_dict(sd)
    env.close()


def test_nesterov_is_accepted_with_a_warning(device):
    env = cx.GaspiEnvironment(8 << 20, device=device)
    with pytest.warns(UserWarning, match="nesterov"):
        ComprexOptimizer(_const_grad_model(device), env, nesterov=True)
    env.close()


def test_checkpoint_follows_parameters_across_bucket_layouts(device):
    """State is keyed by parameter: a checkpoint written with one bucket size loads into an
    optimizer with another one (weights, momentum and residuals land at each parameter's new
    place), and a checkpoint for other parameters is refused."""
    def make(cap, seed=0):
        env = cx.GaspiEnvironment(8 << 20, device=device)
        torch.manual_seed(seed)
        model = LeNet5().to(device)
        opt = ComprexOptimizer(model.named_parameters(), env, single_rank_bypass=False, lr=0.02, momentum=0.9,
                               compression_ratio=0.02, size_factor=1.0, bucket_cap_mb=cap)
        return env, model, opt

    def steps(model, opt, k, start):
        for i in range(start, start + k):
            g = torch.Generator().manual_seed(i)
            x = torch.rand(16, 1, 28, 28, generator=g).to(device)
            y = torch.randint(0, 10, (16,), generator=g).to(device)
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
    env_a, model_a, opt_a = make(0.05)
    steps(model_a, opt_a, 5, 0)
    sd = copy.deepcopy(opt_a.state_dict())
    assert sd["comprex"]["version"] == 2 and sd["comprex"]["layout"][0][0].endswith(("weight", "bias"))
    env_b, model_b, opt_b = make(0.02, seed=1)
    assert len(opt_b._buckets) != len(opt_a._buckets)
    opt_b.load_state_dict(sd)
    by_key_a = {k: (o, p.numel()) for k, o, p in zip(opt_a._keys, opt_a._offsets, opt_a._params)}
    res_a, res_b = opt_a._residual_flat(), opt_b._residual_flat()
    assert float(res_a.abs().sum()) > 0
    for k, o, p in zip(opt_b._keys, opt_b._offsets, opt_b._params):
        oa, n = by_key_a[k]
        assert torch.equal(opt_b._master[o:o + n].cpu(), opt_a._master[oa:oa + n].cpu())
        assert torch.equal(opt_b._update[o:o + n].cpu(), opt_a._update[oa:oa + n].cpu())
        assert torch.equal(res_b[o:o + n], res_a[oa:oa + n])
    steps(model_b, opt_b, 2, 5)            # and training goes on
    other = ComprexOptimizer(_const_grad_model(device), env_b, single_rank_bypass=False)
    with pytest.raises(cx.ComprexError, match="other parameters"):
        other.load_state_dict(sd)
    env_a.close()
    env_b.close()


def test_data_parallel_restores_model_buffers(device):
    """BatchNorm running statistics live in the model's state, not in the optimizer's."""
    from comprex_b200.parallel.data_parallel import DataParallel

    def make(seed):
        torch.manual_seed(seed)
        model = torch.nn.Sequential(torch.nn.Conv2d(1, 4, 3), torch.nn.BatchNorm2d(4), torch.nn.ReLU(),
                                    torch.nn.Flatten(), torch.nn.Linear(4 * 26 * 26, 10)).to(device)
        env = cx.GaspiEnvironment(8 << 20, device=device)
        return env, model, DataParallel(model, env, lr=0.05, momentum=0.9)
    env_a, model_a, dp_a = make(0)
    for i in range(3):
        g = torch.Generator().manual_seed(i)
        x = torch.rand(8, 1, 28, 28, generator=g).to(device) * 3 + 1
        dp_a.zero_grad()
        model_a(x).square().mean().backward()
        dp_a.step()
    state = copy.deepcopy(dp_a.state_dict())
    env_b, model_b, dp_b = make(1)
    assert not torch.equal(model_b[1].running_mean, model_a[1].running_mean)
    dp_b.load_state_dict(state)
    assert torch.equal(model_b[1].running_mean, model_a[1].running_mean)
    assert torch.equal(model_b[1].running_var, model_a[1].running_var)
    assert int(model_b[1].num_batches_tracked) == 3
    for pa, pb in zip(model_a.parameters(), model_b.parameters()):
        assert torch.equal(pa, pb)
    env_a.close()
    env_b.close()


def _gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


@pytest.mark.gpu
@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("overlap", [False, True])
def test_optimizer_replicas_stay_identical_gpus(overlap):
    run_ranks(gpu_world(), "test_optimizer:scenario_optimizer_ranks", backend="nccl", args=(overlap,))


@pytest.mark.gpu
@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
def test_ddp_hook_gpus():
    run_ranks(gpu_world(), "test_optimizer:scenario_ddp_hook", backend="nccl")


@pytest.mark.gpu
@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("kind", ["comprex_ring", "auto", "ring"])
def test_every_collective_runs_bucketed_gpus(kind):
    out = run_ranks(gpu_world(), "test_optimizer:scenario_optimizer_kinds", backend="nccl", args=(kind, True, True))
    assert all(last < first for first, last in out)


@pytest.mark.gpu
def test_overlap_matches_no_overlap_single_gpu():
    """Hooks on a side stream give the same bits as launching everything in step()."""
    res = []
    for overlap in (False, True):
        torch.manual_seed(0)
        env = cx.GaspiEnvironment(16 << 20, device="cuda")
        model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, 96), torch.nn.ReLU(),
                                    torch.nn.Linear(96, 10)).cuda()
        opt = ComprexOptimizer(model.parameters(), env, single_rank_bypass=False, lr=0.05, compression_ratio=0.05, size_factor=1.0,
                               bucket_cap_mb=0.05, overlap=overlap)
        for i in range(6):
            g = torch.Generator().manual_seed(i)
            x = torch.rand(32, 1, 28, 28, generator=g).cuda()
            y = torch.randint(0, 10, (32,), generator=g).cuda()
            opt.zero_grad()
            torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
        env.flush()
        res.append(opt._master.clone())
        env.close()
    assert torch.equal(res[0], res[1])


@pytest.mark.gpu
def test_no_sync_accumulates_like_plain_accumulation():
    """Two micro-batches under ``no_sync`` plus one outside it (overlap on: the buckets go out
    during the last backward) give the bits of plain accumulation without overlap."""
    res = []
    for overlap in (False, True):
        torch.manual_seed(0)
        env = cx.GaspiEnvironment(16 << 20, device="cuda")
        model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(784, 96), torch.nn.ReLU(),
                                    torch.nn.Linear(96, 10)).cuda()
        opt = ComprexOptimizer(model.parameters(), env, single_rank_bypass=False, lr=0.05, compression_ratio=0.05, size_factor=1.0,
                               bucket_cap_mb=0.05, overlap=overlap)
        assert opt.overlap == overlap and len(opt._buckets) > 1
        for step in range(4):
            opt.zero_grad()
            for micro in range(3):
                g = torch.Generator().manual_seed(10 * step + micro)
                x = torch.rand(16, 1, 28, 28, generator=g).cuda()
                y = torch.randint(0, 10, (16,), generator=g).cuda()
                if micro < 2:
                    with opt.no_sync():
                        torch.nn.functional.cross_entropy(model(x), y).backward()
                else:
                    torch.nn.functional.cross_entropy(model(x), y).backward()
            opt.step()
        env.flush()
        res.append(opt._master.clone())
        env.close()
    assert torch.equal(res[0], res[1])
