"""Worker bodies for multi-process tests (spawned with torch.multiprocessing)."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _init(rank: int, world: int, port: int, backend: str) -> None:
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    if backend == "nccl":
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world,
                                device_id=torch.device("cuda", rank))
    else:
        dist.init_process_group("gloo", rank=rank, world_size=world)


def sharded_adamw_matches_single(rank, world, port, backend, collectives, out):
    """Sharded reduce+clip+AdamW over `world` ranks equals one AdamW on the mean gradient."""
    import copy

    from visionrl_b200.ops.optim import FusedAdamW
    from visionrl_b200.parallel.mesh import ProcessMesh
    from visionrl_b200.parallel.sharded import ShardedGradSync

    _init(rank, world, port, backend)
    dev = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    dtype = torch.bfloat16 if backend == "nccl" else torch.float32
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.Linear(40, 8)).to(dev, dtype)
    ref = copy.deepcopy(net).float()
    mesh = ProcessMesh.build()
    sync = ShardedGradSync(mesh, collectives=collectives)
    opt = FusedAdamW(net.parameters(), lr=1e-2, weight_decay=0.01)
    sync.prepare(opt)
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    norms = []
    for step in range(3):
        grads_all = []
        for r in range(world):
            g = torch.Generator().manual_seed(100 * step + r)
            grads_all.append([torch.randn(p.shape, generator=g) for p in ref.parameters()])
        opt.flat_buffers()
        for p, g in zip(net.parameters(), grads_all[rank]):
            p.grad.copy_(g.to(dev, dtype))
        if dev.type == "cuda":
            torch.cuda.synchronize()
        norm = sync.reduce_clip_step(opt, max_norm=1.0)
        norms.append(float(norm))
        mean = [sum(gs[i].to(dtype).float() for gs in grads_all) / world
                for i in range(len(grads_all[0]))]
        for p, g in zip(ref.parameters(), mean):
            p.grad = g.clone().to(p.device)
        ref_norm = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        ref_opt.step()
        tol = 3e-2 if dtype == torch.bfloat16 else 1e-5
        assert abs(float(ref_norm) - norms[-1]) <= tol * max(1.0, float(ref_norm)), (ref_norm, norm)
    if dev.type == "cuda":
        torch.cuda.synchronize()
    err = max((a.detach().float().cpu() - b.detach().float().cpu()).abs().max().item()
              for a, b in zip(net.parameters(), ref.parameters()))
    # every rank must hold identical parameters after the all-gather
    flat = torch.cat([p.detach().float().reshape(-1) for p in net.parameters()]).to(dev)
    gathered = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(gathered, flat)
    same = all(torch.equal(gathered[0], t) for t in gathered)
    state = opt.state_dict()      # collective when sharded
    if rank == 0:
        out.put({"err": err, "same": same, "norms": norms,
                 "state_keys": sorted(state["state"].keys()),
                 "launches": getattr(sync, "kernel_launches", 0)})
    dist.barrier()
    dist.destroy_process_group()


def ulysses_attention_matches_dense(rank, world, port, backend, use_kernels, out):
    """Sequence-parallel attention equals dense attention on the full sequence.  Library path:
    q / k / v in, all-to-all exchanges.  Fused path: the QKV projection output in, exchanges done by
    the producing kernels' stores; checked with and without gradients, several layers in a row so
    that the double-buffered exchange slots and their flags wrap around."""
    from visionrl_b200.ops.attention import attention_reference
    from visionrl_b200.ops.qkv import qkv_prepare_reference
    from visionrl_b200.parallel.mesh import ProcessMesh
    from visionrl_b200.parallel.ulysses import SequenceParallel

    _init(rank, world, port, backend)
    dev = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    dtype = torch.bfloat16 if backend == "nccl" else torch.float32
    mesh = ProcessMesh.build(sp=world)
    pool = None
    if use_kernels:
        from visionrl_b200.parallel.symm import SymmetricPool

        pool = SymmetricPool(mesh, group=mesh.sp_group)
    sp = SequenceParallel(mesh, pool)
    torch.manual_seed(1)
    b, h, s, d = 2, 4 * world, 16 * world, 64
    sl = slice(rank * s // world, (rank + 1) * s // world)
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    ok_fwd = ok_bwd = True
    if not use_kernels:
        q, k, v = (torch.randn(b, h, s, d).to(dev, dtype) for _ in range(3))
        ql, kl, vl = (t[:, :, sl].clone().requires_grad_() for t in (q, k, v))
        o = sp.attention(ql, kl, vl)
        w = torch.randn(b, h, s, d, generator=torch.Generator().manual_seed(5)).to(dev, dtype)
        (o.float() * w[:, :, sl].float()).sum().backward()
        qf, kf, vf = (t.float().requires_grad_() for t in (q, k, v))
        of = attention_reference(qf, kf, vf)
        (of * w.float()).sum().backward()
        ok_fwd = torch.allclose(o.float(), of[:, :, sl], atol=tol, rtol=tol)
        ok_bwd = all(torch.allclose(a.grad.float(), b_.grad[:, :, sl], atol=tol * 4, rtol=tol * 4)
                     for a, b_ in ((ql, qf), (kl, kf), (vl, vf)))
    else:
        gen = torch.Generator().manual_seed(3)
        qw = (1 + 0.1 * torch.randn(h * d, generator=gen)).to(dev, dtype)
        kw = (1 + 0.1 * torch.randn(h * d, generator=gen)).to(dev, dtype)
        ang = torch.rand(s, d // 2, generator=gen) * 6.28
        cos, sin = torch.cos(ang).to(dev), torch.sin(ang).to(dev)
        for layer in range(5):                  # > 2 exchanges per kind: slots and flags wrap
            qkv = torch.randn(b, s, 3 * h * d, generator=gen).to(dev, dtype)
            wgt = torch.randn(b, s, h * d, generator=gen).to(dev)
            # dense oracle on the full sequence, fp32
            qkv_f = qkv.float().requires_grad_()
            qw_f, kw_f = qw.float().requires_grad_(), kw.float().requires_grad_()
            qf, kf, vf = qkv_prepare_reference(qkv_f, h, qw_f, kw_f, 1e-6, (cos, sin))
            of = attention_reference(qf, kf, vf).transpose(1, 2).reshape(b, s, h * d)
            (of * wgt).sum().backward()
            with_grad = layer % 2 == 0
            local = qkv[:, sl].clone().requires_grad_(with_grad)
            qw_l, kw_l = qw.clone().requires_grad_(with_grad), kw.clone().requires_grad_(with_grad)
            assert sp.can_fuse(local, h)
            with torch.set_grad_enabled(with_grad):
                o = sp.fused_attention(local, h, qw_l, kw_l, (cos[sl], sin[sl]))
            ok_fwd = ok_fwd and torch.allclose(o.float(), of[:, sl].detach(), atol=tol, rtol=tol)
            if with_grad:
                (o.float() * wgt[:, sl]).sum().backward()
                scale = max(1.0, qkv_f.grad.abs().max().item())
                ok_bwd = ok_bwd and (local.grad.float() - qkv_f.grad[:, sl]).abs().max().item() <= 4 * tol * scale
                # norm-weight gradients are partial sums over this rank's tokens
                gq = qw_l.grad.float().clone()
                dist.all_reduce(gq)
                ok_bwd = ok_bwd and torch.allclose(gq, qw_f.grad, atol=0.15, rtol=0.1)
        torch.cuda.synchronize()
        pool.check("fused ulysses test")
    flags = torch.tensor([float(ok_fwd), float(ok_bwd)], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put({"fwd": bool(flags[0]), "bwd": bool(flags[1]), "launches": sp.kernel_launches,
                 "fused_layers": sp.fused_layers})
    dist.barrier()
    dist.destroy_process_group()


def weight_broadcast_and_timeout(rank, world, port, out):
    """Owner publishes a versioned buffer to every replica; a wait on a version nobody
    publishes runs out and reports instead of hanging."""
    from visionrl_b200.parallel.mesh import ProcessMesh
    from visionrl_b200.parallel.symm import CollectiveTimeout, SymmetricPool
    from visionrl_b200.parallel.weight_broadcast import DeviceWeightBroadcaster

    _init(rank, world, port, "nccl")
    dev = torch.device("cuda", rank)
    mesh = ProcessMesh.build()
    pool = SymmetricPool(mesh)
    n = 1 << 16
    bc = DeviceWeightBroadcaster(pool, n * world, torch.bfloat16, dev)
    shard = torch.full((n,), float(rank + 1), device=dev, dtype=torch.bfloat16)
    version = bc.publish(shard, offset_elems=rank * n)
    for owner in range(world):
        bc.wait_version(owner, version, timeout_s=5.0)
    torch.cuda.synchronize()
    want = torch.cat([torch.full((n,), float(r + 1)) for r in range(world)])
    ok = torch.equal(bc.replica.float().cpu(), want)
    timed_out = False
    try:
        bc.wait_version((rank + 1) % world, version + 7, timeout_s=0.2)
    except CollectiveTimeout:
        timed_out = True
    flags = torch.tensor([float(ok), float(timed_out)], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put({"ok": bool(flags[0]), "timed_out": bool(flags[1])})
    dist.barrier()
    dist.destroy_process_group()


def allgather_gemm_matches_library(rank, world, port, out):
    """The GEMM with the all-gather fused in equals all_gather + matmul, also on a second call."""
    from visionrl_b200.ops import _ext
    from visionrl_b200.parallel.mesh import ProcessMesh
    from visionrl_b200.parallel.sharded_linear import ShardedLinearWeight
    from visionrl_b200.parallel.symm import SymmetricPool

    _init(rank, world, port, "nccl")
    dev = torch.device("cuda", rank)
    mesh = ProcessMesh.build()
    pool = SymmetricPool(mesh)
    results = []
    for (m, n, k, act, use_bias) in [(1000, 1536, 512, None, False), (4096, 4608, 1536, "gelu_tanh", True)]:
        gen = torch.Generator().manual_seed(7)
        w = (torch.randn(n, k, generator=gen) * 0.05).to(dev)
        b = (torch.randn(n, generator=gen) * 0.1).to(dev)
        x = torch.randn(m, k, generator=torch.Generator().manual_seed(100 + rank)).to(dev, torch.bfloat16)
        layer = ShardedLinearWeight(pool, n, k, dev, bias=use_bias)
        layer.load_full(w)
        if use_bias:
            layer.bias.copy_(b)
        torch.cuda.synchronize()
        pool.barrier()
        ref = torch.nn.functional.linear(x.float(), w.bfloat16().float(), b.bfloat16().float() if use_bias else None)
        if act == "gelu_tanh":
            ref = torch.nn.functional.gelu(ref, approximate="tanh")
        for _ in range(2):
            layer.full.fill_(float("nan"))            # stale contents must never be read
            got = layer.forward(x, act)
            torch.cuda.synchronize()
            status = _ext.load().gemm_last_status()
            ok = status == 0 and bool(torch.isfinite(got.float()).all()) and torch.allclose(
                got.float(), ref, atol=6e-2, rtol=3e-2)
            results.append(ok)
            pool.barrier()
        layer.collectives = "nccl"
        base = layer.forward(x, act)
        results.append(torch.allclose(base.float(), ref, atol=6e-2, rtol=3e-2))
        results.append(layer.kernel_launches == 2)
    flags = torch.tensor([float(all(results))], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    if rank == 0:
        out.put({"ok": bool(flags[0]), "detail": results})
    dist.barrier()
    dist.destroy_process_group()


def _tiny_mmdit(dev, dtype, layers=3):
    from visionrl_b200.models.nn.mmdit import MMDiT, MMDiTConfig

    torch.manual_seed(3)
    cfg = MMDiTConfig(num_layers=layers, hidden_size=128, num_heads=2, patch_size=2, in_channels=4,
                      context_dim=64, pooled_dim=32, max_grid=8)
    return MMDiT(cfg).to(dev, dtype)


def _mmdit_inputs(seed, dev, dtype, batch=2):
    g = torch.Generator().manual_seed(seed)
    lat = torch.randn(batch, 4, 8, 8, generator=g).to(dev, dtype)
    t = torch.rand(batch, generator=g).to(dev) * 1000
    ctx = torch.randn(batch, 8, 64, generator=g).to(dev, dtype)
    pooled = torch.randn(batch, 32, generator=g).to(dev, dtype)
    target = torch.randn(batch, 4, 8, 8, generator=g).to(dev)
    return lat, t, ctx, pooled, target


def fsdp_training_matches_replicated(rank, world, port, backend, collectives, replicate, checkpointing, out,
                                     replica=True):
    """Block weights sharded over the ranks (gather in the consuming GEMM, bucketed reduce-scatter
    during backward, sharded AdamW) train exactly like one replicated model on the mean gradient."""
    import copy

    from visionrl_b200.ops.linear import accumulate_weight_grads_in_place
    from visionrl_b200.ops.optim import FusedAdamW
    from visionrl_b200.parallel.fsdp import shard_model
    from visionrl_b200.parallel.mesh import ProcessMesh
    from visionrl_b200.parallel.sharded import ShardedGradSync

    _init(rank, world, port, backend)
    dev = torch.device("cuda", rank) if backend == "nccl" else torch.device("cpu")
    dtype = torch.bfloat16 if backend == "nccl" else torch.float32
    net = _tiny_mmdit(dev, dtype)
    ref = copy.deepcopy(net).float().cpu()
    net.enable_gradient_checkpointing(checkpointing)
    mesh = ProcessMesh.build(replicate=replicate)
    rt = shard_model(net, mesh, dev, collectives=collectives, ring=2, rollout_replica=replica)
    assert rt is not None and len(rt.handles) > 0
    sync = ShardedGradSync(mesh, collectives=collectives, param_runtime=rt)
    opt = FusedAdamW([p for p in net.parameters() if p.requires_grad], lr=1e-2, weight_decay=0.01)
    sync.prepare(opt)
    ref_opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, weight_decay=0.01)
    micro = 2
    fwd_err = 0.0
    for step in range(2):
        opt.flat_buffers()
        for mb in range(micro):
            lat, t, ctx, pooled, target = _mmdit_inputs(1000 * step + 10 * mb + rank, dev, dtype)
            pred = net(lat, t, ctx, pooled)
            loss = ((pred.float() - target) ** 2).mean() / micro
            with accumulate_weight_grads_in_place():
                loss.backward()
        norm = sync.reduce_clip_step(opt, max_norm=1.0)
        sync.check("test step")
        # reference: the same micro-batches of every rank on one replicated fp32 model
        for r in range(world):
            for mb in range(micro):
                lat, t, ctx, pooled, target = _mmdit_inputs(1000 * step + 10 * mb + r, torch.device("cpu"),
                                                            torch.float32)
                pred = ref(lat, t, ctx, pooled)
                (((pred - target) ** 2).mean() / micro / world).backward()
        ref_norm = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        ref_opt.step()
        ref_opt.zero_grad()
        tol = 5e-2 if dtype == torch.bfloat16 else 1e-4
        assert abs(float(ref_norm) - float(norm)) <= tol * max(1.0, float(ref_norm)), (float(ref_norm), float(norm))
    # no-grad forward (the rollout path) through the gathered weights
    with torch.no_grad():
        lat, t, ctx, pooled, _ = _mmdit_inputs(77, dev, dtype)
        got = net(lat, t, ctx, pooled).float().cpu()
        want = ref(*(_mmdit_inputs(77, torch.device("cpu"), torch.float32)[:4]))
        fwd_err = (got - want).abs().max().item()
        gathers_before = rt.gathers
        net(lat, t, ctx, pooled)
        replica_used = rt.gathers == gathers_before       # a no-grad forward needs no gather
    if replica:
        rt.verify_replicas()                              # every rank holds the same replica bits
        if rank == world - 1:
            # a torn replica on one rank must be noticed by all of them (host-side injection)
            rt.replica_flat[7] += 1.0
        try:
            rt.verify_replicas()
            caught = False
        except RuntimeError as exc:
            caught = "replicas differ" in str(exc)
        assert caught, "a replica that differs on one rank went unnoticed"
        if rank == world - 1:
            rt.replica_flat[7] -= 1.0
    full = net.state_dict()          # gathers every sharded weight to its full shape
    ref_state = ref.state_dict()
    err = max((full[k].float().cpu() - ref_state[k]).abs().max().item() for k in ref_state)
    shapes_ok = all(tuple(full[k].shape) == tuple(ref_state[k].shape) for k in ref_state)
    opt_state = opt.state_dict()
    report = rt.memory_report()
    flags = torch.tensor([err, fwd_err], device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MAX)
    if rank == 0:
        out.put({"err": float(flags[0]), "fwd_err": float(flags[1]), "shapes_ok": shapes_ok,
                 "handles": len(rt.handles), "buckets": rt.buckets_reduced, "gathers": rt.gathers,
                 "fused_gathers": rt.fused_gathers, "report": report, "replica_used": replica_used,
                 "broadcasts": rt.broadcasts,
                 "opt_entries": len(opt_state["state"]),
                 "params": sum(1 for _ in net.parameters())})
    dist.barrier()
    dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# Failure detection: every fault below is made on the host (an exception, a silent thread, a
# process that leaves between steps); no device is involved.
# ---------------------------------------------------------------------------------------------
def _fake_trainer(rank, world, fail_on_step=None, liveness=None):
    from tests.trainers.test_online import _FakeAlgorithm, _FakeCollector, _FakeEvaluator
    from visionrl_b200.trainers.online import OnlineTrainer
    from visionrl_b200.trainers.types import TrainerConfig

    class _FailingCollector(_FakeCollector):
        step = 0

        async def collect(self, prompts, group_size, **kwargs):
            if fail_on_step is not None and self.step == fail_on_step:
                raise RuntimeError("injected collector failure")
            self.step += 1
            return await super().collect(prompts, group_size, **kwargs)

    torch.manual_seed(0)
    cfg = TrainerConfig(n=2, rollout_batch_size=2, bf16=False)
    return OnlineTrainer(_FakeAlgorithm(), _FailingCollector([]), _FakeEvaluator(), torch.nn.Linear(1, 1),
                         config=cfg, prompts=["a", "b"], device="cpu", liveness=liveness)


def rank_raises_between_steps(rank, world, port, out):
    """Rank 1's second step raises; rank 0 learns of it from the store before its next step."""
    import asyncio
    import time

    from visionrl_b200.parallel.liveness import RankFailure, RankLiveness, default_store

    _init(rank, world, port, "gloo")
    live = RankLiveness(default_store(), rank, world, interval_s=0.1, deadline_s=5.0).start()
    trainer = _fake_trainer(rank, world, fail_on_step=1 if rank == 1 else None, liveness=live)
    loop = asyncio.new_event_loop()
    loop.run_until_complete(trainer.step())
    dist.barrier()                      # both ranks finished step 0; nothing is in flight
    result = {}
    if rank == 1:
        try:
            loop.run_until_complete(trainer.step())
            result["raised"] = False
        except RuntimeError as exc:
            result["raised"] = "injected" in str(exc)
    else:
        t0 = time.time()
        caught = None
        while time.time() - t0 < 4.0:
            try:
                loop.run_until_complete(trainer.step())
            except RankFailure as exc:
                caught = exc
                break
            time.sleep(0.05)
        result = {"detected": caught is not None, "failed_rank": getattr(caught, "rank", None),
                  "reason": getattr(caught, "reason", ""), "seconds": time.time() - t0}
        out.put(result)
    live.stop()
    # no barrier: the failed rank leaves; the survivor must not wait for it


def heartbeat_withheld(rank, world, port, out):
    """Rank 1 stays alive but its heartbeat thread stops; rank 0 notices after the deadline."""
    import time

    from visionrl_b200.parallel.liveness import RankFailure, RankLiveness, default_store

    _init(rank, world, port, "gloo")
    live = RankLiveness(default_store(), rank, world, interval_s=0.1, deadline_s=0.8).start()
    dist.barrier()
    if rank == 1:
        live.stop()                    # the process lives on, silent
        time.sleep(2.5)
    else:
        live.check()                   # fresh heartbeats: no complaint
        t0 = time.time()
        caught = None
        while time.time() - t0 < 2.3:
            try:
                live.check()
            except RankFailure as exc:
                caught = exc
                break
            time.sleep(0.05)
        out.put({"detected": caught is not None, "failed_rank": getattr(caught, "rank", None),
                 "reason": getattr(caught, "reason", ""), "seconds": time.time() - t0})
        live.stop()


def rank_leaves_between_steps(rank, world, port, out):
    """A rank exits between steps; the survivor's next collective fails within the (short)
    process-group timeout instead of blocking."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    t = torch.ones(4)
    dist.all_reduce(t)                  # step 0 completes on both ranks
    dist.barrier()
    if rank == 1:
        return                          # leaves with nothing in flight
    time.sleep(0.5)
    t0 = time.time()
    failed = False
    try:
        dist.all_reduce(torch.ones(4))
    except Exception:  # noqa: BLE001 - gloo reports a closed connection or a timeout
        failed = True
    out.put({"failed": failed, "seconds": time.time() - t0})


def barrier_times_out_when_a_rank_skips(rank, world, port, out):
    """GPU, host-side injection: rank 1 never enters the second barrier; rank 0's bounded wait
    gives up, the stream keeps running, and the host raises CollectiveTimeout."""
    import time

    from visionrl_b200.parallel.mesh import ProcessMesh
    from visionrl_b200.parallel.symm import CollectiveTimeout, SymmetricPool

    os.environ["NCCL_NVLS_ENABLE"] = "0"
    _init(rank, world, port, "nccl")
    mesh = ProcessMesh.build()
    pool = SymmetricPool(mesh, timeout_s=5.0)
    pool.barrier()
    pool.check("first barrier")          # everybody arrives: fine
    result = {}
    if rank == 0:
        t0 = time.time()
        pool.barrier(timeout_s=0.5)      # rank 1 does not call this one
        probe = torch.ones(8, device="cuda") * 3      # the stream is still usable afterwards
        try:
            pool.check("skipped barrier")
            result["timed_out"] = False
        except CollectiveTimeout as exc:
            result["timed_out"] = True
            result["message"] = str(exc)
        result["seconds"] = time.time() - t0
        result["stream_ok"] = float(probe.sum().item()) == 24.0
        out.put(result)
    dist.barrier()                       # both ranks leave together, nothing in flight
    dist.destroy_process_group()


def wan_recipe_runs_sharded_and_sequence_parallel(rank, world, port, sp, out_dir, resume_port, out):
    """The Wan GRPO recipe end to end on CPU ranks, through the public entry point: sequence-parallel
    attention over ``sp`` ranks, block weights sharded over all ranks, one epoch, metrics on rank 0."""
    import asyncio
    import csv
    import inspect
    import json
    import pathlib

    from visionrl_b200.config.loader import load_config
    from visionrl_b200.scripts.train import run_config

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    overrides = [
        "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2", "model.arch.ffn_dim=128",
        "model.arch.text_dim=32", "model.arch.freq_dim=32", "model.dtype=float32",
        "sampling.num_frames=5", "sampling.height=32", "sampling.width=32", "sampling.num_steps=3",
        "sampling.max_sequence_length=8", "rollout.n=2", f"rollout.rollout_batch_size={max(1, world // sp)}",
        "rollout.sample_batch_size=2", "trainer.total_epochs=1", f"trainer.output_dir={out_dir}",
        "trainer.save_freq=0", "trainer.debug.first_step=true", "reward.kwargs.vit_scalar.preset=vit_tiny",
        f"distributed.mesh.sp={sp}", "distributed.collectives=nccl", "distributed.param_sharding=full",
        "distributed.heartbeat.enable=false", "actor.gradient_checkpointing=true",
    ]
    def train(extra):
        cfg = load_config("experiment/wan_2_1_1_3b_shape_grpo", overrides=overrides + extra)
        result = run_config(cfg)
        if inspect.isawaitable(result):
            asyncio.new_event_loop().run_until_complete(result)

    train([])
    # the resumed run is a new job: it gets its own rendezvous port (a second process group on the
    # first one's port, inside the same process, can meet the first store's leftovers)
    os.environ["MASTER_PORT"] = str(resume_port)
    # resume from the final checkpoint (written by rank 0 from gathered, full-shape weights and
    # optimiser state; every rank reads it back and keeps its own rows) for one more epoch
    train(["trainer.total_epochs=2", f"trainer.resume_from={out_dir}/checkpoint-final"])
    if rank == 0:
        rows = list(csv.reader((pathlib.Path(out_dir) / "metrics.csv").open()))
        perf = [json.loads(line) for line in (pathlib.Path(out_dir) / "perf.jsonl").read_text().splitlines()]
        out.put({"rows": rows, "perf": perf})
    if dist.is_initialized():
        dist.destroy_process_group()


def recipe_runs_on_cpu_ranks(rank, world, port, experiment, overrides, out_dir, resume_port, out):
    """Any online recipe through the public entry point on ``world`` gloo ranks: one epoch, the final
    checkpoint, a resumed second epoch; rank 0 reports the CSV rows and the performance lines."""
    import asyncio
    import csv
    import inspect
    import json
    import pathlib

    from visionrl_b200.config.loader import load_config
    from visionrl_b200.scripts.train import run_config

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    base = list(overrides) + [f"trainer.output_dir={out_dir}", "trainer.total_epochs=1", "trainer.save_freq=0",
                              "distributed.backend=native", "distributed.collectives=nccl",
                              "distributed.heartbeat.enable=false"]

    def train(extra):
        result = run_config(load_config(experiment, overrides=base + extra))
        if inspect.isawaitable(result):
            asyncio.new_event_loop().run_until_complete(result)

    train([])
    os.environ["MASTER_PORT"] = str(resume_port)          # the resumed run is a new job with its own rendezvous
    train(["trainer.total_epochs=2", f"trainer.resume_from={out_dir}/checkpoint-final"])
    if rank == 0:
        rows = list(csv.reader((pathlib.Path(out_dir) / "metrics.csv").open()))
        perf = [json.loads(line) for line in (pathlib.Path(out_dir) / "perf.jsonl").read_text().splitlines()]
        out.put({"rows": rows, "perf": perf})
    if dist.is_initialized():
        dist.destroy_process_group()


def recipe_restarts_in_place_after_a_rank_raises(rank, world, port, out_dir, second_port, out):
    """Three epochs of the tiny recipe on gloo ranks under the in-place restart loop.  On the first
    attempt rank 1's third step raises on the host before it launches anything (two epochs are
    checkpointed by then); every rank leaves the group, meets again at the second port and resumes
    from the latest checkpoint.  Rank 0 reports rows, restarts and the attempts it made."""
    import csv
    import pathlib

    from visionrl_b200.scripts import elastic

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), VRL_FAULT_INJECT="rank=1,step=2")
    attempts = []
    overrides = ["sampling.num_steps=3", "rollout.n=2", "rollout.rollout_batch_size=2", "rollout.sample_batch_size=2",
                 f"trainer.output_dir={out_dir}", "trainer.total_epochs=3", "trainer.save_freq=1",
                 "distributed.backend=native", "distributed.collectives=nccl",
                 "distributed.heartbeat.interval_s=0.2", "distributed.heartbeat.deadline_s=20",
                 "distributed.timeout_s=20"]
    _, restarts = elastic.run_with_restarts("experiment/tiny_dit_grpo", overrides, max_restarts=1,
                                            ports=[port, second_port], before_attempt=attempts.append)
    if dist.is_initialized():
        dist.destroy_process_group()
    if rank == 0:
        root = pathlib.Path(out_dir)
        out.put({"rows": list(csv.reader((root / "metrics.csv").open())), "restarts": restarts,
                 "attempts": attempts, "checkpoints": sorted(p.name for p in root.glob("checkpoint-*")),
                 "resume_configs": len(list(root.glob("resume_config_*.yaml")))})


def dpo_recipe_runs_on_cpu_ranks(rank, world, port, overrides, out_dir, resume_port, out):
    """The preference recipe on ``world`` gloo ranks: three steps with a checkpoint after the second,
    then a resumed run up to step five; rank 0 reports the CSV rows and the checkpoints."""
    import asyncio
    import csv
    import inspect
    import pathlib

    from visionrl_b200.config.loader import load_config
    from visionrl_b200.scripts.train import run_config

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    base = list(overrides) + [f"trainer.output_dir={out_dir}", "trainer.checkpointing_steps=2", "trainer.log_interval=1",
                              "+distributed.backend=native", "+distributed.collectives=nccl"]

    def train(extra):
        result = run_config(load_config("experiment/wan_2_1_1_3b_shape_dpo", overrides=base + extra))
        if inspect.isawaitable(result):
            asyncio.new_event_loop().run_until_complete(result)
        if dist.is_initialized():
            dist.destroy_process_group()

    train(["trainer.max_train_steps=3"])
    os.environ["MASTER_PORT"] = str(resume_port)
    train(["trainer.max_train_steps=5", "trainer.resume_from=auto"])
    if rank == 0:
        root = pathlib.Path(out_dir)
        out.put({"rows": list(csv.reader((root / "metrics.csv").open())),
                 "checkpoints": sorted(p.name for p in root.glob("checkpoint-*"))})
