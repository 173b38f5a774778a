"""Sharded data-parallel optimiser step: gradient reduce-scatter ⊕ clip ⊕ AdamW ⊕ parameter
all-gather over flat buffers.

Two kinds of parameters pass through here.  The transformer-block weights that a
:class:`visionrl_b200.parallel.fsdp.ShardedParamRuntime` has sharded (``param_runtime``)
already have their gradients reduced bucket by bucket during the backward pass; this step
only waits for the last bucket, adds their sum of squares to the global norm and runs their
sharded AdamW.  Everything else (embedders, biases, norm weights — a per-cent of the model)
is handled as flat buffers: every rank holds those bf16 parameters whole but only
``1/world`` of their fp32 master weights and Adam moments.  After backward the flat bf16
gradient buffer of every rank holds that rank's partial sum.  ``reduce_clip_step`` then

1. reduces the partials so that rank ``r`` owns the mean gradient of slice ``r``
   (reduce-scatter),
2. forms the global gradient norm from the per-slice sums of squares (one tiny all-reduce)
   and the clip coefficient, on the device,
3. updates slice ``r`` of master weights / moments / bf16 parameters, and
4. publishes the updated bf16 slice to every rank (all-gather).

``collectives="fused"`` runs steps 1, 3 and 4 inside hand-written kernels that read the
peers' gradient slices and write the peers' parameter slices directly over NVLink
(symmetric memory, :mod:`visionrl_b200.parallel.symm`); ``"nccl"`` is the library
baseline (``reduce_scatter_tensor`` / ``all_gather_into_tensor``), and on CPU/gloo an
all-reduce based variant keeps the same semantics for tests.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from visionrl_b200.parallel.mesh import ProcessMesh, dist_ready


class ShardedGradSync:
    def __init__(self, mesh: ProcessMesh, shard_optimizer: bool = True,
                 collectives: str = "fused", param_runtime: Any | None = None) -> None:
        self.mesh = mesh
        self.shard_optimizer = shard_optimizer and mesh.world_size > 1
        self.collectives = collectives
        self.param_runtime = param_runtime if (param_runtime is not None
                                               and param_runtime.active) else None
        self._symm = None
        self.kernel_launches = 0
        # ranks of one sequence-parallel group hold partial sums of the same samples' gradient
        # (sum them), data-parallel ranks hold different samples (average them)
        self.grad_scale = float(mesh.sp) / float(max(mesh.world_size, 1))

    # -- set-up ----------------------------------------------------------------------------
    def prepare(self, optimizer: Any) -> None:
        """Configure ``optimizer`` (a flat ``FusedAdamW``) before its buffers are built."""
        if self.mesh.world_size <= 1:
            return
        if self.shard_optimizer and hasattr(optimizer, "set_shard") and not optimizer._built:
            optimizer.set_shard(self.mesh.rank, self.mesh.world_size)
        if (self.collectives == "fused" and torch.cuda.is_available() and not optimizer._built
                and self.shard_optimizer):
            from visionrl_b200.ops import _ext
            from visionrl_b200.parallel.symm import SymmetricPool

            if _ext.kernels_enabled():
                rt = self.param_runtime
                shared = rt.pool if (rt is not None and rt.pool is not None
                                     and rt.pool.world == self.mesh.world_size) else None
                self._symm = shared or SymmetricPool(self.mesh)
                optimizer.set_allocator(self._symm.allocate)

    # -- the step ----------------------------------------------------------------------------
    @torch.no_grad()
    def reduce_clip_step(self, optimizer: Any, max_norm: float) -> torch.Tensor:
        world = self.mesh.world_size
        flat = optimizer.flat_buffers()
        rt = self.param_runtime
        if rt is not None:
            rt.finish_grads()
        if world <= 1 or not dist_ready():
            norm = optimizer.grad_norm()
            coef = (max_norm / (norm + 1e-6)).clamp(max=1.0) if max_norm > 0 else None
            optimizer.step(clip_coef=coef)
            optimizer.zero_grad()
            return norm
        if self._symm is not None and all(e["param"].is_cuda for e in flat):
            for e in flat:
                if not (e["master"].is_cuda and e["exp_avg"].is_cuda and e["exp_avg_sq"].is_cuda):
                    raise RuntimeError(
                        "the fused sharded step needs the optimiser state on the device; it was "
                        "moved (optimizer-state offload hooks only run around optimizer.step(), "
                        "which this path does not call) — use collectives='nccl' with offload")
            return self._fused_step(optimizer, flat, max_norm)
        return self._library_step(optimizer, flat, max_norm)

    # -- the sharded block weights' part of the step -----------------------------------------
    def _runtime_sumsq(self, sq_total):
        rt = self.param_runtime
        if rt is None:
            return sq_total
        # with replica groups (HSDP) every shard exists `replicas` times in the all-reduce
        sq = rt.grad_sumsq() / float(rt.replicas)
        return sq if sq_total is None else sq_total + sq

    def _runtime_step(self, optimizer, coef) -> None:
        rt = self.param_runtime
        if rt is not None:
            rt.adamw_step(optimizer.param_groups[0], coef)

    def check(self, what: str = "sharded optimiser step") -> None:
        """Raise :class:`~visionrl_b200.parallel.symm.CollectiveTimeout` if a bounded wait on a
        peer expired since the last check (one small device-to-host read)."""
        pools = {id(p): p for p in (self._symm, getattr(self.param_runtime, "pool", None))
                 if p is not None}
        for pool in pools.values():
            pool.check(what)

    def _library_step(self, optimizer, flat, max_norm: float) -> torch.Tensor:
        world, rank = self.mesh.world_size, self.mesh.rank
        sq_total = None
        for e in flat:
            n, lo = e["shard"], e["lo"]
            g = e["grad"]
            if g.is_cuda and self.shard_optimizer:
                shard = torch.empty(n, dtype=g.dtype, device=g.device)
                dist.reduce_scatter_tensor(shard, g, op=dist.ReduceOp.SUM)
                shard.mul_(self.grad_scale)
            else:
                dist.all_reduce(g, op=dist.ReduceOp.SUM)
                g.mul_(self.grad_scale)
                shard = g[lo:lo + n] if self.shard_optimizer else g
            e["grad_shard"] = shard if self.shard_optimizer else None
            sq = shard.float().pow(2).sum()
            if not self.shard_optimizer:
                sq = sq / world     # every rank holds the whole gradient
            sq_total = sq if sq_total is None else sq_total + sq
        sq_total = self._runtime_sumsq(sq_total)
        dist.all_reduce(sq_total, op=dist.ReduceOp.SUM)
        norm = sq_total.sqrt()
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0) if max_norm > 0 else None
        optimizer.step(clip_coef=coef)
        self._runtime_step(optimizer, coef)
        if self.shard_optimizer:
            for e in flat:
                p = e["param"]
                own = p[e["lo"]:e["lo"] + e["shard"]].contiguous()
                if p.is_cuda:
                    dist.all_gather_into_tensor(p, own)
                else:
                    parts = [torch.empty_like(own) for _ in range(world)]
                    dist.all_gather(parts, own)
                    p.copy_(torch.cat(parts))
                e["grad_shard"] = None
        if self.param_runtime is not None:
            self.param_runtime.publish()
        optimizer.zero_grad()
        return norm

    def _fused_step(self, optimizer, flat, max_norm: float) -> torch.Tensor:
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        symm = self._symm
        world, rank = self.mesh.world_size, self.mesh.rank
        sq_total = None
        # every rank's backward (which wrote its partial gradients) must be complete
        symm.barrier()
        # phase 1: sum the peers' partials of the owned slice with P2P loads -> fp32 mean gradient
        for e in flat:
            if "grad_f32" not in e:
                e["grad_f32"] = torch.empty(e["shard"], dtype=torch.float32, device=e["grad"].device)
            sq = ext.rs_sum_slice(symm.peer_pointers(e["grad"]), e["grad_f32"], e["lo"], e["shard"],
                                  world, rank, e["grad"].dtype == torch.bfloat16,
                                  self.grad_scale)
            sq_total = sq if sq_total is None else sq_total + sq
        sq_total = self._runtime_sumsq(sq_total)
        dist.all_reduce(sq_total, op=dist.ReduceOp.SUM)
        norm = sq_total.sqrt()
        coef = (max_norm / (norm + 1e-6)).clamp(max=1.0) if max_norm > 0 else None
        self._runtime_step(optimizer, coef)
        # phase 2: AdamW on the slice; the new bf16 values go straight into every rank's buffer
        for e in flat:
            e["step"] += 1
            g = e["group"]
            b1, b2 = g["betas"]
            ext.adamw_slice_broadcast(
                symm.peer_pointers(e["param"]), e["grad_f32"], e["master"], e["exp_avg"],
                e["exp_avg_sq"], e["lo"], e["shard"], world, rank, float(g["lr"]), float(b1),
                float(b2), float(g["eps"]), float(g["weight_decay"]), int(e["step"]), coef,
                e["param"].dtype == torch.bfloat16)
        # peers' stores into this rank's parameters are complete, nobody still reads the
        # gradients that are zeroed next, and every rank's updated block shards are final
        # before a peer gathers them
        symm.barrier()
        rt = self.param_runtime
        if rt is not None:
            rt.publish(barrier=rt.pool is not symm)
        optimizer.zero_grad()
        return norm
