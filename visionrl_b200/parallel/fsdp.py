"""Fully sharded parameters, gradients and optimiser state (FSDP / ZeRO-3) for the transformer blocks.

What is kept per rank (``W`` = size of the shard group):

* ``1/W`` of every block weight — rows ``[r·N/W, (r+1)·N/W)`` of each ``[N, K]`` projection — in ONE
  flat bf16 buffer in symmetric memory (``module.weight`` becomes a view of it), plus the fp32
  master copy, the two Adam moments and an fp32 gradient accumulator of the same ``1/W`` size;
* a small ring of *gather buffers* (default: two blocks' worth) into which a block's full weights
  are materialised while it computes, and a ring of *gradient staging buffers* of the same size in
  symmetric memory.

How the collectives are fused with compute (``collectives="fused"``, bf16 on CUDA):

* **all-gather ⊕ GEMM** — a projection's forward is ONE kernel (``gemm_allgather``): 128 extra
  threads per CTA pull the peers' rows over NVLink into the gather buffer (own rows first) while the
  tcgen05 warps already multiply the tiles whose rows have arrived.  The gathered copy then serves
  the ``dX = dY·W`` product of the same block's backward (activation checkpointing re-runs the
  forward right before it).  Where no GEMM can hide a gather — the weights a backward pass
  without recomputation needs again, and projections applied to a handful of rows (the adaLN
  modulation) whose product is over before the rows arrive — the NEXT block's weights are
  fetched ahead of time by one table-driven peer-copy kernel on a side stream while the current
  block computes; a copy found neither gathered nor prefetched is fetched on the spot.
* **reduce-scatter ⊕ cast ⊕ scale ⊕ accumulate, overlapped with backward** — the ``dW`` GEMMs of a
  block write into that block's staging buffer.  When the backward pass moves on to the next
  block the finished bucket is published to the peers with a release flag and, on a side stream,
  a kernel sums the peers' slices of it over NVLink into this rank's fp32 gradient shard and then
  tells the peers their buffer may be reused.  Only the last bucket, the gradient-norm
  all-reduce and the sharded AdamW remain after the backward pass.  All waits on peers are
  bounded and report through :meth:`SymmetricPool.check`.

* **trainer → rollout weight broadcast** (``rollout_replica=True``) — rollouts read a full bf16
  copy of the block weights that every rank keeps in symmetric memory, so the thousands of
  no-grad forwards of a rollout cost no NVLink traffic at all.  After each optimiser step ONE
  kernel per rank stores that rank's freshly updated shards into every rank's replica over
  NVLink and then publishes the new policy version with a release flag; the next rollout waits
  (bounded) until every owner's version has arrived.  This replaces the reference's
  ``state_dict()`` → CPU → object store → ``load_state_dict`` round trip
  (``vrl/trainers/weight_sync.py:55-60``, ``vrl/distributed/ray/rollout/weight_sync.py:29-48``).

``collectives="nccl"`` performs the same steps with ``all_gather_into_tensor`` /
``reduce_scatter_tensor`` and is the measured baseline; on CPU (gloo) an all-reduce based variant
keeps the semantics for tests.  A ``replicate`` dimension (HSDP) shards inside groups of adjacent
ranks and all-reduces the fp32 gradient shards across the groups once per optimiser step.

The reference has this capability only as an unused wrapper around FSDP1
(``vrl/trainers/fsdp.py:49-103``: FULL_SHARD / HYBRID_SHARD, bf16 parameters and reduction,
BACKWARD_PRE prefetch).
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any, Iterable

import torch
import torch.distributed as dist
from torch import nn

from visionrl_b200.ops import linear as linear_ops


def _kernels_on(t: torch.Tensor) -> bool:
    from visionrl_b200.ops import _ext

    return t.is_cuda and t.dtype == torch.bfloat16 and _ext.kernels_enabled() and _ext.available()


@dataclass
class _Ring:
    """One slot of the gather / staging rings: which unit owns it and how often it changed hands."""

    owner: int = -1
    epoch: int = 0
    uses: int = 0            # staging only: sequence number of the bucket currently in the slot


class ShardedWeight:
    """Handle of one row-sharded ``[N, K]`` weight."""

    def __init__(self, rt: "ShardedParamRuntime", unit: int, index: int, n: int, k: int,
                 shard_off: int, unit_off: int, name: str) -> None:
        self.rt, self.unit, self.index, self.name = rt, unit, index, name
        self.n, self.k = n, k
        self.rows = n // rt.world
        self.numel_shard = self.rows * k
        self.shard_off = shard_off          # into the flat shard buffers
        self.unit_off = unit_off            # into a gather / staging ring slot
        self.param: nn.Parameter | None = None
        self._gather_epoch = -1
        self._gather_version = -1
        self._peers: torch.Tensor | None = None
        self.last_rows = -1                 # rows of the last activation multiplied with this weight

    # -- views -------------------------------------------------------------------------------
    @property
    def shard(self) -> torch.Tensor:
        return self.rt.shard_flat[self.shard_off:self.shard_off + self.numel_shard].view(self.rows, self.k)

    def _slot(self) -> int:
        return self.unit % self.rt.ring

    def _full_view(self) -> torch.Tensor:
        buf = self.rt.gather_ring[self._slot()]
        return buf[self.unit_off:self.unit_off + self.n * self.k].view(self.n, self.k)

    def _stage_view(self) -> torch.Tensor:
        buf = self.rt.stage_ring[self.unit % 2]
        return buf[self.unit_off:self.unit_off + self.n * self.k].view(self.n, self.k)

    def replica_view(self) -> torch.Tensor:
        off = self.rt.replica_off[self.name]
        return self.rt.replica_flat[off:off + self.n * self.k].view(self.n, self.k)

    def peer_pointers(self) -> torch.Tensor:
        if self._peers is None:
            self._peers = self.rt.pool.peer_pointers_at(self.rt.shard_flat, self.shard_off)
        return self._peers

    # -- gathering ---------------------------------------------------------------------------------
    def _claim(self, backward: bool = False) -> torch.Tensor:
        """The gather-ring view of this weight; taking a slot over from another unit evicts it."""
        rt = self.rt
        rt._settle()
        if rt._cursor != (self.unit, backward):
            rt.visit_unit(self.unit, backward)
        return self._full_view()

    def _mark_gathered(self) -> None:
        self._gather_epoch = self.rt.gather_slots[self._slot()].epoch
        self._gather_version = self.rt.version

    def is_gathered(self) -> bool:
        state = self.rt.gather_slots[self._slot()]
        return (state.owner == self.unit and self._gather_epoch == state.epoch
                and self._gather_version == self.rt.version)

    def gather(self, backward: bool = False) -> torch.Tensor:
        """The full ``[N, K]`` weight in its gather buffer (stand-alone all-gather when stale)."""
        rt = self.rt
        full = self._claim(backward)
        if self.is_gathered():
            return full
        rt.standalone_gathers += 1
        if rt.fused and full.is_cuda:
            from visionrl_b200.ops import _ext

            _ext.load().p2p_gather_rows(self.peer_pointers(), full, self.numel_shard, rt.world, rt.rank)
            rt.kernel_launches += 1
        elif rt.world == 1:
            full.copy_(self.shard)
        elif full.is_cuda:
            dist.all_gather_into_tensor(full.view(-1), self.shard.reshape(-1), group=rt.group)
        else:
            parts = [torch.empty_like(self.shard) for _ in range(rt.world)]
            dist.all_gather(parts, self.shard.contiguous(), group=rt.group)
            full.copy_(torch.cat(parts))
        rt.gathers += 1
        self._mark_gathered()
        return full

    def gather_copy(self) -> torch.Tensor:
        """A private copy of the full weight (checkpoints, state dicts)."""
        return self.gather().detach().clone()

    # -- forward ------------------------------------------------------------------------------------
    def gemm(self, x2: torch.Tensor, bias, act=None, gate=None, residual=None, rows_per_gate: int = 0,
             dual: bool = False):
        """``epilogue(x2 @ W.T + bias)`` with the gather fused into the product (no autograd)."""
        from visionrl_b200.ops import _ext

        rt = self.rt
        ext = _ext.load()
        self.last_rows = int(x2.shape[0])
        full = self._claim()
        act_id = linear_ops._ACTS[act]
        if self.is_gathered() or rt.world == 1 or not rt.fused:
            w = self.gather()
            if dual:
                return ext.gemm_bf16_dual(x2, w, bias, act_id)
            return [ext.gemm_bf16(x2, w, bias, gate, residual, act_id, int(rows_per_gate), False, False,
                                  False)]
        outs = ext.gemm_allgather(x2, self.peer_pointers(), full, rt.ready, bias, act_id, rt.rank,
                                  rt.world, gate, residual, int(rows_per_gate), dual)
        rt.kernel_launches += 1
        rt.gathers += 1
        rt.fused_gathers += 1
        self._mark_gathered()
        return outs

    # -- gradients ----------------------------------------------------------------------------------
    def stage_grad(self, gy2: torch.Tensor | None, x2: torch.Tensor | None,
                   dense: torch.Tensor | None = None) -> None:
        """``dW = gy2.T @ x2`` (or a ready ``dense`` gradient) into the staging buffer of this
        weight's bucket; a second contribution within one bucket accumulates."""
        rt = self.rt
        rt.open_bucket(self.unit)
        view = self._stage_view()
        first = self.index not in rt.bucket_written
        rt.bucket_written.add(self.index)
        if dense is not None:
            if first:
                view.copy_(dense)
            else:
                view.add_(dense)
            return
        if _kernels_on(gy2):
            from visionrl_b200.ops import _ext

            ext = _ext.load()
            if first:
                ext.gemm_bf16_out(gy2, x2, view, True, True)
            else:
                ext.gemm_bf16_acc(gy2, x2, view, True, True)
        else:
            dw = gy2.t().to(view.dtype) @ x2.to(view.dtype)
            if first:
                view.copy_(dw)
            else:
                view.add_(dw)

    def local_rows(self, dense: torch.Tensor) -> torch.Tensor:
        lo = self.rt.rank * self.rows
        return dense[lo:lo + self.rows]

    # -- module-facing call ---------------------------------------------------------------------------
    def linear(self, x, bias, act=None, gate=None, residual=None):
        """Differentiable ``linear`` through this weight (what :class:`Linear` calls)."""
        rt = self.rt
        needs_grad = torch.is_grad_enabled() and (
            x.requires_grad or self.param.requires_grad or (bias is not None and bias.requires_grad)
            or (gate is not None and gate.requires_grad)
            or (residual is not None and residual.requires_grad))
        if not needs_grad and rt.replica_ready():
            # rollout path: the rank's full replica, no gather
            return linear_ops.linear(x, self.replica_view(), bias, act=act, gate=gate, residual=residual)
        usable = linear_ops._use_kernel(x, self.shard)
        if not usable:
            # generic path (CPU, fp32, kernels off): gather, then the ordinary differentiable op
            if needs_grad:
                w = _GatheredWeightFn.apply(rt.anchor, self)
            else:
                w = self.gather()
            return linear_ops.linear(x, w, bias, act=act, gate=gate, residual=residual)
        if not needs_grad:
            x2 = x.reshape(-1, x.shape[-1])
            if not x2.is_contiguous():
                x2 = x2.contiguous()
            rows = x.shape[-2] if (gate is not None and x.dim() == 3) else (1 if gate is not None else 0)
            if gate is not None and gate.dim() != 2:
                gate = gate.reshape(-1, self.n)
            res2 = None if residual is None else residual.reshape(-1, self.n)
            y = self.gemm(x2, bias, act, gate, res2, rows)[0]
            return y.view(*x.shape[:-1], self.n)
        y = _ShardedLinearFn.apply(x, bias, rt.anchor, self)
        return linear_ops.linear_epilogue(y, act, gate, residual)


class _GatheredWeightFn(torch.autograd.Function):
    """Generic path: the full weight as a differentiable tensor whose gradient is staged."""

    @staticmethod
    def forward(ctx, anchor, handle: ShardedWeight):
        ctx.handle = handle
        # a private copy: autograd keeps it for the backward pass while the ring moves on
        return handle.gather().detach().clone()

    @staticmethod
    def backward(ctx, gw):
        handle = ctx.handle
        if linear_ops._ACCUMULATE_IN_PLACE[0] or handle.rt.always_stage:
            handle.stage_grad(None, None, dense=gw)
        return None, None


class _ShardedLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, anchor, handle: ShardedWeight):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = handle.gemm(x2, bias)[0]
        ctx.save_for_backward(x2)
        ctx.handle = handle
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], handle.n)

    @staticmethod
    def backward(ctx, gy):
        from visionrl_b200.ops import _ext

        (x2,) = ctx.saved_tensors
        handle = ctx.handle
        gy2 = gy.reshape(-1, gy.shape[-1])
        if not gy2.is_contiguous():
            gy2 = gy2.contiguous()
        gx = gb = None
        if ctx.needs_input_grad[0]:
            gx = linear_ops.gemm_nn(gy2, handle.gather(backward=True)).view(ctx.x_shape)
        if handle.param.requires_grad:
            handle.stage_grad(gy2, x2)
        if ctx.has_bias and ctx.needs_input_grad[1]:
            gb = _ext.load().colsum(gy2).to(gy2.dtype)
        return gx, gb, None, None


class _ShardedGeluMLPFn(torch.autograd.Function):
    """``fc2(gelu_tanh(fc1(x)))`` over two sharded weights; activation folded into the GEMMs."""

    @staticmethod
    def forward(ctx, x, b1, b2, anchor, h1: ShardedWeight, h2: ShardedWeight):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        a, h = h1.gemm(x2, b1, act="gelu_tanh", dual=True)
        y = h2.gemm(a, b2)[0]
        ctx.save_for_backward(x2, h, a)
        ctx.h1, ctx.h2 = h1, h2
        ctx.has_b1, ctx.has_b2 = b1 is not None, b2 is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], h2.n)

    @staticmethod
    def backward(ctx, gy):
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        x2, h, a = ctx.saved_tensors
        h1, h2 = ctx.h1, ctx.h2
        gy2 = gy.reshape(-1, gy.shape[-1])
        if not gy2.is_contiguous():
            gy2 = gy2.contiguous()
        # gh = (gy @ W2) * gelu'(h): W2 is [out, hidden] row-major, the MN-major B operand
        gh = ext.gemm_bf16(gy2, h2.gather(backward=True), None, None, h, 3, 0, False, True, False)
        gx = gb1 = gb2 = None
        if h2.param.requires_grad:
            h2.stage_grad(gy2, a)
        if ctx.has_b2 and ctx.needs_input_grad[2]:
            gb2 = ext.colsum(gy2).to(gy2.dtype)
        if h1.param.requires_grad:
            h1.stage_grad(gh, x2)
        if ctx.has_b1 and ctx.needs_input_grad[1]:
            gb1 = ext.colsum(gh).to(gh.dtype)
        if ctx.needs_input_grad[0]:
            gx = linear_ops.gemm_nn(gh, h1.gather(backward=True)).view(ctx.x_shape)
        return gx, gb1, gb2, None, None, None


def sharded_gelu_mlp(x, fc1, fc2):
    """GELU-tanh MLP over two sharded :class:`Linear` layers."""
    h1, h2 = fc1.sharded, fc2.sharded
    needs_grad = torch.is_grad_enabled()
    if (needs_grad and h1.unit == h2.unit and linear_ops._use_kernel(x, h1.shard)
            and h1.n % 8 == 0 and h2.n % 8 == 0):
        return _ShardedGeluMLPFn.apply(x, fc1.bias, fc2.bias, h1.rt.anchor, h1, h2)
    return fc2(fc1(x, act="gelu_tanh"))


# ------------------------------------------------------------------------------------------------
class ShardedParamRuntime:
    """Owns the shards, the rings and the bucket pipeline of one model."""

    def __init__(self, mesh: Any, device: torch.device, collectives: str = "fused",
                 dtype: torch.dtype = torch.bfloat16, ring: int = 2, grad_scale: float | None = None,
                 pool: Any | None = None, rollout_replica: bool = False) -> None:
        self.mesh = mesh
        self.device = torch.device(device)
        self.dtype = dtype
        self.group = getattr(mesh, "shard_group", None)
        self.replicate_group = getattr(mesh, "replicate_group", None)
        ready = dist.is_available() and dist.is_initialized()
        self.world = dist.get_world_size(self.group) if ready else 1
        self.rank = dist.get_rank(self.group) if ready else 0
        self.replicas = int(getattr(mesh, "replicate", 1) or 1)
        self.ring = max(1, int(ring))
        self.collectives = collectives
        self.fused = (collectives == "fused" and self.device.type == "cuda" and self.world > 1
                      and dtype == torch.bfloat16 and _kernels_on(torch.empty(0, device=self.device,
                                                                              dtype=dtype)))
        self.pool = pool
        if self.fused and self.pool is None:
            from visionrl_b200.parallel.symm import SymmetricPool

            self.pool = SymmetricPool(mesh, group=self.group)
        total_ranks = max(int(getattr(mesh, "world_size", self.world * self.replicas)), 1)
        # sum over every rank that holds a partial gradient, times this factor = the mean over the
        # data-parallel replicas (ranks of one sequence-parallel group hold partial sums)
        self.grad_scale = float(grad_scale) if grad_scale is not None else \
            float(getattr(mesh, "sp", 1)) / float(total_ranks)
        self.handles: list[ShardedWeight] = []
        self.unit_sizes: dict[int, int] = {}
        self.version = 0
        self.anchor = torch.zeros((), device=self.device, requires_grad=True)
        self.always_stage = False
        # counters (reported by benchmarks and tests)
        self.kernel_launches = 0
        self.gathers = 0
        self.fused_gathers = 0
        self.standalone_gathers = 0
        self.prefetches = 0
        # gather-ahead of the next unit's weights on a side stream
        self.prefetch = True
        self.small_rows = 1024              # a product of fewer rows cannot hide its own gather
        # which weights the forward pass fetches ahead (the backward pass always fetches the whole
        # unit): "small" = only products too short to hide their own gather; "deep" = those plus
        # weights with more columns than rows (few n-tiles, long k loop: the in-product gather has
        # nothing to overlap with); "all" = the whole unit, the in-product gather then only serves
        # the first unit of a pass
        self.forward_ahead = os.environ.get("VRL_GATHER_AHEAD", "deep")
        if self.forward_ahead not in ("small", "deep", "all"):
            raise ValueError("VRL_GATHER_AHEAD must be small, deep or all")
        self._cursor: tuple[int, bool] = (-1, False)
        self._last_unit = -1
        self._pending: dict[int, tuple[Any, list, int]] = {}
        self._fetch_tables: dict[tuple, tuple[torch.Tensor, int]] = {}
        self._prefetch_stream: Any = None
        self.buckets_reduced = 0
        # bucket pipeline
        self.current_bucket = -1
        self.bucket_written: set[int] = set()
        self._side: Any = None
        self._pending_event: Any = None
        self._built = False
        self._dirty = False
        self.step_count = 0
        # full-weight rollout replica (None = rollouts gather like training does)
        self.want_replica = bool(rollout_replica)
        self.replica_flat: torch.Tensor | None = None
        self.replica_off: dict[str, int] = {}
        self.replica_version = -1
        self.replica_waited = -1
        self.broadcasts = 0

    # -- construction ----------------------------------------------------------------------------------
    def shard_units(self, units: Iterable[nn.Module]) -> int:
        """Shard every eligible :class:`Linear` weight under the given modules (one unit = one
        gather / reduce bucket, normally a transformer block).  Returns the number of weights."""
        from visionrl_b200.models.nn.layers import Linear

        if self._built:
            raise RuntimeError("shard_units may be called once")
        plan: list[tuple[int, int, str, Any]] = []
        shard_off = 0
        for u, unit in enumerate(units):
            unit_off = 0
            index = 0
            for name, mod in unit.named_modules():
                if not isinstance(mod, Linear) or mod.sharded is not None:
                    continue
                w = mod.weight
                n, k = w.shape
                if (not w.requires_grad or w.dtype != self.dtype or n % self.world
                        or ((n // self.world) * k) % 8 or k % 8 or n % 8):
                    continue
                handle = ShardedWeight(self, u, index, n, k, shard_off, unit_off, f"{u}.{name}")
                plan.append((u, index, name, (mod, handle)))
                shard_off += handle.numel_shard
                unit_off += n * k
                index += 1
            self.unit_sizes[u] = unit_off
        if not plan:
            self._built = True
            return 0
        total = shard_off
        slot = max(self.unit_sizes.values())
        dev, dt = self.device, self.dtype
        if self.fused:
            self.shard_flat = self.pool.allocate(total, dt, dev, "param_shards")
            self.stage_ring = [self.pool.allocate(slot, dt, dev, f"grad_stage{i}") for i in range(2)]
            base = self.pool.reserve_slots(64)
            self.ready_slot = [base, base + 16]
            self.done_slot = [base + 32, base + 48]
        else:
            self.shard_flat = torch.empty(total, device=dev, dtype=dt)
            self.stage_ring = [torch.empty(slot, device=dev, dtype=dt) for _ in range(2)]
        units_count = len(self.unit_sizes)
        self.ring = min(self.ring, max(units_count, 1))
        self.gather_ring = [torch.empty(slot, device=dev, dtype=dt) for _ in range(self.ring)]
        self.gather_slots = [_Ring() for _ in range(self.ring)]
        self.stage_slots = [_Ring() for _ in range(2)]
        self.ready = torch.zeros(16, device=dev, dtype=torch.int32)
        for _u, _i, _name, (mod, handle) in plan:
            full = mod.weight.data
            lo = self.rank * handle.rows
            handle.shard.copy_(full[lo:lo + handle.rows])
            param = nn.Parameter(handle.shard, requires_grad=True)
            param._vrl_sharded = handle
            handle.param = param
            mod.weight = param
            mod.sharded = handle
            self.handles.append(handle)
        self.master = self.shard_flat.float()
        self.exp_avg = torch.zeros(total, device=dev, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(total, device=dev, dtype=torch.float32)
        self.grad_shard = torch.zeros(total, device=dev, dtype=torch.float32)
        # per-unit segment tables of the bucket reduction: (source offset of this rank's rows in
        # the staging slot, destination offset in the gradient shard, element count)
        self._tables: dict[int, tuple[torch.Tensor, int]] = {}
        for u in self.unit_sizes:
            rows = [(h.unit_off + self.rank * h.numel_shard, h.shard_off, h.numel_shard)
                    for h in self.handles if h.unit == u]
            if rows:
                self._tables[u] = (torch.tensor(rows, dtype=torch.int64, device=dev),
                                   max(r[2] for r in rows))
        if self.want_replica:
            self._build_replica()
        if self.fused:
            self._side = torch.cuda.Stream(device=dev)
            self._prefetch_stream = torch.cuda.Stream(device=dev)
            torch.cuda.synchronize(dev)
            self.pool.barrier()          # every rank's shards are in place before the first gather
        if self.want_replica:
            self.publish_replica()
        self._built = True
        return len(self.handles)

    # -- rollout replica (trainer -> rollout weight broadcast) -----------------------------------------
    def _build_replica(self) -> None:
        dev, dt = self.device, self.dtype
        off = 0
        for h in self.handles:
            self.replica_off[h.name] = off
            off += h.n * h.k
        if self.fused:
            self.replica_flat = self.pool.allocate(off, dt, dev, "rollout_replica")
            self.version_slot = self.pool.reserve_slots(16)
            rows = [(h.shard_off, self.replica_off[h.name] + self.rank * h.numel_shard, h.numel_shard)
                    for h in self.handles]
            self._replica_table = (torch.tensor(rows, dtype=torch.int64, device=dev),
                                   max(r[2] for r in rows))
        else:
            self.replica_flat = torch.empty(off, device=dev, dtype=dt)

    def publish_replica(self) -> None:
        """Bring every rank's rollout replica to the current parameter version."""
        if self.replica_flat is None:
            return
        version = self.version + 1          # flag values start at 1
        if self.fused:
            from visionrl_b200.ops import _ext

            table, longest = self._replica_table
            _ext.load().p2p_broadcast_table(self.shard_flat, self.pool.peer_pointers(self.replica_flat),
                                            table, self.world, self.rank, longest)
            self.pool.signal(self.version_slot + self.rank, version)
            self.kernel_launches += 2
        else:
            for h in self.handles:
                dst = h.replica_view()
                if self.world == 1:
                    dst.copy_(h.shard)
                elif dst.is_cuda:
                    dist.all_gather_into_tensor(dst.view(-1), h.shard.reshape(-1), group=self.group)
                else:
                    parts = [torch.empty_like(h.shard) for _ in range(self.world)]
                    dist.all_gather(parts, h.shard.contiguous(), group=self.group)
                    dst.copy_(torch.cat(parts))
        self.replica_version = self.version
        self.broadcasts += 1

    def verify_replicas(self) -> None:
        """Cross-rank consistency check of the rollout replicas: every rank sums the bit patterns
        of its replica and the sums are compared over the process group.  Ranks whose fused
        broadcast lost or tore a write would roll out with different weights than their peers
        and silently bias the gradient; here that is an error naming the ranks that disagree."""
        if self.replica_flat is None or not (dist.is_available() and dist.is_initialized()) \
                or dist.get_world_size() == 1 or not self.replica_ready():
            return
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()
        words = self.replica_flat.view(torch.int16).to(torch.int64)
        mine = torch.stack([words.sum(), (words * (torch.arange(words.numel(), device=words.device) % 8191 + 1)).sum()])
        # every rank of the job holds the same full replica, whatever shard or replica group it is in
        seen = [torch.empty_like(mine) for _ in range(dist.get_world_size())]
        dist.all_gather(seen, mine)
        bad = [r for r, other in enumerate(seen) if not torch.equal(other.cpu(), seen[0].cpu())]
        if bad:
            raise RuntimeError(f"rollout replicas differ across ranks: ranks {bad} disagree with rank 0 "
                               f"at parameter version {self.version}")

    def replica_ready(self) -> bool:
        """True when rollouts may read the replica; the first use after a publish enqueues the
        bounded wait for every owner's version flag."""
        if self.replica_flat is None or self._dirty or self.replica_version != self.version:
            return False
        if self.fused and self.replica_waited != self.version:
            self.pool.wait(self.version_slot, self.world, self.version + 1)
            self.kernel_launches += 1
            self.replica_waited = self.version
        return True

    @property
    def active(self) -> bool:
        return bool(self.handles)

    # -- unit traversal and gather-ahead ---------------------------------------------------------------
    def visit_unit(self, unit: int, backward: bool) -> None:
        """Called when the computation moves to another unit (or turns from forward to backward
        inside one): take the unit's ring slot over, adopt what was fetched ahead for it, and
        start fetching the unit that comes next in the direction of travel."""
        step = unit - self._last_unit if self._last_unit >= 0 and unit != self._last_unit else 0
        direction = (1 if step > 0 else -1) if step else (-1 if backward else 1)
        self._cursor = (unit, backward)
        self._last_unit = unit
        slot = self.gather_slots[unit % self.ring]
        pending = self._pending.pop(unit, None)
        if slot.owner != unit:
            slot.owner = unit
            slot.epoch += 1
        if pending is not None:
            event, handles, version = pending
            if version == self.version:
                torch.cuda.current_stream(self.device).wait_event(event)
                for h in handles:
                    h._mark_gathered()
        if self.fused and self.prefetch and self.ring >= 2:
            self._fetch_ahead(unit + direction, whole_unit=backward)

    def _fetch_ahead(self, unit: int, whole_unit: bool) -> None:
        if unit < 0 or unit not in self.unit_sizes or unit in self._pending:
            return
        everything = whole_unit or self.forward_ahead == "all"
        deep = self.forward_ahead == "deep"
        wanted = [h for h in self.handles if h.unit == unit and not h.is_gathered()
                  and (everything or 0 <= h.last_rows < self.small_rows or (deep and h.k > h.n))]
        if not wanted:
            return
        from visionrl_b200.ops import _ext

        slot_index = unit % self.ring
        slot = self.gather_slots[slot_index]
        # the slot changes hands now: whatever its previous owner had gathered there is void
        if slot.owner != unit:
            slot.owner = -1
            slot.epoch += 1
        key = (unit, tuple(h.index for h in wanted))
        cached = self._fetch_tables.get(key)
        if cached is None:
            rows = [(h.shard_off, h.unit_off, h.numel_shard) for h in wanted]
            cached = (torch.tensor(rows, dtype=torch.int64, device=self.device), max(r[2] for r in rows))
            self._fetch_tables[key] = cached
        table, longest = cached
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)                       # the slot's previous readers are all enqueued before this
        with torch.cuda.stream(self._prefetch_stream):
            self._prefetch_stream.wait_event(ready)
            _ext.load().p2p_gather_table(self.pool.peer_pointers(self.shard_flat), self.gather_ring[slot_index],
                                         table, self.world, self.rank, longest)
            done = torch.cuda.Event()
            done.record(self._prefetch_stream)
        self._pending[unit] = (done, wanted, self.version)
        self.prefetches += 1
        self.gathers += len(wanted)
        self.kernel_launches += 1

    # -- bucket pipeline ---------------------------------------------------------------------------------
    def open_bucket(self, unit: int) -> None:
        if self.current_bucket == unit:
            return
        self.close_bucket()
        self.current_bucket = unit
        self.bucket_written = set()
        state = self.stage_slots[unit % 2]
        if self.fused and state.uses > 0:
            # every peer has finished reading the bucket that used this staging slot before
            self.pool.wait(self.done_slot[unit % 2], self.world, state.uses)
            self.kernel_launches += 1
        state.uses += 1
        state.owner = unit

    def close_bucket(self) -> None:
        """Publish the open bucket and start its reduction (side stream when fused)."""
        unit = self.current_bucket
        if unit < 0:
            return
        self.current_bucket = -1
        table = self._tables.get(unit)
        if table is None:
            return
        missing = [h for h in self.handles if h.unit == unit and h.param.requires_grad
                   and h.index not in self.bucket_written]
        for h in missing:               # a weight the backward pass never reached contributes zero
            h._stage_view().zero_()
        slot = unit % 2
        seq = self.stage_slots[slot].uses
        if self.fused:
            from visionrl_b200.ops import _ext

            ext = _ext.load()
            pool = self.pool
            pool.signal(self.ready_slot[slot] + self.rank, seq)
            main = torch.cuda.current_stream(self.device)
            event = torch.cuda.Event()
            event.record(main)
            with torch.cuda.stream(self._side):
                self._side.wait_event(event)
                pool.wait(self.ready_slot[slot], self.world, seq)
                ext.bucket_reduce_acc(pool.peer_pointers(self.stage_ring[slot]), table[0], self.grad_shard,
                                      self.grad_scale, self.world, self.rank, table[1])
                pool.signal(self.done_slot[slot] + self.rank, seq)
                done = torch.cuda.Event()
                done.record(self._side)
            self._pending_event = done
            self.kernel_launches += 4
        else:
            stage = self.stage_ring[slot]
            for h in (h for h in self.handles if h.unit == unit):
                view = stage[h.unit_off:h.unit_off + h.n * h.k]
                dst = self.grad_shard[h.shard_off:h.shard_off + h.numel_shard]
                if self.world == 1:
                    dst.add_(view.float(), alpha=self.grad_scale)
                elif view.is_cuda:
                    part = torch.empty(h.numel_shard, device=view.device, dtype=view.dtype)
                    dist.reduce_scatter_tensor(part, view, op=dist.ReduceOp.SUM, group=self.group)
                    dst.add_(part.float(), alpha=self.grad_scale)
                else:
                    dist.all_reduce(view, op=dist.ReduceOp.SUM, group=self.group)
                    lo = self.rank * h.numel_shard
                    dst.add_(view[lo:lo + h.numel_shard].float(), alpha=self.grad_scale)
        self.buckets_reduced += 1

    def finish_grads(self) -> None:
        """All buckets of this step are reduced into ``grad_shard`` (current stream ordered after)."""
        self.close_bucket()
        if self.fused and self._pending_event is not None:
            torch.cuda.current_stream(self.device).wait_event(self._pending_event)
            self._pending_event = None
        if self.replicas > 1 and self.replicate_group is not None and self.active:
            dist.all_reduce(self.grad_shard, op=dist.ReduceOp.SUM, group=self.replicate_group)

    # -- optimiser ------------------------------------------------------------------------------------------
    def grad_sumsq(self) -> torch.Tensor:
        g = self.grad_shard
        if g.is_cuda and _kernels_on(self.shard_flat):
            from visionrl_b200.ops import _ext

            return _ext.load().sum_squares(g)
        return g.float().pow(2).sum()

    @torch.no_grad()
    def adamw_step(self, group: dict, clip_coef: torch.Tensor | None) -> None:
        """AdamW on this rank's shards (fp32 master + moments → bf16 shard), then zero the gradient
        accumulator.  Peers read the new shards only after the caller's barrier."""
        from visionrl_b200.ops import optim as optim_ops

        if not self.active:
            return
        self._settle()
        self._drain_fetches()
        self.step_count += 1
        b1, b2 = group["betas"]
        kw = dict(lr=float(group["lr"]), beta1=float(b1), beta2=float(b2), eps=float(group["eps"]),
                  weight_decay=float(group["weight_decay"]), step=int(self.step_count))
        if self.shard_flat.is_cuda and _kernels_on(self.shard_flat):
            from visionrl_b200.ops import _ext

            _ext.load().adamw_flat(self.shard_flat, self.grad_shard, self.master, self.exp_avg,
                                   self.exp_avg_sq, kw["lr"], kw["beta1"], kw["beta2"], kw["eps"],
                                   kw["weight_decay"], kw["step"], clip_coef)
        else:
            master = self.master if self.shard_flat.dtype != torch.float32 else self.shard_flat
            optim_ops.adamw_flat_reference(self.shard_flat, self.grad_shard, master, self.exp_avg,
                                           self.exp_avg_sq, clip_coef=clip_coef, **kw)
        self.grad_shard.zero_()
        self.version += 1

    def publish(self, barrier: bool = True) -> None:
        """Order the peers' next gathers after this rank's shard update (``barrier=False`` when
        the caller has just run one on the same pool), and push the new shards into the rollout
        replicas."""
        if self.fused and barrier:
            self.pool.barrier()
        self.publish_replica()

    def _drain_fetches(self) -> None:
        """No gather-ahead of the old parameter version may still be writing a ring slot."""
        if self._prefetch_stream is not None and self._pending:
            torch.cuda.current_stream(self.device).wait_stream(self._prefetch_stream)
        self._pending.clear()
        self._cursor = (-1, False)

    def invalidate(self) -> None:
        """Shards were changed behind the runtime's back (state-dict load, EMA swap): refresh the
        fp32 master copy and drop every gathered copy."""
        self._dirty = False
        self._drain_fetches()
        if self.active:
            self.master.copy_(self.shard_flat)
        self.version += 1
        self.publish()

    def mark_dirty(self) -> None:
        """Like :meth:`invalidate`, applied lazily before the next gather or optimiser step."""
        self._dirty = True

    def _settle(self) -> None:
        if self._dirty:
            self.invalidate()

    def check(self, what: str = "sharded step") -> None:
        if self.fused:
            self.pool.check(what)

    # -- state ------------------------------------------------------------------------------------------------
    def gather_state(self, handle: ShardedWeight, which: str) -> torch.Tensor:
        """Full ``[N, K]`` fp32 optimiser state of one weight (collective on every rank)."""
        src = getattr(self, which)[handle.shard_off:handle.shard_off + handle.numel_shard]
        if self.world == 1:
            return src.view(handle.n, handle.k).clone()
        parts = [torch.empty_like(src) for _ in range(self.world)]
        dist.all_gather(parts, src.contiguous(), group=self.group)
        return torch.cat(parts).view(handle.n, handle.k)

    def load_state(self, handle: ShardedWeight, which: str, full: torch.Tensor) -> None:
        dst = getattr(self, which)[handle.shard_off:handle.shard_off + handle.numel_shard]
        dst.copy_(handle.local_rows(full.reshape(handle.n, handle.k)).reshape(-1))

    def memory_report(self) -> dict[str, int]:
        if not self.active:
            return {}
        e = self.shard_flat.element_size()
        full = sum(h.n * h.k for h in self.handles)
        return {
            "sharded_weights": len(self.handles),
            "full_param_bytes": full * e,
            "param_shard_bytes": self.shard_flat.numel() * e,
            "grad_shard_bytes": self.grad_shard.numel() * 4,
            "optimizer_shard_bytes": 3 * self.master.numel() * 4,
            "gather_ring_bytes": sum(b.numel() for b in self.gather_ring) * e,
            "grad_staging_bytes": sum(b.numel() for b in self.stage_ring) * e,
            "rollout_replica_bytes": 0 if self.replica_flat is None else self.replica_flat.numel() * e,
        }


def find_units(model: nn.Module) -> list[nn.Module]:
    """The transformer blocks of a policy / network: the first ``nn.ModuleList`` named ``blocks``
    or ``layers`` found under it."""
    for root in (model, getattr(model, "transformer", None)):
        if root is None:
            continue
        for name, mod in root.named_modules():
            if isinstance(mod, nn.ModuleList) and name.split(".")[-1] in ("blocks", "layers") and len(mod):
                return list(mod)
    return []


def shard_model(model: nn.Module, mesh: Any, device: torch.device, collectives: str = "fused",
                ring: int = 2, rollout_replica: bool = False,
                units: list[nn.Module] | None = None) -> ShardedParamRuntime | None:
    """Shard the block weights of ``model`` in place; ``None`` when nothing qualifies.  ``units``
    names the blocks explicitly (default: :func:`find_units`)."""
    units = find_units(model) if units is None else list(units)
    if not units:
        return None
    first = next((p for p in units[0].parameters() if p.dim() == 2), None)
    if first is None:
        return None
    rt = ShardedParamRuntime(mesh, device, collectives=collectives, dtype=first.dtype, ring=ring,
                             rollout_replica=rollout_replica)
    if rt.world <= 1:
        return None
    if rt.shard_units(units) == 0:
        return None
    return rt


__all__ = ["ShardedParamRuntime", "ShardedWeight", "find_units", "shard_model", "sharded_gelu_mlp"]
