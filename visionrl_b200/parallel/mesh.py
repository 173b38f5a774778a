"""Process mesh ``(dp, sp)`` × ``(replicate, shard)`` over ``torch.distributed``.

Ranks are laid out ``rank = dp_rank * sp + sp_rank`` so a sequence-parallel group is
a run of adjacent ranks (adjacent GPUs).  Independently of that, parameter sharding
(``fsdp``) uses a second factorisation of the same ranks, ``rank = replica * shard +
shard_rank``: parameters, gradients and optimiser state are sharded over a *shard group* of
``world / replicate`` adjacent ranks and replicated across the ``replicate`` groups
(hybrid sharding; ``replicate = 1`` shards over the whole world).  The reference describes
the same ``(replicate, shard)`` device mesh for its FSDP wrapper
(``vrl/trainers/fsdp.py:59-67``).  One process owns one GPU; with no initialised process
group everything degenerates to a single rank.
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist


def dist_ready() -> bool:
    return dist.is_available() and dist.is_initialized()


def init_distributed(backend: str | None = None, timeout_s: float = 1800.0) -> tuple[int, int, int]:
    """Initialise from the ``RANK`` / ``WORLD_SIZE`` / ``MASTER_*`` environment (torchrun).

    Returns ``(rank, world_size, local_rank)``.  Without those variables nothing is
    initialised and ``(0, 1, 0)`` is returned.
    """
    if dist_ready():
        return dist.get_rank(), dist.get_world_size(), int(os.environ.get("LOCAL_RANK", 0))
    if "RANK" not in os.environ or "WORLD_SIZE" not in os.environ:
        return 0, 1, 0
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    use_cuda = torch.cuda.is_available()
    if backend is None:
        backend = "nccl" if use_cuda else "gloo"
    kwargs: dict[str, Any] = {}
    if use_cuda:
        torch.cuda.set_device(local)
        if backend == "nccl":
            kwargs["device_id"] = torch.device("cuda", local)
    factory = _STORE_FACTORY[0]
    relaunches = int(os.environ.get("TORCHELASTIC_RESTART_COUNT") or 0)
    if factory is None and relaunches > 0 and agent_store_in_use():
        # workers started again by the launcher share the launcher's store with the workers they
        # replace, whose connection addresses are still in it
        def factory(rank: int, world: int) -> Any:
            return fresh_prefix_store(rank, world, f"vrl/relaunch/{relaunches}")
    if factory is None:
        dist.init_process_group(backend=backend, init_method="env://", rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    else:
        # a job that re-forms its group (an in-place restart) brings its own key-value store, so
        # that the keys of the group it left cannot be mistaken for the new group's
        dist.init_process_group(backend=backend, store=factory(rank, world), rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
    return rank, world, local


# optional `(rank, world) -> store` used instead of the env:// rendezvous (see scripts/elastic.py)
_STORE_FACTORY: list = [None]


def agent_store_in_use() -> bool:
    """True under ``torchrun``: the launcher's agent hosts the store, all ranks are clients."""
    return os.environ.get("TORCHELASTIC_USE_AGENT_STORE", "").lower() == "true"


def fresh_prefix_store(rank: int, world: int, prefix: str, rendezvous_timeout_s: float = 600.0) -> Any:
    """A key-value store for a group that is formed a second time in the life of a job: the TCP
    store at ``MASTER_ADDR:MASTER_PORT`` (hosted by rank 0 unless the launcher's agent hosts it)
    seen through ``prefix``, returned once all ``world`` ranks have signed in.  Forming a group
    waits for the other ranks' addresses only as long as a collective would, and a rank that
    survived a failure can be that late by itself; the sign-in waits ``rendezvous_timeout_s``."""
    import time

    store = dist.TCPStore(
        os.environ.get("MASTER_ADDR", "127.0.0.1"), int(os.environ["MASTER_PORT"]), world,
        is_master=(rank == 0 and not agent_store_in_use()),
        timeout=datetime.timedelta(seconds=rendezvous_timeout_s), wait_for_workers=False)
    store = dist.PrefixStore(prefix, store)
    store.add("arrived", 1)
    deadline = time.monotonic() + rendezvous_timeout_s
    while int(store.add("arrived", 0)) < world:
        if time.monotonic() > deadline:
            raise TimeoutError(f"{prefix}: only {int(store.add('arrived', 0))} of {world} ranks reached "
                               f"the rendezvous within {rendezvous_timeout_s:.0f} s")
        time.sleep(0.05)
    return store


def set_rendezvous_store_factory(factory) -> None:
    _STORE_FACTORY[0] = factory


# mesh of the running job: components that are constructed far from the recipe (the rollout
# runtime) pick it up here instead of rebuilding a default (sp = 1) mesh
_CURRENT: list = [None]


@dataclass
class ProcessMesh:
    rank: int = 0
    world_size: int = 1
    dp: int = 1
    sp: int = 1
    fsdp: bool = True
    sp_group: Any = None
    dp_group: Any = None
    replicate: int = 1
    shard_group: Any = None          # None = the whole world
    replicate_group: Any = None

    @classmethod
    def build(cls, sp: int = 1, dp: int = -1, fsdp: bool = True, replicate: int = 1) -> "ProcessMesh":
        if not dist_ready():
            if sp not in (1, None):
                raise ValueError(f"sp={sp} needs an initialised process group")
            if replicate not in (1, None):
                raise ValueError(f"replicate={replicate} needs an initialised process group")
            return cls(fsdp=fsdp)
        rank, world = dist.get_rank(), dist.get_world_size()
        sp = int(sp or 1)
        replicate = int(replicate or 1)
        if replicate < 1 or world % replicate != 0:
            raise ValueError(f"world_size={world} is not divisible by replicate={replicate}")
        if world % sp != 0:
            raise ValueError(f"world_size={world} is not divisible by sp={sp}")
        if dp in (-1, None):
            dp = world // sp
        if dp * sp != world:
            raise ValueError(f"dp*sp = {dp}*{sp} != world_size {world}")
        sp_group = dp_group = None
        if sp > 1:
            for d in range(dp):
                ranks = list(range(d * sp, (d + 1) * sp))
                g = dist.new_group(ranks)
                if rank in ranks:
                    sp_group = g
            for s in range(sp):
                ranks = list(range(s, world, sp))
                g = dist.new_group(ranks)
                if rank in ranks:
                    dp_group = g
        shard_group = replicate_group = None
        if replicate > 1:
            shard = world // replicate
            for rep in range(replicate):
                ranks = list(range(rep * shard, (rep + 1) * shard))
                g = dist.new_group(ranks)
                if rank in ranks:
                    shard_group = g
            for s in range(shard):
                ranks = list(range(s, world, shard))
                g = dist.new_group(ranks)
                if rank in ranks:
                    replicate_group = g
        mesh = cls(rank=rank, world_size=world, dp=dp, sp=sp, fsdp=fsdp, sp_group=sp_group,
                   dp_group=dp_group, replicate=replicate, shard_group=shard_group,
                   replicate_group=replicate_group)
        _CURRENT[0] = mesh
        return mesh

    @classmethod
    def current(cls) -> "ProcessMesh | None":
        """The mesh the running job was set up with (``None`` before any :meth:`build`)."""
        return _CURRENT[0]

    @property
    def dp_rank(self) -> int:
        return self.rank // self.sp

    @property
    def sp_rank(self) -> int:
        return self.rank % self.sp

    @property
    def shard_size(self) -> int:
        return self.world_size // max(self.replicate, 1)

    @property
    def shard_rank(self) -> int:
        return self.rank % self.shard_size

    @property
    def replica_rank(self) -> int:
        return self.rank // self.shard_size

    @property
    def is_main(self) -> bool:
        return self.rank == 0

    def barrier(self) -> None:
        if dist_ready():
            dist.barrier()

    def all_gather_1d(self, t: torch.Tensor, group: Any = None) -> torch.Tensor:
        """Concatenate equally sized 1-D tensors from every rank of ``group``."""
        if not dist_ready():
            return t
        n = dist.get_world_size(group)
        out = torch.empty(n * t.numel(), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out, t.contiguous(), group=group)
        return out

    def all_gather_varlen(self, t: torch.Tensor, group: Any = None) -> list[torch.Tensor]:
        """Gather 1-D tensors whose lengths differ between ranks."""
        if not dist_ready():
            return [t]
        n = dist.get_world_size(group)
        size = torch.tensor([t.numel()], dtype=torch.long, device=t.device)
        sizes = [torch.zeros_like(size) for _ in range(n)]
        dist.all_gather(sizes, size, group=group)
        lens = [int(s.item()) for s in sizes]
        pad = max(lens) if lens else 0
        buf = torch.zeros(pad, dtype=t.dtype, device=t.device)
        buf[: t.numel()] = t
        outs = [torch.zeros_like(buf) for _ in range(n)]
        dist.all_gather(outs, buf, group=group)
        return [o[:k] for o, k in zip(outs, lens)]
