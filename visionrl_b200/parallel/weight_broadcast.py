"""Trainer → rollout weight synchronisation on the device (F4).

When rollout replicas keep their own parameter copy (not the trainer's flat buffer), the owner
of every updated slice stores it into each replica's symmetric parameter buffer with one
kernel and then publishes a monotonically increasing ``policy_version`` with a
release-ordered store; a replica checks (bounded wait) that the version it is asked to sample
with has arrived before its next rollout.  The NCCL variant (``broadcast`` per tensor) is the
measured baseline.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from visionrl_b200.parallel.symm import SymmetricPool

VERSION_SLOT = 16      # slots [16, 32): one published policy version per owner rank


class DeviceWeightBroadcaster:
    def __init__(self, pool: SymmetricPool, numel: int, dtype: torch.dtype, device: Any) -> None:
        self.pool = pool
        self.replica = pool.allocate(numel, dtype, device, "rollout_params").zero_()
        # a peer's first publish must not race with this rank's zero-fill
        torch.cuda.synchronize(device)
        pool.barrier()
        self.version = 0
        self.launches = 0

    def publish(self, source: torch.Tensor, offset_elems: int = 0, version: int | None = None,
                include_self: bool = True) -> int:
        """Store ``source`` into every replica at ``offset_elems`` and publish the version."""
        from visionrl_b200.ops import _ext

        self.version = int(version) if version is not None else self.version + 1
        _ext.load().p2p_broadcast_versioned(
            source.contiguous(), self.pool.peer_pointers(self.replica),
            offset_elems * source.element_size(), self.pool.peer_pointers(self.pool.flags),
            VERSION_SLOT + self.pool.rank, self.pool.world, self.pool.rank, self.version,
            include_self)
        self.launches += 2
        return self.version

    def wait_version(self, owner_rank: int, version: int, timeout_s: float = 1.0) -> None:
        """Bounded device-side wait until ``owner_rank`` has published ``version``."""
        from visionrl_b200.ops import _ext

        status = _ext.load().wait_flag(self.pool.flags, VERSION_SLOT + owner_rank, int(version),
                                       float(timeout_s))
        self.pool.check_wait(status, f"weight version {version} from rank {owner_rank}")


def nccl_broadcast_baseline(tensors: list[torch.Tensor], src: int = 0) -> None:
    for t in tensors:
        dist.broadcast(t, src=src)
